"""Token embedding and output head.

Embedding: row t of the table, upcast to the float32 residual stream, no scaling
(crates/model/src/weights.rs:29-51).  Output head: logits = W_out x on the wanted rows only;
W_out is its own matrix or, when the file has none, the embedding table
(crates/model/src/llama.rs:28-40,103-111).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import ParamSpec, Part
from .linear import STORE_F32, linear


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, n_vocab, width):
        self.n_vocab, self.width = n_vocab, width
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.n_vocab, self.width))}

    def forward(self, ctx):
        h = ctx.buf("hidden", (ctx.token_capacity, self.width), torch.float32)
        ops.embedding(self.w_weight, ctx.token_ids, h, ctx.err)
        return h


class OutputHead(Part):
    graph_safe = True

    def __init__(self, n_vocab, width, tied_to: TokenEmbedding = None, tied="auto"):
        """tied: True (no matrix of its own), False (must have one), "auto" (use the file's
        matrix when present, else the embedding: the reference's rule)."""
        self.n_vocab, self.width, self.tied_to, self.tied = n_vocab, width, tied_to, tied
        self.w_weight = None

    def param_specs(self):
        if self.tied is True:
            return {}
        return {"weight": ParamSpec((self.n_vocab, self.width), optional=self.tied == "auto")}

    def finalize(self):
        if self.w_weight is None:
            if self.tied_to is None:
                raise ValueError("output head has neither a matrix nor an embedding to share")
            self.w_weight = self.tied_to.w_weight

    def forward(self, x, ctx, n_rows):
        logits = ctx.buf("logits", (ctx.want_capacity, self.n_vocab), torch.float32)
        linear(x, self.w_weight, logits, STORE_F32, ctx, M=n_rows)
        return logits
