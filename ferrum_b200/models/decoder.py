"""A decoder put together from parts: embedding, blocks, a run order, final norm, head.

The run order is data: `schedule` is a list of `Run(block, cache_of)`.  `block` indexes
`blocks` (naming a block twice runs it twice, each run with cache planes of its own);
`cache_of = j` lets run k read the cache that run j wrote instead of writing one.  The model
never looks at which architecture it is; `weight_specs` and `cache_needs` are derived from
the parts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import os

import torch

from ..parts.base import Part

# FERRUM_NVTX=1: every step and every run of a block is an NVTX range (for a system profiler's timeline)
NVTX = os.environ.get("FERRUM_NVTX", "0") == "1"


@dataclass(frozen=True)
class Run:
    block: int
    cache_of: Optional[int] = None      # index of an earlier run whose cache this run reads


class DecoderModel(Part):
    graph_safe = True

    def __init__(self, config, dtype, embedding, position, blocks, final_norm, head, schedule=None,
                 block_prefix="blk.{}.", names=("token_embd.", "output_norm.", "output.")):
        self.config, self.dtype = config, dtype
        self.embedding, self.position, self.blocks = embedding, position, list(blocks)
        self.final_norm, self.head = final_norm, head
        self.schedule: List[Run] = list(schedule) if schedule is not None else [Run(i) for i in range(len(self.blocks))]
        self._block_prefix, self._names = block_prefix, names
        for k, run in enumerate(self.schedule):
            if not 0 <= run.block < len(self.blocks):
                raise ValueError(f"schedule entry {k} names block {run.block}, which does not exist")
            if run.cache_of is not None and not (0 <= run.cache_of < k and self.schedule[run.cache_of].cache_of is None):
                raise ValueError(f"schedule entry {k} must read the cache of an earlier run that writes one")

    # ------------------------------------------------------------------ structure
    def children(self):
        out = [(self._names[0], self.embedding)]
        if self.position is not None:
            out.append(("position.", self.position))
        out += [(self._block_prefix.format(i), b) for i, b in enumerate(self.blocks)]
        out += [(self._names[1], self.final_norm), (self._names[2], self.head)]
        return out

    def weight_specs(self):
        """Canonical tensor name -> (ParamSpec, owner part, local name)."""
        return {name: (spec, part, local) for name, spec, part, local in self.named_specs()}

    def cache_needs(self):
        """One CacheNeed per schedule entry (what that run's mixer keeps per request)."""
        return [self.blocks[r.block].mixer.cache_need() for r in self.schedule]

    @property
    def n_vocab(self):
        return self.head.n_vocab

    # ------------------------------------------------------------------ the forward pass
    def plan(self, ctx, cache):
        """Lets every run's mixer build this step's host-made work lists (see `Mixer.plan`)."""
        for k, run in enumerate(self.schedule):
            self.blocks[run.block].mixer.plan(ctx, cache.layer_cache(k))

    def forward(self, ctx, cache):
        """Run the batch described by ctx; returns float32 logits [want_capacity, V] whose
        first ctx.n_want rows are valid, or None when nothing is wanted."""
        h = self.embedding.forward(ctx)
        if self.position is not None:
            self.position.on_embedding(h, ctx)
        for k, run in enumerate(self.schedule):
            if NVTX:
                torch.cuda.nvtx.range_push(f"run {k} block {run.block}")
            self.blocks[run.block].forward(h, ctx, cache.layer_cache(k))
            if NVTX:
                torch.cuda.nvtx.range_pop()
        if ctx.n_want == 0:
            ctx.pending_residual = None      # nobody reads the residual stream any more
            return None
        x = self.final_norm.forward(h, ctx, rows=ctx.want_rows, n_rows=ctx.n_want, tag="final_norm")
        ctx.flush_residual()
        return self.head.forward(x, ctx, ctx.n_want)
