"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), added to the residual stream.

crates/model/src/llama.rs:261-285; silu(g) = g / (1 + exp(-g)) (crates/kernels/src/math.rs:8-10).
Gate and up are stored as one matrix [2F, E] so that one kernel reads x once; on the
tensor-core path that kernel also applies the activation (two accumulators, one epilogue).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import FeedForward, ParamSpec
from .linear import RESIDUAL, STORE, linear, linear_swiglu


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, width, hidden, dtype):
        self.width, self.hidden, self.dtype = width, hidden, dtype
        self.w_gate_weight = self.w_up_weight = self.w_down_weight = None
        self.w_gate_up = None

    def param_specs(self):
        return {"gate.weight": ParamSpec((self.hidden, self.width)),
                "up.weight": ParamSpec((self.hidden, self.width)),
                "down.weight": ParamSpec((self.width, self.hidden))}

    def finalize(self):
        self.w_gate_up = torch.cat([self.w_gate_weight, self.w_up_weight], dim=0).contiguous()
        self.w_gate_weight = self.w_up_weight = None

    def forward(self, x, ctx, residual):
        F, T = self.hidden, ctx.n_tokens
        act = ctx.buf("ffn_act", (ctx.token_capacity, F), self.dtype)
        if ops.gemm_tc_supported(x, self.w_gate_up):
            linear_swiglu(x, self.w_gate_up, act, F, ctx, M=T)
        else:
            gu = ctx.buf("ffn_gate_up", (ctx.token_capacity, 2 * F), self.dtype)
            linear(x, self.w_gate_up, gu, STORE, ctx, M=T)
            ops.swiglu(gu, act, T, F)
        linear(act, self.w_down_weight, residual, RESIDUAL, ctx, M=T)
