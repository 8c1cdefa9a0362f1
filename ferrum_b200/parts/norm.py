"""RMSNorm: x * rsqrt(mean(x^2) + eps) * w (crates/kernels/src/scalar.rs:143-156)."""
from __future__ import annotations

from ..ops import lib as ops
from .base import Norm, ParamSpec


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, out_dtype):
        self.width, self.eps, self.out_dtype = width, float(eps), out_dtype
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), kind="vector", init="ones_normal")}

    def forward(self, h, ctx, rows=None, n_rows=None, tag="norm"):
        """h float32 [T, width] -> compute-dtype rows; `rows` (int32) picks source rows."""
        n = n_rows if n_rows is not None else ctx.n_tokens
        cap = ctx.want_capacity if rows is not None else ctx.token_capacity
        out = ctx.buf(tag + ("_rows" if rows is not None else ""), (cap, self.width), self.out_dtype)
        ops.rmsnorm(h, self.w_weight, out, self.eps, rows=rows, n_rows=n, partials=ctx.take_pending_residual(h))
        return out
