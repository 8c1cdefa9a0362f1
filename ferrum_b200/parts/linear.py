"""y = x W^T for the parts: picks the tensor-core kernel when the operands allow it.

The weight keeps the file's layout [out_features, in_features] with the input dimension
contiguous (the reference's GEMV layout, crates/model/src/weights.rs:124-140), which is the
K-major operand both kernels want.
"""
from __future__ import annotations

import torch

from ..ops import lib as ops

STORE, STORE_F32, RESIDUAL = "store", "store_f32", "residual"
_GENERIC = {STORE: ops.EPI_STORE, STORE_F32: ops.EPI_STORE_F32, RESIDUAL: ops.EPI_RESIDUAL}
_TC = {STORE: ops.TC_STORE_BF16, STORE_F32: ops.TC_STORE_F32, RESIDUAL: ops.TC_RESIDUAL}

def linear_deferred(x, w, ctx, M, N=None, dual_offset=0):
    """The product as float32 partials for the next kernel to sum (`ops.Partials`), or None
    when the shape or the operands do not allow it.  The partials live in the step's product
    workspace: they must be consumed before the next tensor-core product runs."""
    if M == 0 or not ops.gemm_tc_supported(x, w):
        return None
    N = (w.shape[0] - dual_offset) if N is None else N
    K = w.shape[1]
    if not ops.gemm_tc_can_defer(M, N, K, dual_offset > 0):
        return None
    ctx.flush_residual()
    ws, _ = ctx.gemm_scratch(M, N, K, dual_offset > 0)
    return ops.gemm_tc_deferred(x, w, ctx.err, ws, M=M, N=N, dual_offset=dual_offset)


def linear(x, w, out, mode, ctx, M=None):
    """out (=, or += when mode is RESIDUAL) x[:M] @ w.T.  A residual sum of a few tokens may be
    left pending in `ctx` (see StepContext.pending_residual): the next norm adds it."""
    M = x.shape[0] if M is None else M
    if M == 0:
        return
    if mode == RESIDUAL and ctx.defer_residuals:
        part = linear_deferred(x, w, ctx, M)
        if part is not None:
            ctx.pending_residual = (out, part)
            return
    ctx.flush_residual()
    if ops.gemm_tc_supported(x, w):
        N, K = w.shape
        ws, cnt = ctx.gemm_scratch(M, N, K, False)
        ops.gemm_tc(x, w, out, _TC[mode], ctx.err, ws, cnt, M=M)
    else:
        ops.gemm_generic(x, w, out, _GENERIC[mode], M=M)


def linear_swiglu(x, w_gate_up, act, F, ctx, M=None):
    """act = silu(x @ w_gate_up[:F].T) * (x @ w_gate_up[F:].T) in one kernel.  The caller
    checks `ops.gemm_tc_supported` first."""
    M = x.shape[0] if M is None else M
    if M == 0:
        return
    K = w_gate_up.shape[1]
    part = linear_deferred(x, w_gate_up, ctx, M, N=F, dual_offset=F) if ctx.defer_swiglu else None
    if part is not None:
        ops.swiglu_reduce(act, M, F, part)
        return
    ctx.flush_residual()
    # (with many tokens the library runs both products as one on its CTA-pair kernel, gate and
    # up rows interleaved, and applies the activation in that kernel's epilogue)
    ws, cnt = ctx.gemm_scratch(M, F, K, True)
    ops.gemm_tc(x, w_gate_up, act, ops.TC_SWIGLU, ctx.err, ws, cnt, M=M, N=F, dual_offset=F)
