"""The allocation-free entry point of the kernel library, called the way an embedder calls it.

Some users of the library cannot allocate device memory at the time they need a product: a
host application that owns all GPU memory through its own pool, or a latency-critical loop
where cudaMalloc is forbidden.  `ferrum_gemm_tc_noalloc` is for them; it keeps its scratch
inside the library.  Here it is reached through its exported C symbol with raw pointers, and
its output is compared with the regular entry point's, twice in a row, since every call
shares the same built-in scratch.  The file sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def call_noalloc(lib, x, w, out, M, N, K, epilogue, dual_offset, err):
    fn = lib.ferrum_gemm_tc_noalloc
    fn.restype = c_int
    return fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
              c_int(x.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(w.shape[0]), c_int(epilogue),
              c_int(dual_offset), c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("M,N,K", [(8, 6144, 4096), (1, 384, 512), (33, 1000, 264)])
def test_noalloc_product_matches_the_regular_entry_point_twice(cuda, M, N, K):
    from ferrum_b200.ops import lib as ops
    lib = ops.lib()
    g = torch.Generator(device="cuda").manual_seed(21)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    floats, tiles = ops.gemm_tc_workspace(M, N, K, False)
    ws, cnt = torch.empty(floats, device="cuda"), torch.zeros(tiles, dtype=torch.int32, device="cuda")
    for round_ in range(2):                                   # the second call meets the first call's leftovers
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        want = torch.empty(M, N, device="cuda")
        ops.gemm_tc(x, w, want, ops.TC_STORE_F32, err, ws, cnt)
        got = torch.full((M, N), float("nan"), device="cuda")
        assert call_noalloc(lib, x, w, got, M, N, K, ops.TC_STORE_F32, 0, err) == 0, lib.ferrum_last_error()
        torch.cuda.synchronize()
        assert err.item() == 0
        # both paths add the same partial sums in the same order
        assert torch.equal(got, want), (round_, (got - want).abs().max().item())
        ref = x.double() @ w.double().T
        lim = torch.clamp(2e-5 * torch.clamp(ref.abs(), min=1.0), min=1e-6) * (K ** 0.5)
        assert ((got.double() - ref).abs() <= lim).all()
        # the residual epilogue adds into the caller's output
        res = torch.randn(M, N, device="cuda", generator=g)
        a, b = res.clone(), res.clone()
        ops.gemm_tc(x, w, a, ops.TC_RESIDUAL, err, ws, cnt)
        assert call_noalloc(lib, x, w, b, M, N, K, ops.TC_RESIDUAL, 0, err) == 0
        assert torch.equal(a, b)


def test_noalloc_swiglu_and_refusals(cuda):
    from ferrum_b200.ops import lib as ops
    lib = ops.lib()
    g = torch.Generator(device="cuda").manual_seed(22)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    M, F, K = 16, 512, 256
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * F, K, device="cuda", generator=g) * 0.2).bfloat16()
    floats, tiles = ops.gemm_tc_workspace(M, F, K, True)
    want = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc(x, w, want, ops.TC_SWIGLU, err, torch.empty(floats, device="cuda"),
                torch.zeros(tiles, dtype=torch.int32, device="cuda"), N=F, dual_offset=F)
    for _ in range(2):
        got = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
        assert call_noalloc(lib, x, w, got, M, F, K, ops.TC_SWIGLU, F, err) == 0
        assert torch.equal(got, want)
    # ... and against exact arithmetic on the same operands: silu(gate) * up, rounded to bfloat16 once
    gate, up = x.double() @ w[:F].double().T, x.double() @ w[F:].double().T
    ref = gate / (1 + torch.exp(-gate)) * up
    assert ((got.double() - ref).abs() <= 8e-3 * torch.clamp(ref.abs(), min=1.0)).all()
    # shapes beyond the built-in scratch are refused before anything is launched
    big = torch.zeros(512, K, device="cuda", dtype=torch.bfloat16)
    out = torch.full((512, 2 * F), 7.0, device="cuda")
    assert call_noalloc(lib, big, w, out, 512, 2 * F, K, ops.TC_STORE_F32, 0, err) != 0
    assert b"scratch" in lib.ferrum_last_error()
    torch.cuda.synchronize()
    assert (out == 7.0).all() and err.item() == 0
    bad = torch.zeros(4, 172, device="cuda", dtype=torch.bfloat16)          # rows that TMA cannot address
    assert call_noalloc(lib, bad, bad, out, 4, 4, 172, ops.TC_STORE_F32, 0, err) != 0


def test_noalloc_call_leaves_the_free_memory_as_it_was(cuda):
    """A warmed-up call takes no device memory: the driver's free figure is the same before and
    after (the first call on a device may resolve the built-in scratch's address and is made here
    before the measurement)."""
    from ferrum_b200.ops import lib as ops
    lib = ops.lib()
    M, N, K = 8, 1024, 512
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert call_noalloc(lib, x, w, out, M, N, K, ops.TC_STORE_F32, 0, err) == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call_noalloc(lib, x, w, out, M, N, K, ops.TC_STORE_F32, 0, err) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and err.item() == 0
