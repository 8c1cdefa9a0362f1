"""Failure paths on the device, in the forms that leave the GPU usable: a bounded wait that runs
out returns an error code, a missing page is reported instead of read.  Nothing here traps,
faults or hangs: every kernel involved returns by itself and the next launch works.

The reference's analogue is the fault injection of its scheduler tests, a model that fails on
call N (crates/scheduler/src/batcher.rs:366-372,459-462), and the rule that a failed forward
leaves the sequence lengths as they were (crates/model/src/llama.rs:368-389)."""
import ctypes
import math

import numpy as np
import pytest
import torch

from conftest import TINY
from helpers import Replay, assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ops(cuda):
    from ferrum_b200.ops import lib
    lib.require_cuda()
    yield lib
    lib.gemm_tc_test_hooks()        # whatever a test set is set back


@pytest.mark.parametrize("M,N,K,dual", [(8, 512, 1024, False), (100, 256, 512, False), (16, 256, 512, True)])
def test_a_wait_that_runs_out_becomes_an_error_code(ops, M, N, K, dual):
    """The producer of the tensor-core product requests nothing (a test hook) and every wait is
    cut to 200 000 cycles: the matrix-unit thread and the epilogue give up, the kernel raises
    an error code between 10 and 13, frees its tensor memory and returns.  The same launch with
    the hooks off is then correct, on the same context."""
    g = torch.Generator(device="cuda").manual_seed(51)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn((2 if dual else 1) * N, K, device="cuda", generator=g) * 0.1).bfloat16()
    floats, tiles = ops.gemm_tc_workspace(M, N, K, dual)
    ws, cnt = torch.empty(floats, device="cuda"), torch.zeros(tiles, dtype=torch.int32, device="cuda")
    e = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if dual else torch.float32)
    epi = ops.TC_SWIGLU if dual else ops.TC_STORE_F32

    def launch():
        ops.gemm_tc(x, w, out, epi, e, ws, cnt, N=N, dual_offset=N if dual else 0)
        torch.cuda.synchronize()

    ops.gemm_tc_test_hooks(wait_cycles=200_000, drop_loads=True)
    launch()
    assert 10 <= e.item() <= 13, e.item()
    ops.gemm_tc_test_hooks()
    e.zero_()
    cnt.zero_()
    launch()
    assert e.item() == 0
    ref = x.double() @ w[:N].double().T
    if dual:
        up = x.double() @ w[N:].double().T
        ref = ref / (1 + torch.exp(-ref)) * up
    assert ((out.double() - ref).abs() <= torch.clamp(1e-2 * ref.abs().clamp(min=1.0), min=1e-6)).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("what", ["write", "read"])
def test_a_missing_page_fails_the_step_and_nothing_else(cuda, model_dirs, dtype, what, monkeypatch):
    """One entry of a block table is -1 on the host for one step: where the step's own token
    would be written (error 4, the rotary kernel) or where an earlier key lies (error 5, the
    attention kernels).  The step raises KernelError, the request's length is unchanged, and the
    same step run again with the true table gives the right logits."""
    from ferrum_b200 import KernelError, host
    from ferrum_b200.engine.trace import TraceSession
    toks = random_tokens(60, TINY["D"][0]["vocab_size"], 90)
    s = TraceSession(model_dirs["D"], dtype, 64)
    r = Replay(s)
    r.step([("a", toks[:40], "all")])
    slot = s.slots["a"]
    assert s.cache.manager.seq_len(slot) == 40
    real = host.module().copy_tables

    def with_a_hole(cache, group, slots, dst, row_stride):
        real(cache, group, slots, dst, row_stride)
        row = (ctypes.c_int32 * row_stride).from_address(dst)
        row[40 // 16 if what == "write" else 0] = -1          # the page of position 40, or of positions 0..15

    monkeypatch.setattr(host.module(), "copy_tables", with_a_hole)
    # (a missing page of the step's own tokens is also missing for the attention that follows: 4 or 5)
    with pytest.raises(KernelError, match="device error [45]" if what == "write" else "device error 5"):
        r.step([("a", toks[40:45], "all")])
    monkeypatch.setattr(host.module(), "copy_tables", real)
    assert s.cache.manager.seq_len(slot) == 40 and s.cache.manager.check() == ""
    r.step([("a", toks[40:45], "all")])
    for t in toks[45:]:
        r.step([("a", [t], "all")])
    assert_close(r.logits("a", 60), plain_logits(model_dirs["D"], dtype, toks), dtype, f"after a failed step ({what})")


def test_engine_abandons_a_failed_step(cuda, model_dirs, monkeypatch):
    """Through the Python entry point: a step whose kernels report an error raises, the scheduler
    forgets the plan (no token is emitted, no length advances), and stepping again generates what
    an undisturbed engine generates."""
    from ferrum_b200 import Engine, KernelError, host
    prompt = random_tokens(20, TINY["D"][0]["vocab_size"], 91)
    args = dict(dtype="bfloat16", num_pages=32, max_batch_tokens=64, max_batch_seqs=4, max_model_len=128, plan_ahead=False)
    want = Engine(model_dirs["D"], **args).generate([prompt], max_new_tokens=8)[0]
    eng = Engine(model_dirs["D"], **args)
    rid = eng.submit(prompt, 8)
    real = host.module().copy_tables

    def with_a_hole(cache, group, slots, dst, row_stride):
        real(cache, group, slots, dst, row_stride)
        (ctypes.c_int32 * row_stride).from_address(dst)[0] = -1

    monkeypatch.setattr(host.module(), "copy_tables", with_a_hole)
    with pytest.raises(KernelError, match="device error"):
        eng.step()
    monkeypatch.setattr(host.module(), "copy_tables", real)
    got = []
    while len(got) < 8:
        for ev in eng.step():
            if ev.kind == "token":
                got.append(ev.token)
    assert got == want and eng.stats()["preemptions"] == 0
