"""Each CUDA kernel alone against a plain float64 reference of the same op, at sizes the
engine's own models do not use (odd widths, tails, several tile shapes)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda):
    from ferrum_b200.ops import lib
    lib.require_cuda()
    return lib


def err_flag():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


H16 = [torch.bfloat16, torch.float16]          # the 16-bit types of the tensor-core kernels
REL16 = {torch.bfloat16: 8e-3, torch.float16: 1e-3}      # one rounding to the type, relative
ATT16 = {torch.bfloat16: 1.5e-2, torch.float16: 2.5e-3}   # attention output of unit-variance values (P and the output are rounded)


def lim(ref, rel):
    return torch.clamp(rel * torch.clamp(ref.abs(), min=1.0), min=1e-6)


# ---------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("V,E,T", [(301, 80, 7), (1000, 1537, 33)])
def test_embedding(ops, dtype, V, E, T):
    g = torch.Generator(device="cuda").manual_seed(1)
    table = torch.randn(V, E, device="cuda", generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
    out = torch.empty(T, E, device="cuda")
    e = err_flag()
    ops.embedding(table, ids, out, e)
    assert torch.equal(out, table[ids.long()].float()) and e.item() == 0
    ids[2] = V
    ops.embedding(table, ids, out, e)
    assert e.item() == 1 and out[2].abs().sum().item() == 0      # refused, not read


# ---------------------------------------------------------------- rmsnorm
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("E,T,eps", [(80, 5, 3e-6), (1537, 9, 1e-5), (4096, 3, 1e-5), (2048, 70, 1e-5)])
def test_rmsnorm(ops, out_dtype, E, T, eps):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, E, device="cuda", generator=g) * 3
    w = 1 + 0.1 * torch.randn(E, device="cuda", generator=g)
    out = torch.empty(T, E, device="cuda", dtype=out_dtype)
    ops.rmsnorm(x, w, out, eps)
    ref = torch.from_numpy(P.rms_norm(x.double().cpu().numpy(), w.double().cpu().numpy(), eps)).cuda()
    tol = 1e-4 if out_dtype == torch.float32 else 8e-3
    assert ((out.double() - ref).abs() <= lim(ref, tol)).all()
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device="cuda")
    out2 = torch.empty(3, E, device="cuda", dtype=out_dtype)
    ops.rmsnorm(x, w, out2, eps, rows=rows)
    assert torch.equal(out2, out[rows.long()])


def test_rmsnorm_anchor(ops):
    """crates/kernels/src/tests.rs:170-176: rms of [3,4] with weights [2,0.5]."""
    x = torch.tensor([[3.0, 4.0]], device="cuda")
    w = torch.tensor([2.0, 0.5], device="cuda")
    out = torch.empty(1, 2, device="cuda")
    ops.rmsnorm(x, w, out, 1e-12)
    inv = 1 / math.sqrt(12.5)
    assert torch.allclose(out.cpu(), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]]), rtol=1e-6)


# ---------------------------------------------------------------- generic product
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 6, 3), (7, 172, 64), (16, 1000, 4100), (17, 130, 64), (40, 200, 260), (65, 129, 173),
                                   (130, 64, 300), (300, 384, 1024)])
def test_gemm_generic(ops, dtype, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = torch.randn(N, K, device="cuda", generator=g).to(dtype)
    ref = x.double() @ w.double().T
    out = torch.empty(M, N, device="cuda", dtype=dtype)
    ops.gemm_generic(x, w, out, ops.EPI_STORE)
    # The products are summed in float32 whatever the storage.  One accumulator walks K: its partial
    # sums grow like sqrt(K) and each of the K additions rounds at that size (6e-8 relative), so the
    # bound grows with K; at K = 4096 it is the reference's own 1e-3 (docs/ARCHITECTURE.md:142-153).
    f32 = max(1e-6, 2.5e-7 * K)
    assert ((out.double() - ref).abs() <= lim(ref, f32) + (0 if dtype == torch.float32 else lim(ref, REL16[dtype]))).all()
    out32 = torch.empty(M, N, device="cuda")
    ops.gemm_generic(x, w, out32, ops.EPI_STORE_F32)
    assert ((out32.double() - ref).abs() <= lim(ref, f32)).all()
    res = torch.randn(M, N, device="cuda", generator=g)
    acc = res.clone()
    ops.gemm_generic(x, w, acc, ops.EPI_RESIDUAL)
    assert ((acc.double() - (res.double() + ref)).abs() <= lim(ref, f32)).all()


def test_gemm_generic_anchor(ops):
    """crates/kernels/src/tests.rs:247-268: [[1,2,3],[4,5,6]] . [1,1,1] = [6,15]."""
    w = torch.tensor([[1.0, 2, 3], [4, 5, 6]], device="cuda")
    x = torch.tensor([[1.0, 1, 1], [1, 0, 0]], device="cuda")
    out = torch.empty(2, 2, device="cuda")
    ops.gemm_generic(x, w, out, ops.EPI_STORE)
    assert out.cpu().tolist() == [[6.0, 15.0], [1.0, 4.0]]


@pytest.mark.parametrize("K", [333, 4096])
def test_gemm_generic_row_independent_of_batch(ops, K):
    """A token's product is bit-identical whatever else is in the call, within each of the two
    kernels (up to 64 tokens: the weight-streaming kernel; more: the tiled kernel), and the two
    agree to float32 rounding."""
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(70, K, device="cuda", generator=g)
    w = torch.randn(90, K, device="cuda", generator=g)

    def run(rows):
        out = torch.empty(len(rows), 90, device="cuda")
        ops.gemm_generic(x[rows].contiguous(), w, out, ops.EPI_STORE)
        return out

    x = torch.cat([x, torch.randn(130, K, device="cuda", generator=g)])
    full = run(list(range(200)))                                 # tiled, 128-token tiles
    assert torch.equal(run(list(range(100)))[37], full[37])      # tiled, another grid
    assert torch.equal(run(list(range(30, 110)))[7], full[37])   # tiled, another place in the tile
    one = run([37])                                              # streaming
    assert torch.equal(run([3, 37, 5, 9, 11, 2, 1, 0, 8, 37])[1], one[0])
    assert torch.equal(run(list(range(37, 53)))[0], one[0])
    assert torch.equal(run(list(range(0, 64)))[37], one[0])      # streaming, several passes
    assert (one[0] - full[37]).abs().max() <= 2.5e-7 * K * full[37].abs().max()


# ---------------------------------------------------------------- tensor-core product
TC_SHAPES = [(1, 128, 64), (5, 200, 136), (16, 384, 512), (33, 1000, 264), (64, 256, 1024), (100, 130, 4096),
             (200, 640, 320), (300, 256, 192), (515, 384, 128), (2500, 640, 128)]   # the last: ten token tiles, two groups


def tc_scratch(ops, M, N, K, dual, n_ctas):
    floats, tiles = ops.gemm_tc_workspace(M, N, K, dual, n_ctas)
    return torch.empty(floats, device="cuda"), torch.zeros(tiles, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("h16", H16)
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("n_ctas", [0, 1, 3, 7])
def test_gemm_tc(ops, M, N, K, n_ctas, h16):
    """n_ctas 0 is the production grid (one CTA per SM, ranges end inside tiles); small
    grids make every CTA walk several tiles and share some with its neighbours."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(M, K, device="cuda", generator=g)).to(h16)
    w = (torch.randn(N, K, device="cuda", generator=g)).to(h16)
    ref = x.double() @ w.double().T
    e = err_flag()
    ws, cnt = tc_scratch(ops, M, N, K, False, n_ctas)
    out = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_tc(x, w, out, ops.TC_STORE_F32, e, ws, cnt, n_ctas=n_ctas)
    assert e.item() == 0
    assert ((out.double() - ref).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all(), (out.double() - ref).abs().max()
    outb = torch.empty(M, N, device="cuda", dtype=h16)
    ops.gemm_tc(x, w, outb, ops.TC_STORE_BF16, e, ws, cnt, n_ctas=n_ctas)
    assert ((outb.double() - ref).abs() <= lim(ref, REL16[h16])).all()
    res = torch.randn(M, N, device="cuda", generator=g)
    acc = res.clone()
    ops.gemm_tc(x, w, acc, ops.TC_RESIDUAL, e, ws, cnt, n_ctas=n_ctas)
    assert ((acc.double() - (res.double() + ref)).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all()
    assert cnt.sum().item() == 0          # the counters are left ready for the next launch
    assert e.item() == 0
    again = torch.empty(M, N, device="cuda")
    ops.gemm_tc(x, w, again, ops.TC_STORE_F32, e, ws, cnt, n_ctas=n_ctas)
    assert torch.equal(again, out)        # shared tiles are summed in K order: run-to-run identical


@pytest.mark.parametrize("h16", H16)
@pytest.mark.parametrize("M,N,K,n_ctas", [(300, 256, 8192, 12), (300, 256, 8192, 40), (300, 256, 8192, 0), (515, 640, 8192, 8),
                                          (515, 640, 8192, 0), (700, 384, 4096, 6)])
def test_gemm_tc_pair_shared_tiles(ops, M, N, K, n_ctas, h16):
    """The CTA-pair kernel where left-over tiles are long enough to be cut among pairs: tiles
    shared by 3 pairs (the finisher adds the others' partials to its accumulator), by 10 (in
    several passes), by dozens (the last arriver sums), and a cut that takes the last whole wave
    with it.  Every epilogue; the float32 result is the same bits from run to run."""
    g = torch.Generator(device="cuda").manual_seed(15)
    x = torch.randn(M, K, device="cuda", generator=g).to(h16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(h16)
    ref = x.double() @ w.double().T
    e = err_flag()
    ws, cnt = tc_scratch(ops, M, N, K, False, n_ctas)
    outb = torch.empty(M, N, device="cuda", dtype=h16)
    ops.gemm_tc(x, w, outb, ops.TC_STORE_BF16, e, ws, cnt, n_ctas=n_ctas)
    assert ((outb.double() - ref).abs() <= lim(ref, REL16[h16])).all(), (outb.double() - ref).abs().max()
    res = torch.randn(M, N, device="cuda", generator=g)
    acc = res.clone()
    ops.gemm_tc(x, w, acc, ops.TC_RESIDUAL, e, ws, cnt, n_ctas=n_ctas)
    assert ((acc.double() - (res.double() + ref)).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all()
    again = res.clone()
    ops.gemm_tc(x, w, again, ops.TC_RESIDUAL, e, ws, cnt, n_ctas=n_ctas)
    assert torch.equal(again, acc)
    out = torch.empty(M, N, device="cuda")
    ops.gemm_tc(x, w, out, ops.TC_STORE_F32, e, ws, cnt, n_ctas=n_ctas)
    assert ((out.double() - ref).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all()
    assert cnt.sum().item() == 0 and e.item() == 0
    # gate and up as one product of interleaved rows
    F = N // 2
    gate, up = ref[:, :F], ref[:, F:]
    want = gate / (1 + torch.exp(-gate)) * up
    ws2, cnt2 = tc_scratch(ops, M, F, K, True, n_ctas)
    act = torch.empty(M, F, device="cuda", dtype=h16)
    ops.gemm_tc(x, w, act, ops.TC_SWIGLU, e, ws2, cnt2, N=F, dual_offset=F, n_ctas=n_ctas)
    assert e.item() == 0 and cnt2.sum().item() == 0
    assert ((act.double() - want).abs() <= lim(want, REL16[h16] + 2e-3)).all(), (act.double() - want).abs().max()


@pytest.mark.parametrize("M,F,K", [(3, 172 * 2, 64), (16, 256, 96), (40, 200, 320), (130, 384, 256), (300, 128, 128),
                                   (129, 72, 64), (515, 200, 320), (700, 1000, 2048)])
@pytest.mark.parametrize("n_ctas", [0, 2, 5])
@pytest.mark.parametrize("h16", H16)
def test_gemm_tc_swiglu(ops, M, F, K, n_ctas, h16):
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(M, K, device="cuda", generator=g).to(h16)
    w = (torch.randn(2 * F, K, device="cuda", generator=g) * 0.2).to(h16)
    gate, up = x.double() @ w[:F].double().T, x.double() @ w[F:].double().T
    ref = gate / (1 + torch.exp(-gate)) * up
    e = err_flag()
    ws, cnt = tc_scratch(ops, M, F, K, True, n_ctas)
    act = torch.empty(M, F, device="cuda", dtype=h16)
    ops.gemm_tc(x, w, act, ops.TC_SWIGLU, e, ws, cnt, N=F, dual_offset=F, n_ctas=n_ctas)
    assert e.item() == 0
    # (the activation uses the fast exponential: 2e-3 on top of the rounding to the type)
    assert ((act.double() - ref).abs() <= lim(ref, REL16[h16] + 2e-3)).all(), (act.double() - ref).abs().max()


def test_gemm_tc_refuses_unaligned(ops):
    from ferrum_b200.errors import KernelError
    x = torch.zeros(4, 172, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(8, 172, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(4, 8, device="cuda")
    assert not ops.gemm_tc_supported(x, w)
    with pytest.raises(KernelError):
        ops.gemm_tc(x, w, out, ops.TC_STORE_F32, err_flag(), torch.empty(1 << 20, device="cuda"),
                    torch.zeros(16, dtype=torch.int32, device="cuda"))


# ---------------------------------------------------------------- rope + cache write, attention
def paged_setup(lens, Hkv, D, page_size, dtype, seed, extra_pages=3):
    """Random K/V for requests of the given lengths, scattered over shuffled pages."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = sum((n + page_size - 1) // page_size for n in lens) + extra_pages
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((n + page_size - 1) // page_size for n in lens) + 1
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    plane = torch.full((n_pages, 2, Hkv, page_size, D), float("nan"), device="cuda").to(dtype)
    ks, vs, p = [], [], 0
    for r, n in enumerate(lens):
        k = torch.randn(n, Hkv, D, device="cuda", generator=g).to(dtype)
        v = torch.randn(n, Hkv, D, device="cuda", generator=g).to(dtype)
        for lp in range((n + page_size - 1) // page_size):
            page = perm[p]; p += 1
            table[r, lp] = page
            lo, hi = lp * page_size, min(n, (lp + 1) * page_size)
            plane[page, 0, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            plane[page, 1, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        ks.append(k); vs.append(v)
    return plane, table.cuda(), ks, vs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(4, 2, 16, 16, 0), (6, 3, 48, 8, 0), (8, 1, 128, 16, 0),
                                                (3, 3, 80, 32, 0), (4, 2, 32, 16, 21), (2, 1, 256, 16, 0)])
def test_attention_generic(ops, dtype, Hq, Hkv, D, ps, window):
    """Mixed batch: a whole prompt, a late portion, two single decoded tokens."""
    lens = [37, 1300, 65, 1]
    qlens = [37, 9, 1, 1]
    plane, table, ks, vs = paged_setup(lens, Hkv, D, ps, dtype, 7)
    g = torch.Generator(device="cuda").manual_seed(8)
    T = sum(qlens)
    q = torch.randn(T, Hq * D, device="cuda", generator=g).to(dtype)
    pos, req = [], []
    for r, (n, ql) in enumerate(zip(lens, qlens)):
        pos += list(range(n - ql, n)); req += [r] * ql
    out = torch.empty(T, Hq * D, device="cuda", dtype=dtype)
    e = err_flag()
    posd, reqd = torch.tensor(pos, dtype=torch.int32, device="cuda"), torch.tensor(req, dtype=torch.int32, device="cuda")
    ops.attention_generic(q, out, T, posd, reqd, table, plane, plane.stride(0), ps, Hq, Hkv, D, 1.0 / math.sqrt(D), window, e)
    # the same rows with their keys cut into splits of 512 among CTAs (what a batch of few tokens runs)
    slots = max(lens) // ops.attention_generic_split() + 2
    part = torch.full((T * Hq * slots * (D + 2),), float("nan"), device="cuda")
    out2 = torch.empty_like(out)
    ops.attention_generic(q, out2, T, posd, reqd, table, plane, plane.stride(0), ps, Hq, Hkv, D, 1.0 / math.sqrt(D), window, e,
                          part, slots)
    # and with up to eight tokens of a request sharing every tile of keys (what a batch of many tokens runs)
    out3 = torch.full_like(out, float("nan"))
    qstart = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32, device="cuda")
    ops.attention_generic(q, out3, T, posd, reqd, table, plane, plane.stride(0), ps, Hq, Hkv, D, 1.0 / math.sqrt(D), window, e,
                          q_start=qstart, n_reqs=len(lens))
    assert e.item() == 0
    for res in (out, out2, out3):
        t0 = 0
        for r, (n, ql) in enumerate(zip(lens, qlens)):
            qfull = np.zeros((n, Hq, D))
            qfull[n - ql:] = q[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
            ref = P.attention(qfull, ks[r].double().cpu().numpy(), vs[r].double().cpu().numpy(), window)[n - ql:]
            got = res[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
            tol = 1e-5 if dtype == torch.float32 else (1.5e-2 if dtype == torch.bfloat16 else 2e-3)
            assert np.abs(got - ref).max() <= tol, (r, np.abs(got - ref).max())
            t0 += ql


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("far_key", [0, 15, 16, 17, 255, 256, 511, 512, 1023, 1024, 1099])
def test_attention_finds_one_far_key(ops, dtype, far_key):
    """One key among 1100 matches the query strongly; its value must come through.  A kernel
    that skips a page edge or the first or last key shows at once."""
    Hq = Hkv = 2; D = 32; ps = 16; n = 1100
    plane, table, ks, vs = paged_setup([n], Hkv, D, ps, dtype, 9)
    kq = ks[0][far_key].float()                       # [Hkv, D]; Hq == Hkv here
    # score of the far key = 40, of every other key ~ N(0, 7)
    q = (kq * (40.0 * math.sqrt(D) / kq.pow(2).sum(-1, keepdim=True))).reshape(1, Hq * D)
    q = q.to(dtype)
    out = torch.empty(1, Hq * D, device="cuda", dtype=dtype)
    e = err_flag()
    slots = n // ops.attention_generic_split() + 2
    part = torch.full((Hq * slots * (D + 2),), float("nan"), device="cuda")
    ops.attention_generic(q, out, 1, torch.tensor([n - 1], dtype=torch.int32, device="cuda"),
                          torch.zeros(1, dtype=torch.int32, device="cuda"), table, plane, plane.stride(0), ps, Hq, Hkv,
                          D, 1.0 / math.sqrt(D), 0, e, part, slots)
    qfull = np.zeros((n, Hq, D)); qfull[-1] = q.double().cpu().numpy().reshape(Hq, D)
    ref = P.attention(qfull, ks[0].double().cpu().numpy(), vs[0].double().cpu().numpy())[-1]
    got = out.double().cpu().numpy().reshape(Hq, D)
    assert np.abs(ref - vs[0][far_key].double().cpu().numpy()).max() < 0.05      # the construction works
    assert np.abs(got - ref).max() <= (1e-4 if dtype == torch.float32 else 2e-2)


def run_flash(ops, q, lens, qlens, table, plane, ps, Hq, Hkv, D, window, use_tc=False, counts=None, comb_warps=1):
    """Drive the tensor-core attention the way the attention part does: plan, launch per
    row-tile class (the tcgen05 kernel for its class when use_tc), merge splits."""
    from ferrum_b200.parts.attention_plan import build_host
    T = sum(qlens)
    out = torch.full((T, Hq * D), float("nan"), device="cuda", dtype=q.dtype)
    pos0 = [n - ql for n, ql in zip(lens, qlens)]
    qs = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    req = np.repeat(np.arange(len(lens)), qlens).astype(np.int32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32).cuda()
    n_split_items = 0
    tc_tokens = ops.attention_tc_tokens(D, Hq // Hkv, ps, plane, plane.stride(0)) if use_tc else 0
    assert tc_tokens > 0 or not use_tc
    e = err_flag()
    for h in build_host(qlens, pos0, Hq // Hkv, window, Hkv, tc_tokens):
        if h is None:
            continue
        part_o = torch.empty(max(1, h["n_slots"] * h["bm"] * D), device="cuda")
        part_ml = torch.empty(max(1, h["n_slots"] * h["bm"] * 2), device="cuda")
        if counts is not None:
            counts[h["kind"]] = counts.get(h["kind"], 0) + h["n_work"]
            counts["split_" + h["kind"]] = counts.get("split_" + h["kind"], 0) + h["n_slots"]
        if h["kind"] == "tc":
            ops.attention_tc(q, out, plane, plane.stride(0), ps, table, dev(qs), dev(pos0), dev(h["work"]), h["n_work"],
                             part_o, part_ml, Hq, Hkv, D, 1.0 / math.sqrt(D), window, e)
            assert e.item() == 0
        else:
            ops.attention_flash(q, out, plane, plane.stride(0), ps, table, dev(qs), dev(pos0), dev(h["work"]), h["n_work"],
                                part_o, part_ml, Hq, Hkv, D, 1.0 / math.sqrt(D), window, h["bm"], e,
                                dev(h["cta_items"]) if h["n_ctas"] else None, h["n_ctas"])
            assert e.item() == 0
        if h["comb"].size:
            ops.attention_combine(out, part_o, part_ml, dev(qs), dev(req), dev(h["req_tile0"]), dev(h["tile_info"]),
                                  dev(h["comb"]), int(h["comb"].size), Hq, Hkv, D, h["bm"], comb_warps)
        n_split_items += h["n_slots"]
    return out, n_split_items


@pytest.mark.parametrize("h16", H16)
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(4, 2, 64, 16, 0), (6, 2, 64, 8, 0), (8, 1, 128, 16, 0), (32, 8, 128, 16, 0),
                                                (3, 3, 128, 32, 0), (4, 2, 64, 16, 21), (8, 2, 128, 16, 300),
                                                (40, 2, 64, 16, 0)])
def test_attention_flash(ops, Hq, Hkv, D, ps, window, h16):
    """Mixed batch on the tensor-core kernel: a whole prompt, a late portion of a long
    request, decoded tokens at short and long contexts (the long ones are split)."""
    lens = [137, 1500, 65, 1, 2300, 700]
    qlens = [137, 70, 1, 1, 1, 2]
    plane, table, ks, vs = paged_setup(lens, Hkv, D, ps, h16, 17)
    g = torch.Generator(device="cuda").manual_seed(18)
    T = sum(qlens)
    q = torch.randn(T, Hq * D, device="cuda", generator=g).to(h16)
    out, n_split = run_flash(ops, q, lens, qlens, table, plane, ps, Hq, Hkv, D, window)
    assert n_split > 0 or window > 0
    t0 = 0
    for r, (n, ql) in enumerate(zip(lens, qlens)):
        qfull = np.zeros((n, Hq, D))
        qfull[n - ql:] = q[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
        ref = P.attention(qfull, ks[r].double().cpu().numpy(), vs[r].double().cpu().numpy(), window)[n - ql:]
        got = out[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
        assert np.abs(got - ref).max() <= ATT16[h16], (r, np.abs(got - ref).max())
        t0 += ql


@pytest.fixture(params=[True, False], ids=["pair", "single"])
def pair(request, ops):
    """Head size 128 runs on CTA pairs by default; the single-CTA kernel is tested too."""
    ops.set_attention_pair_kernel(request.param)
    yield request.param
    ops.set_attention_pair_kernel(True)


@pytest.mark.parametrize("h16", H16)
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(4, 2, 64, 16, 0), (6, 2, 64, 8, 0), (8, 1, 128, 16, 0), (32, 8, 128, 16, 0),
                                                (3, 3, 128, 32, 0), (4, 2, 64, 64, 21), (8, 2, 128, 16, 300),
                                                (10, 2, 128, 16, 0), (14, 2, 64, 16, 90), (4, 1, 128, 8, 700)])
def test_attention_tc(ops, Hq, Hkv, D, ps, window, h16, pair):
    """The tcgen05 kernel on prompt portions: a whole prompt, a late portion of a long request
    (its key range is split), a portion that ends inside a tile, beside decoded tokens that
    stay on the other kernel.  Groups that do not divide 128 leave padding rows in the tiles."""
    lens = [137, 5400, 65, 1, 700, 333]
    qlens = [137, 130, 1, 1, 450, 200]
    plane, table, ks, vs = paged_setup(lens, Hkv, D, ps, h16, 27)
    g = torch.Generator(device="cuda").manual_seed(28)
    T = sum(qlens)
    q = torch.randn(T, Hq * D, device="cuda", generator=g).to(h16)
    if window > 0:
        # pages that every query's window has passed are given back, as the cache manager does:
        # their table entries are -1 and their contents belong to someone else (NaN here)
        for r, (n, ql) in enumerate(zip(lens, qlens)):
            first_needed = max(0, n - ql - window + 1) // ps
            for lp in range(first_needed):
                plane[table[r, lp].item()] = float("nan")
                table[r, lp] = -1
    counts = {}
    out, _ = run_flash(ops, q, lens, qlens, table, plane, ps, Hq, Hkv, D, window, use_tc=True, counts=counts)
    assert counts.get("tc", 0) > 0 and (window > 0 or counts.get("split_tc", 0) > 0), counts
    t0 = 0
    for r, (n, ql) in enumerate(zip(lens, qlens)):
        qfull = np.zeros((n, Hq, D))
        qfull[n - ql:] = q[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
        ref = P.attention(qfull, ks[r].double().cpu().numpy(), vs[r].double().cpu().numpy(), window)[n - ql:]
        got = out[t0:t0 + ql].double().cpu().numpy().reshape(ql, Hq, D)
        assert np.isfinite(got).all(), r
        assert np.abs(got - ref).max() <= ATT16[h16], (r, np.abs(got - ref).max())
        t0 += ql


@pytest.mark.parametrize("Hq,Hkv,D,comb_warps", [(8, 2, 128, 8), (4, 4, 64, 3), (8, 2, 128, 1)])
def test_attention_merge_of_many_splits(ops, Hq, Hkv, D, comb_warps):
    """One decoded token over 20000 keys: its (request, head) pairs are cut into dozens of
    splits, which the merge kernel's warps share; one key far back carries the weight."""
    ps = 16; n = 20000; far_key = 777
    plane, table, ks, vs = paged_setup([n], Hkv, D, ps, torch.bfloat16, 31)
    g = torch.Generator(device="cuda").manual_seed(32)
    q = torch.randn(1, Hq * D, device="cuda", generator=g).bfloat16()
    counts = {}
    out, n_split = run_flash(ops, q, [n], [1], table, plane, ps, Hq, Hkv, D, 0, counts=counts, comb_warps=comb_warps)
    assert n_split >= 16 * Hkv, n_split
    G = Hq // Hkv                                              # the last row sees every key: softmax(q k / sqrt(D)) v
    qd = q.double().reshape(Hkv, G, D)
    sc = torch.einsum("hgd,nhd->hgn", qd, ks[0].double()) / math.sqrt(D)
    ref = torch.einsum("hgn,nhd->hgd", torch.softmax(sc, dim=-1), vs[0].double()).reshape(1, Hq * D)
    assert (out.double() - ref).abs().max().item() <= 1.5e-2
    # and with one query made to match one key: the split that holds it must win the merge
    kq = ks[0][far_key].float()
    q2 = (kq * (40.0 * math.sqrt(D) / kq.pow(2).sum(-1, keepdim=True))).reshape(1, Hkv, 1, D).expand(1, Hkv, Hq // Hkv, D)
    q2 = q2.reshape(1, Hq * D).bfloat16().contiguous()
    out2, _ = run_flash(ops, q2, [n], [1], table, plane, ps, Hq, Hkv, D, 0, comb_warps=comb_warps)
    want = vs[0][far_key].float().reshape(Hkv, 1, D).expand(Hkv, Hq // Hkv, D).reshape(1, Hq * D)
    assert (out2.float() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("far_key", [0, 15, 16, 63, 64, 255, 256, 1023, 1024, 2047, 2048, 2999])
def test_attention_tc_finds_one_far_key(ops, far_key):
    """One strongly matching key among 3000, at stage, page and split edges, for a prompt portion
    on the tcgen05 kernel."""
    Hq = Hkv = 2; D = 64; ps = 16; n = 3000; qlen = 200
    plane, table, ks, vs = paged_setup([n], Hkv, D, ps, torch.bfloat16, 19)
    kq = ks[0][far_key].float()
    qrow = (kq * (40.0 * math.sqrt(D) / kq.pow(2).sum(-1, keepdim=True))).reshape(1, Hq * D)
    q = qrow.repeat(qlen, 1).bfloat16()
    out, _ = run_flash(ops, q, [n], [qlen], table, plane, ps, Hq, Hkv, D, 0, use_tc=True)
    want = vs[0][far_key].float().reshape(1, Hq * D)
    sees = max(0, far_key - (n - qlen))          # rows before this one come before the key
    assert (out[sees:].float() - want).abs().max().item() <= 2e-2


def test_attention_tc_ignores_what_lies_past_the_keys(ops):
    """Rows of the last page beyond the request's length hold NaN: no weight may touch them."""
    Hq, Hkv, D, ps = 4, 2, 128, 16
    lens, qlens = [200], [200]
    plane, table, ks, vs = paged_setup(lens, Hkv, D, ps, torch.bfloat16, 33)
    last_page = table[0, (lens[0] - 1) // ps].item()
    plane[last_page, :, :, lens[0] % ps:] = float("nan")
    g = torch.Generator(device="cuda").manual_seed(34)
    q = torch.randn(200, Hq * D, device="cuda", generator=g).bfloat16()
    out, _ = run_flash(ops, q, lens, qlens, table, plane, ps, Hq, Hkv, D, 0, use_tc=True)
    qfull = q.double().cpu().numpy().reshape(200, Hq, D)
    ref = P.attention(qfull, ks[0].double().cpu().numpy(), vs[0].double().cpu().numpy(), 0)
    got = out.double().cpu().numpy().reshape(200, Hq, D)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 1.5e-2


@pytest.mark.parametrize("far_key", [0, 15, 16, 63, 64, 255, 256, 1023, 1024, 2999])
@pytest.mark.parametrize("qlen", [1, 40])
def test_attention_flash_finds_one_far_key(ops, far_key, qlen):
    """As for the generic kernel: one strongly matching key among 3000, at tile, page and
    split edges, for a decoded token (split key range) and for a prompt portion."""
    Hq = Hkv = 2; D = 64; ps = 16; n = 3000
    plane, table, ks, vs = paged_setup([n], Hkv, D, ps, torch.bfloat16, 19)
    kq = ks[0][far_key].float()
    qrow = (kq * (40.0 * math.sqrt(D) / kq.pow(2).sum(-1, keepdim=True))).reshape(1, Hq * D)
    q = qrow.repeat(qlen, 1).bfloat16()
    out, _ = run_flash(ops, q, [n], [qlen], table, plane, ps, Hq, Hkv, D, 0)
    qfull = np.zeros((n, Hq, D)); qfull[n - qlen:] = q.double().cpu().numpy().reshape(qlen, Hq, D)
    ref = P.attention(qfull, ks[0].double().cpu().numpy(), vs[0].double().cpu().numpy())[n - qlen:]
    got = out.double().cpu().numpy().reshape(qlen, Hq, D)
    assert np.abs(ref[-1] - vs[0][far_key].double().cpu().numpy()).max() < 0.05
    assert np.abs(got - ref).max() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("pairing", ["adjacent", "half"])
@pytest.mark.parametrize("Hq,Hkv,D,R", [(4, 2, 16, 16), (3, 1, 48, 32), (2, 2, 128, 128), (5, 1, 48, 48)])
@pytest.mark.parametrize("many", [False, True])
def test_rope_cache_write(ops, dtype, pairing, Hq, Hkv, D, R, many):
    from ferrum_b200.parts.rope import RotaryEmbedding
    ps, n_pos = 8, 300
    rot = RotaryEmbedding(D, R, 10000.0, None, pairing, n_pos, "cuda")
    positions = [0, 1, 7, 8, 9, 250, 299, 64]
    req = [0, 0, 0, 0, 0, 1, 1, 1]
    if many:   # the many-token kernels; every (request, position) once
        extra = [p for p in np.random.default_rng(5).permutation(n_pos).tolist() if p not in positions][:90]
        positions = positions + extra
        req = req + [i % 2 for i in range(len(extra))]
        taken = set()
        for i, pr in enumerate(zip(req, positions)):
            assert pr not in taken
            taken.add(pr)
    T = len(positions)
    g = torch.Generator(device="cuda").manual_seed(10)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", generator=g).to(dtype)
    orig = qkv.clone()
    width = (n_pos + ps - 1) // ps
    # the two requests share no page; logical pages map to shuffled page ids
    table = torch.stack([torch.arange(width), torch.arange(width) + width]).to(torch.int32)
    table = table[:, torch.randperm(width, generator=torch.Generator().manual_seed(3))].contiguous().cuda()
    plane = torch.zeros(2 * width, 2, Hkv, ps, D, device="cuda", dtype=dtype)
    e = err_flag()
    ops.rope_cache_write(qkv, T, torch.tensor(positions, dtype=torch.int32, device="cuda"),
                         torch.tensor(req, dtype=torch.int32, device="cuda"), table, rot.cos_sin, plane,
                         plane.stride(0), ps, Hq, Hkv, D, R, rot.pairing, True, e)
    assert e.item() == 0
    inv = np.array([10000.0 ** (-2.0 * i / R) for i in range(R // 2)])
    o = orig.double().cpu().numpy()
    qref = o[:, :Hq * D].reshape(T, Hq, D).copy()
    kref = o[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).copy()
    qref[..., :R] = P.rope(qref[..., :R], np.array(positions), inv, pairing)
    kref[..., :R] = P.rope(kref[..., :R], np.array(positions), inv, pairing)
    vref = o[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(qkv[:, :Hq * D].double().cpu().numpy().reshape(T, Hq, D) - qref).max() <= tol
    for t, (p, r) in enumerate(zip(positions, req)):
        page = table[r, p // ps].item()
        assert np.abs(plane[page, 0, :, p % ps].double().cpu().numpy() - kref[t]).max() <= tol
        assert np.abs(plane[page, 1, :, p % ps].double().cpu().numpy() - vref[t]).max() == 0
    # position 0 is the identity (crates/kernels/src/tests.rs:197-238)
    assert torch.equal(qkv[0, :Hq * D], orig[0, :Hq * D])


# ---------------------------------------------------------------- swiglu, sampling
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,F", [(3, 172), (17, 1000)])
def test_swiglu(ops, dtype, T, F):
    g = torch.Generator(device="cuda").manual_seed(11)
    gu = (torch.randn(T, 2 * F, device="cuda", generator=g) * 3).to(dtype)
    act = torch.empty(T, F, device="cuda", dtype=dtype)
    ops.swiglu(gu, act, T, F)
    a = gu.double()
    ref = torch.from_numpy(P.silu(a[:, :F].cpu().numpy())).cuda() * a[:, F:]
    assert ((act.double() - ref).abs() <= lim(ref, 1e-5 if dtype == torch.float32 else 8e-3)).all()


def test_argmax_rules(ops):
    """crates/core-types/src/model.rs:304-309: [1,3,3,NaN] -> 1; all NaN is an error."""
    logits = torch.tensor([[1.0, 3.0, 3.0, float("nan")], [float("nan")] * 4, [-5.0, -7.0, -5.0, -9.0]], device="cuda")
    ids = torch.empty(3, dtype=torch.int32, device="cuda")
    e = err_flag()
    ops.sample(logits, 3, ids, e)
    assert ids.cpu().tolist() == [1, -1, 0] and e.item() == 6
    # a second destination gets the same ids (the token buffer of a step queued behind this one)
    again = torch.full((5,), 77, dtype=torch.int32, device="cuda")
    ops.sample(logits, 3, ids, e, also_to=again)
    assert again.cpu().tolist() == [1, -1, 0, 77, 77]


@pytest.mark.parametrize("V", [301, 128256])
def test_sampling_matches_plain(ops, V):
    g = torch.Generator(device="cuda").manual_seed(12)
    R = 6
    logits = torch.randn(R, V, device="cuda", generator=g) * 2
    temps = [0.0, 0.8, 0.8, 1.5, 0.3, 0.8]
    seeds = [0, 1, 2 ** 40 + 7, 5, 5, 1]
    counters = [0, 0, 3, 9, 9, 1]
    inv_t = torch.tensor([np.float32(1.0 / t) if t else 0.0 for t in temps], dtype=torch.float32, device="cuda")
    ids = torch.empty(R, dtype=torch.int32, device="cuda")
    e = err_flag()
    ops.sample(logits, R, ids, e, inv_t, torch.tensor(seeds, dtype=torch.int64, device="cuda"),
               torch.tensor(counters, dtype=torch.int32, device="cuda"))
    host = logits.cpu().numpy()
    for r in range(R):
        want = P.sample(host[r], temps[r], seeds[r], counters[r])
        got = ids[r].item()
        if got != want:      # only a near-tie of the perturbed logits may differ (logf rounding)
            u = P.gumbel_uniform(seeds[r], counters[r], V)
            z = host[r].astype(np.float64) / temps[r] - np.log(-np.log(u))
            assert abs(z[got] - z[want]) < 1e-4, (r, got, want)
    # the draw follows softmax(logits / T): frequencies over many seeds, small vocabulary
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device="cuda").repeat(4000, 1)
    n = small.shape[0]
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(small, n, out, e, torch.full((n,), 1.0, device="cuda"),
               torch.arange(n, dtype=torch.int64, device="cuda"), torch.zeros(n, dtype=torch.int32, device="cuda"))
    freq = np.bincount(out.cpu().numpy(), minlength=4) / n
    p = np.exp([2.0, 1, 0, -1]); p /= p.sum()
    assert np.abs(freq - p).max() < 0.03, (freq, p)


# ---------------------------------------------------------------- deferred reduction
@pytest.mark.parametrize("h16", H16)
@pytest.mark.parametrize("M,N,K", [(1, 384, 512), (8, 6144, 4096), (33, 1000, 264), (64, 4096, 2048), (100, 4096, 4096),
                                   (200, 2048, 1024), (256, 4096, 14336)])
def test_gemm_deferred_partials_and_their_consumers(ops, M, N, K, h16):
    """The product left as partials, summed by each kind of consumer: the residual reduce,
    the norm that adds a pending residual, and (two products) the SwiGLU reduce."""
    if not ops.gemm_tc_can_defer(M, N, K, False):
        pytest.skip("shape cannot defer")
    g = torch.Generator(device="cuda").manual_seed(31)
    x = torch.randn(M, K, device="cuda", generator=g).to(h16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(h16)
    ref = x.double() @ w.double().T
    e = err_flag()
    floats, _ = ops.gemm_tc_workspace(M, N, K, False)
    ws = torch.empty(floats, device="cuda")
    part = ops.gemm_tc_deferred(x, w, e, ws)
    h0 = torch.randn(M, N, device="cuda", generator=g)
    h = h0.clone()
    ops.residual_reduce(h, M, part)
    assert e.item() == 0
    assert ((h.double() - (h0.double() + ref)).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all()
    # same numbers as the kernel's own reduction: both add the partials in K order
    floats2, tiles = ops.gemm_tc_workspace(M, N, K, False)
    own = h0.clone()
    ops.gemm_tc(x, w, own, ops.TC_RESIDUAL, e, torch.empty(floats2, device="cuda"),
                torch.zeros(tiles, dtype=torch.int32, device="cuda"))
    if ops.gemm_tc_token_tile(M, False) <= 128:
        assert torch.equal(own, h)
    else:   # more than 128 tokens: the kernel's own reduction runs on CTA pairs, which cut K elsewhere
        assert ((own.double() - (h0.double() + ref)).abs() <= lim(ref, 2e-5) * math.sqrt(K)).all()
    # the norm adds the pending sum, writes the residual back and normalises it
    part = ops.gemm_tc_deferred(x, w, e, ws)
    h2 = h0.clone()
    wn = 1 + 0.1 * torch.randn(N, device="cuda", generator=g)
    out = torch.empty(M, N, device="cuda", dtype=h16)
    ops.rmsnorm(h2, wn, out, 1e-5, partials=part)
    assert torch.equal(h2, h)
    want = torch.from_numpy(P.rms_norm(h.double().cpu().numpy(), wn.double().cpu().numpy(), 1e-5)).cuda()
    assert ((out.double() - want).abs() <= lim(want, REL16[h16])).all()
    if N % 2 == 0 and ops.gemm_tc_can_defer(M, N // 2, K, True):
        F = N // 2
        ws2 = torch.empty(ops.gemm_tc_workspace(M, F, K, True)[0], device="cuda")
        part = ops.gemm_tc_deferred(x, w, e, ws2, N=F, dual_offset=F)
        act = torch.empty(M, F, device="cuda", dtype=h16)
        ops.swiglu_reduce(act, M, F, part)
        gate, up = ref[:, :F], ref[:, F:]
        want = gate / (1 + torch.exp(-gate)) * up
        assert ((act.double() - want).abs() <= lim(want, REL16[h16] + 2e-3)).all()
    assert e.item() == 0
