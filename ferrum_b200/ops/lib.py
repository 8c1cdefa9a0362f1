"""The kernel library, loaded once, and thin checked wrappers around its C entry points.

There is no fallback: if the library cannot be built or loaded, or there is no CUDA
device, every op raises `KernelError`.  Wrappers take torch tensors only as typed
memory (pointer, shape, stride); no torch operator runs on the product path.
"""
from __future__ import annotations

import ctypes
import functools
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from . import build

F32, BF16, F16 = 0, 1, 2
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
SIXTEEN_BIT = (torch.bfloat16, torch.float16)       # the tensor-core kernels take either

EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL = 0, 1, 2                       # generic product
TC_STORE_BF16, TC_STORE_F32, TC_RESIDUAL, TC_SWIGLU = 0, 1, 2, 3       # tcgen05 product

_lib = None
_lock = threading.Lock()
ABI = 7


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.build_kernels()
                try:
                    handle = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the kernel library {path}: {e}") from None
                handle.ferrum_last_error.restype = ctypes.c_char_p
                handle.ferrum_gemm_tc_workspace.restype = c_longlong
                if handle.ferrum_kernels_abi() != ABI:
                    raise KernelError(f"{path} is a stale build; delete it and call again")
                if os.environ.get("FERRUM_DEPENDENT_LAUNCH", "1") == "0":
                    handle.ferrum_set_dependent_launch(c_int(0))
                _lib = handle
    return _lib


def require_cuda(device=None):
    if not torch.cuda.is_available():
        raise KernelError("ferrum_b200 runs on a CUDA device only (sm_100a); none is visible")
    lib()


def sm_count():
    """Multiprocessors of the current CUDA device, as the kernels' own grids count them."""
    return int(lib().ferrum_gemm_tc_default_ctas())


def gemm_tc_test_hooks(wait_cycles=0, drop_loads=False):
    """For tests of the failure path only: shorten every bounded wait of the tensor-core product
    kernels to `wait_cycles` clock cycles (0: the default of about a second), and make the
    producer of the single-CTA kernel request nothing, so that the waits run out and the kernel
    leaves with an error code.  Call again without arguments to restore."""
    lib().ferrum_gemm_tc_test_hooks(c_longlong(int(wait_cycles)), c_int(1 if drop_loads else 0))


def set_dependent_launch(on: bool):
    """Programmatic dependent launch between the kernels of a step (on by default): a kernel's
    prologue may overlap the tail of the kernel before it.  Off: plain stream order."""
    lib().ferrum_set_dependent_launch(c_int(1 if on else 0))


launches = 0          # kernel launches made through this module (every entry point launches one kernel)


class _Profile:
    """Per-kernel timing for `profile_begin` / `profile_report`: one CUDA event after every launch;
    a launch's time is the span from the event before it to its own (its wait for the kernel ahead
    of it included).  `work` is (bytes it must move, flops) where the wrapper knows them."""

    def __init__(self):
        self.rows = []        # (name, event after, work)
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def mark(self, name, work):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.rows.append((name, ev, work))


_profile = None
_work = None          # set by a wrapper just before its launch: (bytes, flops)


def profile_begin():
    """Start timing every kernel launched through this module (steps must run without CUDA graphs:
    `Engine(profile=True)` sees to it)."""
    global _profile
    require_cuda()
    _profile = _Profile()


def profile_report(peaks=None):
    """Stops the timing and returns one row per kernel name, largest total first: launches, total
    milliseconds, share of the total, microseconds per launch and, where the wrapper knows the
    kernel's work, GB/s and TFLOP/s (with `peaks` = {"hbm_gbs", "bf16_tflops"} also the fraction of
    whichever bound is nearer)."""
    global _profile
    prof, _profile = _profile, None
    if prof is None:
        return []
    torch.cuda.synchronize()
    acc, prev = {}, prof.start
    for name, ev, work in prof.rows:
        r = acc.setdefault(name, {"kernel": name, "launches": 0, "ms": 0.0, "bytes": 0, "flops": 0.0, "known": 0})
        r["launches"] += 1
        r["ms"] += prev.elapsed_time(ev)
        if work is not None:
            r["bytes"] += work[0]
            r["flops"] += work[1]
            r["known"] += 1
        prev = ev
    total = sum(r["ms"] for r in acc.values()) or 1.0
    out = []
    for r in sorted(acc.values(), key=lambda r: -r["ms"]):
        row = {"kernel": r["kernel"], "launches": r["launches"], "ms": round(r["ms"], 3), "share": round(r["ms"] / total, 4),
               "us_per_launch": round(r["ms"] * 1e3 / r["launches"], 2)}
        if r["known"] == r["launches"] and r["ms"] > 0:
            row["GBps"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9, 1)
            row["TFLOPs"] = round(r["flops"] / (r["ms"] * 1e-3) / 1e12, 2)
            if peaks:
                row["frac_of_roofline"] = round(max(row["GBps"] / peaks["hbm_gbs"], row["TFLOPs"] / peaks["bf16_tflops"]), 4)
        out.append(row)
    return out


def _check(rc, name):
    global launches, _work
    if rc != 0:
        _work = None
        raise KernelError(f"{name}: {lib().ferrum_last_error().decode()}")
    launches += 1
    if _profile is not None:
        _profile.mark(name, _work)
    _work = None


def _gemm_work(x, w, out, M, N, K, products=1):
    """(bytes, flops) of a product for the profile: every weight once, the tokens and the result."""
    global _work
    if _profile is not None:
        _work = (products * N * K * w.element_size() + M * K * x.element_size() + M * N * out.element_size(),
                 2.0 * products * M * N * K)


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (the capture stream inside a graph capture)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name, ndim=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, found {t.dim()}")
    if t.dim() and t.stride(-1) != 1 and t.shape[-1] > 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


def _need16(t, name, ndim=None, like=None):
    """A CUDA tensor of a 16-bit float type (the same as `like`'s when given)."""
    _need(t, like.dtype if like is not None else None, name, ndim)
    if t.dtype not in SIXTEEN_BIT:
        raise KernelError(f"{name} must be bfloat16 or float16, found {t.dtype}")


def dtype_code(dtype):
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"unsupported compute dtype {dtype}") from None


# ----------------------------------------------------------------------------- ops
def embedding(table, ids, out, err):
    """out[t] = table[ids[t]] as float32."""
    _need(table, None, "table", 2); _need(ids, torch.int32, "ids", 1); _need(out, torch.float32, "out", 2)
    V, E = table.shape
    T = ids.shape[0]
    if out.shape[0] < T or out.shape[1] != E or not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embedding: out must be contiguous [>=T, E] and table contiguous")
    _check(lib().ferrum_embedding(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), c_int(T), c_int(E),
                                  c_int(V), _ptr(err), _stream()), "embedding")


class Partials:
    """A product that the tensor-core kernel left as float32 partials (see gemm_tc_deferred):
    the workspace that holds them and the four numbers a consumer needs to sum them."""

    def __init__(self, workspace, layout):
        self.workspace, self.layout = workspace, layout
        self._c = (c_int * 4)(*layout)


def rmsnorm(x, weight, out, eps, rows=None, n_rows=None, partials=None):
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight; x float32, out float32 or bfloat16.
    With `partials` (a deferred residual product) the rows of x first get the partials added,
    in place."""
    _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1); _need(out, None, "out", 2)
    E = x.shape[1]
    if n_rows is None:
        n_rows = rows.shape[0] if rows is not None else x.shape[0]
    if weight.shape[0] != E or out.shape[1] != E or out.shape[0] < n_rows or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("rmsnorm: shapes do not agree")
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    if partials is not None:
        _check(lib().ferrum_rmsnorm_reduce(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows),
                                           c_int(n_rows), c_int(E), c_float(eps), _ptr(partials.workspace), partials._c,
                                           _stream()), "rmsnorm_reduce")
        return
    _check(lib().ferrum_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), c_int(n_rows),
                                c_int(E), c_float(eps), _stream()), "rmsnorm")


def residual_reduce(h, n_rows, partials):
    """h[:n_rows] += the deferred product."""
    _need(h, torch.float32, "h", 2)
    _check(lib().ferrum_residual_reduce(_ptr(h), c_int(n_rows), c_int(h.shape[1]), _ptr(partials.workspace), partials._c,
                                        _stream()), "residual_reduce")


def swiglu_reduce(act, n_tokens, F, partials):
    """act[t, f] = silu(gate) * up from a deferred two-product launch."""
    _need16(act, "act", 2)
    _check(lib().ferrum_swiglu_reduce(_ptr(act), dtype_code(act.dtype), c_int(n_tokens), c_int(F), c_int(act.stride(0)), _ptr(partials.workspace),
                                      partials._c, _stream()), "swiglu_reduce")


@functools.lru_cache(maxsize=4096)
def gemm_tc_can_defer(M, N, K, dual):
    """(A pure function of the shape, asked for every product of every step: remembered.)"""
    return bool(lib().ferrum_gemm_tc_can_defer(c_int(M), c_int(N), c_int(K), c_int(1 if dual else 0), c_int(0)))


def gemm_tc_deferred(x, w, err, workspace, M=None, N=None, dual_offset=0, n_ctas=0):
    """The tensor-core product without its final reduction: returns `Partials` for the kernel
    that consumes the product.  Only for shapes that `gemm_tc_can_defer` accepts."""
    _need16(x, "x", 2); _need16(w, "w", 2, like=x); _need(workspace, torch.float32, "workspace")
    M = x.shape[0] if M is None else M
    K = w.shape[1]
    N = (w.shape[0] - dual_offset) if N is None else N
    if x.shape[1] != K or x.shape[0] < M:
        raise KernelError(f"gemm_tc_deferred: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)}")
    layout = (c_int * 4)()
    _gemm_work(x, w, workspace, M, N, K, 2 if dual_offset else 1)
    _check(lib().ferrum_gemm_tc_deferred(_ptr(x), _ptr(w), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K), c_int(x.stride(0)),
                                         c_int(w.stride(0)), c_int(w.shape[0]), c_int(dual_offset), c_int(n_ctas),
                                         _ptr(workspace), c_longlong(workspace.numel()), layout, _ptr(err), _stream()),
           "gemm_tc_deferred")
    return Partials(workspace, tuple(layout))


def gemm_generic(x, w, out, epilogue, M=None):
    """out[t, n] (=, or += for EPI_RESIDUAL) sum_k x[t, k] w[n, k]; CUDA cores, float32 accumulate."""
    _need(x, None, "x", 2); _need(w, x.dtype, "w", 2); _need(out, None, "out", 2)
    M = x.shape[0] if M is None else M
    N, K = w.shape
    if x.shape[1] != K or out.shape[1] < N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: out must be {want} for epilogue {epilogue}")
    _gemm_work(x, w, out, M, N, K)
    _check(lib().ferrum_gemm_generic(_ptr(x), _ptr(w), _ptr(out), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K),
                                     c_int(x.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue),
                                     _stream()), "gemm_generic")


def gemm_tc_supported(x, w):
    """True when the tcgen05 kernel takes these operands (one 16-bit type, 16-byte rows)."""
    return (x.dtype in SIXTEEN_BIT and w.dtype == x.dtype and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_token_tile(M, dual):
    return lib().ferrum_gemm_tc_token_tile(c_int(M), c_int(1 if dual else 0))


@functools.lru_cache(maxsize=4096)
def gemm_tc_workspace(M, N, K, dual, n_ctas=0):
    """(workspace floats, tile counters) that a launch needs."""
    tiles = c_int(0)
    need = lib().ferrum_gemm_tc_workspace(c_int(M), c_int(N), c_int(K), c_int(1 if dual else 0), c_int(n_ctas),
                                          ctypes.byref(tiles))
    return int(need), tiles.value


def gemm_tc(x, w, out, epilogue, err, workspace, counters, M=None, N=None, dual_offset=0, n_ctas=0):
    """16-bit (bfloat16 or float16) tensor-core product; see csrc/kernels/gemm_tc.cu.  `N` is the number of
    output features (rows of w used per product); with dual_offset > 0 rows dual_offset + n
    feed the second product of the SwiGLU epilogue.  `workspace` (float32) and `counters`
    (int32, all zero) are scratch for tiles that several CTAs share; n_ctas = 0 means one CTA
    per SM."""
    _need16(x, "x", 2); _need16(w, "w", 2, like=x); _need(out, None, "out", 2)
    M = x.shape[0] if M is None else M
    K = w.shape[1]
    N = (w.shape[0] - dual_offset) if N is None else N
    if x.shape[1] != K or out.shape[1] < N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"gemm_tc: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    want = x.dtype if epilogue in (TC_STORE_BF16, TC_SWIGLU) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: out must be {want} for epilogue {epilogue}")
    _need(workspace, torch.float32, "workspace")
    _need(counters, torch.int32, "counters")
    _gemm_work(x, w, out, M, N, K, 2 if dual_offset else 1)
    _check(lib().ferrum_gemm_tc(_ptr(x), _ptr(w), _ptr(out), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K), c_int(x.stride(0)),
                                c_int(w.stride(0)), c_int(out.stride(0)), c_int(w.shape[0]), c_int(epilogue),
                                c_int(dual_offset), c_int(n_ctas), _ptr(workspace), c_longlong(workspace.numel()),
                                _ptr(counters), c_int(counters.numel()), _ptr(err), _stream()), "gemm_tc")


def rope_cache_write(qkv, n_tokens, positions, req_of_token, block_table, cos_sin, kv_plane, page_stride, page_size,
                     Hq, Hkv, D, R, pairing, write_kv, err, partials=None):
    """Rotate q (in place) and k, store k and v into the paged cache plane.  With `partials`
    the q, k, v rows are first summed from a deferred product into `qkv`."""
    _need(qkv, None, "qkv", 2); _need(positions, torch.int32, "positions", 1)
    _need(req_of_token, torch.int32, "req_of_token", 1); _need(block_table, torch.int32, "block_table", 2)
    if R:
        _need(cos_sin, torch.float32, "cos_sin", 3)
        if cos_sin.shape[1] != R // 2 or cos_sin.shape[2] != 2 or not cos_sin.is_contiguous():
            raise KernelError("rope: cos_sin must be contiguous [positions, rope_dim/2, 2]")
    if write_kv:
        _need(kv_plane, qkv.dtype, "kv_plane")
    if not block_table.is_contiguous():
        raise KernelError("rope: block_table must be contiguous")
    _check(lib().ferrum_rope_cache_write(_ptr(qkv), dtype_code(qkv.dtype), c_int(n_tokens), c_int(qkv.stride(0)),
                                         _ptr(positions), _ptr(req_of_token), _ptr(block_table),
                                         c_int(block_table.shape[1]), _ptr(cos_sin if R else None),
                                         c_int(cos_sin.shape[0] if R else 0), _ptr(kv_plane if write_kv else None),
                                         c_longlong(page_stride), c_int(page_size), c_int(Hq), c_int(Hkv), c_int(D),
                                         c_int(R), c_int(pairing), c_int(1 if write_kv else 0), _ptr(err),
                                         _ptr(partials.workspace if partials is not None else None),
                                         partials._c if partials is not None else None, _stream()),
           "rope_cache_write")


def attention_generic_split():
    """Keys per split of the generic attention kernel's split mode."""
    return int(lib().ferrum_attention_generic_split())


def attention_generic(q, out, n_tokens, positions, req_of_token, block_table, kv_plane, page_stride, page_size, Hq,
                      Hkv, D, scale, window, err, part=None, split_slots=0, q_start=None, n_reqs=0):
    """Causal GQA attention of every token over its request's pages on the CUDA cores, float32
    arithmetic.  part=None: one CTA per (token, group of heads) walks the whole key range (many
    tokens).  With `part` (float32, n_tokens * Hq * split_slots * (D + 2) elements) every row's keys
    are cut at multiples of `attention_generic_split()` among split_slots CTAs and folded by a
    second launch (few tokens); split_slots must cover the longest row.  With q_start (the device's
    n_reqs + 1 token offsets of the requests, tokens of a request in ascending positions) and no
    `part`, up to eight tokens of a request that follow each other share every tile of keys."""
    _need(q, None, "q", 2); _need(out, q.dtype, "out", 2); _need(kv_plane, q.dtype, "kv_plane")
    _need(positions, torch.int32, "positions", 1); _need(req_of_token, torch.int32, "req_of_token", 1)
    _need(block_table, torch.int32, "block_table", 2)
    if not block_table.is_contiguous():
        raise KernelError("attention: block_table must be contiguous")
    if part is not None:
        _need(part, torch.float32, "part")
        if part.numel() < n_tokens * Hq * split_slots * (D + 2):
            raise KernelError("attention: the partials buffer is too small")
    _check(lib().ferrum_attention_generic(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)),
                                          dtype_code(q.dtype), c_int(n_tokens), _ptr(positions), _ptr(req_of_token),
                                          _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_plane),
                                          c_longlong(page_stride), c_int(page_size), c_int(Hq), c_int(Hkv), c_int(D),
                                          c_float(scale), c_int(window), _ptr(err), _ptr(part), c_int(split_slots),
                                          _ptr(q_start) if part is None else None, c_int(n_reqs), _stream()),
           "attention_generic")


def attention_flash_supported(dtype, D, page_stride=0):
    """True when the tensor-core attention kernel is built for this dtype and head size."""
    return dtype in SIXTEEN_BIT and bool(lib().ferrum_attention_flash_supported(c_int(D), c_int(16)))


def attention_flash(q, out, kv_plane, page_stride, page_size, block_table, q_start, pos0, work, n_work, part_o,
                    part_ml, Hq, Hkv, D, scale, window, bm, err, cta_items=None, n_ctas=0, trigger_early=False):
    """Tensor-core attention over the work items of one row-tile class (bm 16 or 64).
    trigger_early: the kernels that follow in the stream may start while this one runs."""
    _need16(q, "q", 2); _need16(out, "out", 2, like=q); _need16(kv_plane, "kv_plane", like=q)
    _need(block_table, torch.int32, "block_table", 2); _need(work, torch.int32, "work", 1)
    _check(lib().ferrum_attention_flash(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), dtype_code(q.dtype),
                                        _ptr(kv_plane),
                                        c_longlong(page_stride), c_int(page_size), _ptr(block_table),
                                        c_int(block_table.shape[1]), _ptr(q_start), _ptr(pos0), _ptr(work),
                                        c_int(n_work), _ptr(cta_items), c_int(n_ctas), _ptr(part_o), _ptr(part_ml),
                                        c_int(Hq), c_int(Hkv), c_int(D),
                                        c_float(scale), c_int(window), c_int(bm), c_int(1 if trigger_early else 0),
                                        _ptr(err), _stream()), "attention_flash")


def attention_tc_tokens(D, G, page_size, kv_plane=None, page_stride=0):
    """Tokens per work item of the tcgen05 attention kernel for this head size, group size and
    page size (an item has that many tokens x G rows); 0 where the kernel does not apply (other
    sizes, float32, pages that are not dense in the plane)."""
    if kv_plane is not None and (kv_plane.dtype not in SIXTEEN_BIT or kv_plane.dim() != 5 or
                                 page_stride != kv_plane[0].numel()):
        return 0
    return int(lib().ferrum_attention_tc_tokens(c_int(D), c_int(G), c_int(page_size)))


def set_attention_pair_kernel(on: bool):
    """Head size 128 runs the tcgen05 attention on CTA pairs (on by default); off: the single-CTA
    kernel takes the same work items (for comparisons)."""
    lib().ferrum_set_attention_pair_kernel(c_int(1 if on else 0))


def attention_tc(q, out, kv_plane, page_stride, page_size, block_table, q_start, pos0, work, n_work, part_o, part_ml,
                 Hq, Hkv, D, scale, window, err):
    """tcgen05 attention over work items of attention_tc_tokens * G rows (prompt portions)."""
    _need16(q, "q", 2); _need16(out, "out", 2, like=q); _need16(kv_plane, "kv_plane", like=q)
    _need(block_table, torch.int32, "block_table", 2); _need(work, torch.int32, "work", 1)
    _check(lib().ferrum_attention_tc(_ptr(q), c_int(q.stride(0)), c_longlong(q.shape[0]), _ptr(out), c_int(out.stride(0)),
                                     dtype_code(q.dtype), _ptr(kv_plane), c_longlong(page_stride), c_longlong(kv_plane.shape[0]),
                                     c_int(page_size), _ptr(block_table), c_int(block_table.shape[1]), _ptr(q_start),
                                     _ptr(pos0), _ptr(work), c_int(n_work), _ptr(part_o), _ptr(part_ml), c_int(Hq),
                                     c_int(Hkv), c_int(D), c_float(scale), c_int(window), _ptr(err), _stream()),
           "attention_tc")


def attention_combine(out, part_o, part_ml, q_start, req_of_token, req_tile0, tile_info, token_list, n_tokens, Hq, Hkv,
                      D, bm, n_warps=1):
    """Merges the key-range splits written by attention_flash into `out`.  n_warps (1..8): warps
    per (token, head) that share its splits; more than one pays from about 16 splits on."""
    _need16(out, "out", 2)
    _check(lib().ferrum_attention_combine(_ptr(out), c_int(out.stride(0)), dtype_code(out.dtype), _ptr(part_o), _ptr(part_ml), _ptr(q_start),
                                          _ptr(req_of_token), _ptr(req_tile0), _ptr(tile_info), _ptr(token_list),
                                          c_int(n_tokens), c_int(Hq), c_int(Hkv), c_int(D), c_int(bm), c_int(n_warps), _stream()),
           "attention_combine")


def swiglu(gu, act, n_tokens, F):
    """act[t, f] = silu(gu[t, f]) * gu[t, F + f]."""
    _need(gu, None, "gu", 2); _need(act, gu.dtype, "act", 2)
    _check(lib().ferrum_swiglu(_ptr(gu), _ptr(act), dtype_code(gu.dtype), c_int(n_tokens), c_int(F),
                               c_int(gu.stride(0)), c_int(act.stride(0)), _stream()), "swiglu")


def sample(logits, n_rows, out_ids, err, inv_temperature=None, seeds=None, counters=None, also_to=None):
    """out_ids[r] = argmax, or the Gumbel-max draw where inv_temperature[r] != 0.  `also_to`
    (int32) receives the ids as well."""
    _need(logits, torch.float32, "logits", 2); _need(out_ids, torch.int32, "out_ids", 1)
    if inv_temperature is not None:
        _need(inv_temperature, torch.float32, "inv_temperature", 1)
        _need(seeds, torch.int64, "seeds", 1); _need(counters, torch.int32, "counters", 1)
    _check(lib().ferrum_sample(_ptr(logits), c_int(logits.stride(0)), c_int(n_rows), c_int(logits.shape[1]),
                               _ptr(inv_temperature), _ptr(seeds), _ptr(counters), _ptr(out_ids), _ptr(also_to),
                               _ptr(err), _stream()), "sample")
