"""Work lists of the tensor-core attention kernels for one step: the planner that the
attention mixer brings with it (`PagedAttention.plan`).  The engine knows nothing of it: a
step's context only offers a per-step cache and buffers that keep their addresses
(`StepContext.step_cache`, `StepContext.plan_store`).

Every request's rows (tokens x query heads of one KV group) are cut into tiles, and a
tile's key range may be cut into splits so that a step with few requests and long contexts
still fills the GPU.  The plan depends on the batch (lengths, positions), on the group size
G = Hq / Hkv and on the window, not on the layer, so it is built once per step and used by
every layer with the same (G, window).

Requests with at most 16 rows (decoded tokens) go to the 16-row kernel, requests with at
least TC_MIN_ROWS rows to the tcgen05 kernel where it takes the layer's shape (its items are
one or two 128-row tiles), the others to the 64-row kernel; each class has its own work list.  A work item is
[request, first row, key begin, key end, number of splits, partial slot, KV head, 0]; an item
with zero splits is padding.  The 64-row class runs a grid of (items, KV heads).  The 16-row
class runs a balanced list: every CTA slot of the GPU gets an equal share of all (request,
head, 64-key tile) units.  Split boundaries are multiples of 64 keys counted from the tile's
first key and the splits are merged in key order; where they fall depends on the batch, so a
row's bfloat16 result may differ between batches by rounding, never by more.

The lists live in device buffers that keep their address from step to step, and a plan can
be padded to a fixed number of items, so that a captured CUDA graph can be replayed with the
next step's lists.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

CLASSES = (16, 64)
MIN_SPLIT_KEYS = {16: 256, 64: 1024}
TC_MIN_ROWS = 128           # a request with fewer rows would leave the 128-row tiles mostly empty
TC_MIN_SPLIT_KEYS = 2048


CTAS_PER_SM = 3             # the 16-row kernel keeps three CTAs on an SM (registers and shared memory)
_slots = {}


def sm_count():
    """Multiprocessors of the current device, asked of the kernel library once per device."""
    from ..ops import lib as ops
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if dev not in _slots:
        _slots[dev] = ops.sm_count() if dev >= 0 else 148
    return _slots[dev]


def cta_slots():
    """CTAs of the 16-row kernel that the device holds at once."""
    return CTAS_PER_SM * sm_count()


# A share may be a single 64-key tile: with few requests or short contexts more CTAs beat
# longer shares (batch 1, 8192 keys: 3.68 -> 3.55 ms a step; 1024 keys: 3.66 -> 3.39), now that
# the merge kernel spreads a pair's splits over several warps.
MIN_TILES_PER_CTA = 1


def item_capacity(n_requests, Hkv):
    """Upper bound of the balanced list's items: one per CTA slot plus one per (request, head)."""
    return cta_slots() + n_requests * Hkv


def _tiles(q_len, pos0, G, window, bm, sel):
    """Row tiles of the selected requests: (request, first row, first key, end key) per tile."""
    rows = q_len * G
    n_tiles = (rows[sel] + bm - 1) // bm
    req_of_tile = np.repeat(sel, n_tiles)
    tile_in_req = np.arange(n_tiles.sum()) - np.repeat(np.cumsum(n_tiles) - n_tiles, n_tiles)
    row0 = tile_in_req * bm
    first_tok = row0 // G
    last_tok = np.minimum(q_len[req_of_tile] - 1, (row0 + bm - 1) // G)
    hi = pos0[req_of_tile] + last_tok + 1
    lo = np.maximum(0, pos0[req_of_tile] + first_tok - window + 1) if window > 0 else np.zeros_like(hi)
    return n_tiles, req_of_tile, row0, lo, hi


def _grid_class(q_len, pos0, G, window, Hkv, bm, sel, R, q_start, slots=None, min_split=None, kind="flash"):
    """One item per (tile, key split); the kernel runs it once per KV head."""
    n_tiles, req_of_tile, row0, lo, hi = _tiles(q_len, pos0, G, window, bm, sel)
    length = hi - lo
    slots = cta_slots() if slots is None else slots
    # about one item per CTA slot of the GPU, never splits shorter than the minimum
    min_split = MIN_SPLIT_KEYS[bm] if min_split is None else min_split
    chunk = int(max(min_split, -(-int(length.sum()) // max(1, slots // Hkv))))
    chunk = (chunk + 63) // 64 * 64
    n_splits = np.maximum(1, (length + chunk - 1) // chunk)
    T = int(n_splits.sum())
    tile_of_work = np.repeat(np.arange(len(req_of_tile)), n_splits)
    split_idx = np.arange(T) - np.repeat(np.cumsum(n_splits) - n_splits, n_splits)
    kb = lo[tile_of_work] + split_idx * chunk
    ke = np.minimum(hi[tile_of_work], kb + chunk)
    ns = n_splits[tile_of_work]
    is_split = ns > 1
    slot = np.where(is_split, np.cumsum(is_split) - 1, -1)
    work = np.zeros((T, 8), dtype=np.int32)
    work[:, 0], work[:, 1], work[:, 2], work[:, 3] = req_of_tile[tile_of_work], row0[tile_of_work], kb, ke
    work[:, 4], work[:, 5] = ns, slot
    order = np.argsort(-(ke - kb), kind="stable")          # long items first
    # per (tile, head): first partial slot, number of splits, slot stride.  The kernel gives
    # item s of head h the slot (first item slot + s) * Hkv + h.
    split_sizes = np.where(n_splits > 1, n_splits, 0)
    first_slot = np.cumsum(split_sizes) - split_sizes
    info = np.zeros((len(req_of_tile), Hkv, 4), dtype=np.int32)
    info[:, :, 0] = first_slot[:, None] * Hkv + np.arange(Hkv)[None, :]
    info[:, :, 1] = n_splits[:, None]
    info[:, :, 2] = Hkv
    req_tile0 = np.zeros(R, dtype=np.int32)
    req_tile0[sel] = (np.cumsum(n_tiles) - n_tiles).astype(np.int32)
    split_reqs = np.unique(req_of_tile[n_splits > 1])
    comb = np.concatenate([np.arange(q_start[r], q_start[r + 1]) for r in split_reqs]).astype(np.int32) \
        if len(split_reqs) else np.zeros(0, dtype=np.int32)
    return {"bm": bm, "kind": kind, "work": work[order].reshape(-1), "n_work": T, "n_slots": int(is_split.sum()) * Hkv,
            "tile_info": info.reshape(-1), "req_tile0": req_tile0, "comb": comb,
            "cta_items": np.zeros(0, dtype=np.int32), "n_ctas": 0}


def _balanced_class(q_len, pos0, G, window, Hkv, bm, sel, R, q_start):
    """Requests with one row tile each (decoded tokens).  All (request, head, 64-key tile)
    units form one line; CTA slot c owns units [c*U/P, (c+1)*U/P); a share is cut into items
    at (request, head) borders."""
    n_tiles, req_of_tile, row0, lo, hi = _tiles(q_len, pos0, G, window, bm, sel)
    assert (n_tiles == 1).all()
    n_req = len(sel)
    kt = np.maximum(1, (hi - lo + 63) // 64)                       # key tiles per request
    pair_tiles = np.repeat(kt, Hkv)                                 # pairs in (request, head) order
    pair_start = np.concatenate([[0], np.cumsum(pair_tiles)])
    U = int(pair_start[-1])
    P = int(min(cta_slots(), max(1, U // MIN_TILES_PER_CTA)))     # no share shorter than a few tiles
    bounds = (np.arange(P + 1, dtype=np.int64) * U) // P
    cuts = np.unique(np.concatenate([pair_start, bounds]))
    seg_b, seg_e = cuts[:-1], cuts[1:]
    pair = np.searchsorted(pair_start, seg_b, side="right") - 1
    r_idx, head = pair // Hkv, pair % Hkv
    t0, t1 = seg_b - pair_start[pair], seg_e - pair_start[pair]
    kb = lo[r_idx] + t0 * 64
    ke = np.minimum(hi[r_idx], lo[r_idx] + t1 * 64)
    per_pair = np.bincount(pair, minlength=n_req * Hkv)
    ns = per_pair[pair]
    is_split = ns > 1
    slot = np.where(is_split, np.cumsum(is_split) - 1, -1)
    n_seg = len(seg_b)
    work = np.zeros((n_seg, 8), dtype=np.int32)
    work[:, 0], work[:, 1], work[:, 2], work[:, 3] = sel[r_idx], 0, kb, ke
    work[:, 4], work[:, 5], work[:, 6] = ns, slot, head
    cta_items = np.searchsorted(seg_b, bounds[:-1], side="left").astype(np.int32)
    cta_items = np.concatenate([cta_items, [n_seg]]).astype(np.int32)
    split_sizes = np.where(per_pair > 1, per_pair, 0)
    first_slot = np.cumsum(split_sizes) - split_sizes              # a pair's items are consecutive
    info = np.zeros((n_req * Hkv, 4), dtype=np.int32)
    info[:, 0], info[:, 1], info[:, 2] = first_slot, per_pair, 1
    req_tile0 = np.zeros(R, dtype=np.int32)
    req_tile0[sel] = np.arange(n_req, dtype=np.int32)
    split_reqs = np.unique(r_idx[is_split])
    comb = np.concatenate([np.arange(q_start[sel[r]], q_start[sel[r] + 1]) for r in split_reqs]).astype(np.int32) \
        if len(split_reqs) else np.zeros(0, dtype=np.int32)
    return {"bm": bm, "kind": "flash", "work": work.reshape(-1), "n_work": n_seg, "n_slots": int(is_split.sum()),
            "tile_info": info.reshape(-1), "req_tile0": req_tile0, "comb": comb, "cta_items": cta_items, "n_ctas": P}


def build_host(q_len, pos0, G, window, Hkv, tc_tokens=0):
    """numpy description of the classes (16 rows, 64 rows, tcgen05 tile pairs): None or a dict
    of int32 arrays per class.  tc_tokens: tokens per work item of the tcgen05 kernel, 0
    where it does not take the layer's shape."""
    q_len = np.asarray(q_len, dtype=np.int64)
    pos0 = np.asarray(pos0, dtype=np.int64)
    R = len(q_len)
    rows = q_len * G
    q_start = np.concatenate([[0], np.cumsum(q_len)])
    to_tc = (rows >= TC_MIN_ROWS) if tc_tokens > 0 else np.zeros(R, dtype=bool)
    out = []
    for bm in CLASSES:
        sel = np.nonzero((rows <= 16) if bm == 16 else ((rows > 16) & ~to_tc))[0]
        if len(sel) == 0:
            out.append(None)
        elif bm == 16:
            out.append(_balanced_class(q_len, pos0, G, window, Hkv, bm, sel, R, q_start))
        else:
            out.append(_grid_class(q_len, pos0, G, window, Hkv, bm, sel, R, q_start))
    sel = np.nonzero(to_tc)[0]
    out.append(_grid_class(q_len, pos0, G, window, Hkv, tc_tokens * G, sel, R, q_start, slots=sm_count(),
                           min_split=TC_MIN_SPLIT_KEYS, kind="tc") if len(sel) else None)
    return out


@dataclass
class ClassPlan:
    bm: int                                     # rows per item
    n_work: int = 0                             # grid size (includes padding items)
    work: Optional[torch.Tensor] = None        # int32 [n_work * 8]
    n_slots: int = 0                            # partial slots to provide
    req_tile0: Optional[torch.Tensor] = None
    tile_info: Optional[torch.Tensor] = None
    comb_tokens: Optional[torch.Tensor] = None  # None: every token of the batch
    n_comb: int = 0
    cta_items: Optional[torch.Tensor] = None    # balanced list: first item of every CTA (+ end)
    n_ctas: int = 0
    kind: str = "flash"                         # "flash": the mma.sync kernel; "tc": the tcgen05 kernel
    comb_warps: int = 1                         # warps per (token, head) of the merge kernel


def _decode_plans(ctx, key, G, window, Hkv, fixed):
    """Every request brings one row tile: the balanced list, built by the native module
    straight into the pinned staging buffer."""
    from .. import host as host_module
    R = len(ctx.h_q_len)
    slots = cta_slots()
    cap = item_capacity(R, Hkv)
    total = cap * 8 + R * Hkv * 4 + R + slots + 1
    ring, dev = ctx.plan_store.buffers(("attention", key), total)
    pinned = ring.next()
    hi = [p + n for p, n in zip(ctx.h_pos0, ctx.h_q_len)]
    lo = [max(0, p - window + 1) for p in ctx.h_pos0] if window > 0 else [0] * R
    d = host_module.module().build_decode_plan(lo, hi, Hkv, slots, MIN_TILES_PER_CTA, cap, slots, bool(fixed),
                                               pinned.data_ptr())
    dev[:total].copy_(pinned[:total], non_blocking=True)
    ring.sent()
    ctx.h2d_bytes += total * 4
    o1 = cap * 8
    o2 = o1 + R * Hkv * 4
    o3 = o2 + R
    cp = ClassPlan(16, cap if fixed else d.n_items, dev[:o1], cap if fixed else d.n_slots)
    cp.tile_info, cp.req_tile0 = dev[o1:o2], dev[o2:o3]
    cp.cta_items, cp.n_ctas = dev[o3:total], slots if fixed else d.n_ctas
    # the merge visits every token; those whose keys were not split return at once
    cp.comb_tokens, cp.n_comb = None, (ctx.n_tokens if (fixed or d.n_slots) else 0)
    # a (request, KV head) gets about slots / (R * Hkv) splits; one warp takes eight at a time
    cp.comb_warps = int(min(8, max(1, -(-slots // (R * Hkv * 8)))))
    return [cp, None, None]


def plans_for(ctx, G, window, Hkv, tc_tokens=0) -> List[Optional[ClassPlan]]:
    """The step's plans for a layer shape (group size, window, KV heads, tokens per tcgen05 tile;
    0 where that kernel does not apply), one per row-tile class; built on first use in a step and
    kept in `ctx.step_cache`, so that every layer of the same shape shares them.

    While `ctx.fixed_shapes` is set (a decode-only batch that runs under a CUDA graph) the
    16-row list is padded to `item_capacity` items and the merge visits every token, so that the
    launch shapes depend on the number of requests only; such a batch must consist of requests
    with at most 16 rows each (`graph_safe` of the mixer says whether its shape allows that)."""
    key = (G, window, Hkv, tc_tokens)
    cache_key = ("attention", key)
    if cache_key in ctx.step_cache:
        return ctx.step_cache[cache_key]
    fixed = ctx.fixed_shapes
    if max(ctx.h_q_len) * G <= 16:
        plans = _decode_plans(ctx, key, G, window, Hkv, fixed)     # native fast path
        ctx.step_cache[cache_key] = plans
        return plans
    if fixed:
        raise ValueError("a fixed-shape plan needs requests of at most 16 rows (one decoded token, group size <= 16)")
    host = build_host(ctx.h_q_len, ctx.h_pos0, G, window, Hkv, tc_tokens)
    arrays = []
    for h in host:
        if h is not None:
            arrays += [h["work"], h["tile_info"], h["req_tile0"], h["comb"], h["cta_items"]]
    total = sum(a.size for a in arrays)
    ring, dev = ctx.plan_store.buffers(cache_key, total)
    pinned = ring.next()
    if arrays:
        np.concatenate(arrays, out=pinned.numpy()[:total])
    dev[:total].copy_(pinned[:total], non_blocking=True)
    ring.sent()
    ctx.h2d_bytes += total * 4
    plans, o = [], 0
    for h in host:
        if h is None:
            plans.append(None)
            continue
        views = []
        for name in ("work", "tile_info", "req_tile0", "comb", "cta_items"):
            views.append(dev[o:o + h[name].size])
            o += h[name].size
        cp = ClassPlan(h["bm"], h["n_work"], views[0], h["n_slots"])
        cp.kind = h["kind"]
        cp.tile_info, cp.req_tile0 = views[1], views[2]
        if h["n_ctas"]:
            cp.cta_items, cp.n_ctas = views[4], h["n_ctas"]
        cp.comb_tokens, cp.n_comb = views[3], int(h["comb"].size)
        plans.append(cp)
    ctx.step_cache[cache_key] = plans
    return plans
