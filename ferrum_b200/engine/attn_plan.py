"""Work lists of the tensor-core attention kernel for one step.

Every request's rows (tokens x query heads of one KV group) are cut into tiles, and a
tile's key range may be cut into splits so that a step with few requests and long contexts
still fills the GPU.  The plan depends on the batch (lengths, positions), on the group size
G = Hq / Hkv and on the window, not on the layer, so it is built once per step and used by
every layer with the same (G, window).

Requests with at most 16 rows (decoded tokens) go to the 16-row kernel, the others to the
64-row kernel; each class has its own work list.  A work item is
[request, first row, key begin, key end, number of splits, partial slot, 0, 0]; an item with
zero splits is padding.  Split boundaries are multiples of 64 keys counted from the tile's
first key, and the splits are merged in order, so a row's result does not depend on the
other requests in the batch beyond the choice of the split length.

The lists live in device buffers that keep their address from step to step, and a plan can
be padded to a fixed number of items, so that a captured CUDA graph can be replayed with the
next step's lists.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

N_SMS = 148
CLASSES = (16, 64)
MIN_SPLIT_KEYS = {16: 256, 64: 1024}


def target_items(Hkv):
    """Work items per class that fill the GPU once at two CTAs per SM."""
    return max(1, (2 * N_SMS) // Hkv)


def item_capacity(n_requests, Hkv):
    """Upper bound of the 16-row class's work items for n_requests decoded tokens."""
    return target_items(Hkv) + 2 * n_requests


def build_host(q_len, pos0, G, window, Hkv):
    """numpy description of both classes: None or a dict of int32 arrays per class."""
    q_len = np.asarray(q_len, dtype=np.int64)
    pos0 = np.asarray(pos0, dtype=np.int64)
    R = len(q_len)
    rows = q_len * G
    q_start = np.concatenate([[0], np.cumsum(q_len)])
    out = []
    for bm in CLASSES:
        sel = np.nonzero((rows <= 16) if bm == 16 else (rows > 16))[0]
        if len(sel) == 0:
            out.append(None)
            continue
        n_tiles = (rows[sel] + bm - 1) // bm
        req_of_tile = np.repeat(sel, n_tiles)
        tile_in_req = np.arange(n_tiles.sum()) - np.repeat(np.cumsum(n_tiles) - n_tiles, n_tiles)
        row0 = tile_in_req * bm
        first_tok = row0 // G
        last_tok = np.minimum(q_len[req_of_tile] - 1, (row0 + bm - 1) // G)
        hi = pos0[req_of_tile] + last_tok + 1
        lo = np.maximum(0, pos0[req_of_tile] + first_tok - window + 1) if window > 0 else np.zeros_like(hi)
        length = hi - lo
        # about one item per CTA slot of the GPU, never splits shorter than the minimum
        chunk = int(max(MIN_SPLIT_KEYS[bm], -(-int(length.sum()) // target_items(Hkv))))
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
        # per tile: first partial slot and number of splits (slots of a tile are consecutive)
        split_sizes = np.where(n_splits > 1, n_splits, 0)
        first_slot = np.where(n_splits > 1, np.cumsum(split_sizes) - split_sizes, 0)
        tile_info = np.stack([first_slot, n_splits], axis=1).astype(np.int32)
        req_tile0 = np.zeros(R, dtype=np.int32)
        req_tile0[sel] = (np.cumsum(n_tiles) - n_tiles).astype(np.int32)
        split_reqs = np.unique(req_of_tile[n_splits > 1])
        comb = np.concatenate([np.arange(q_start[r], q_start[r + 1]) for r in split_reqs]).astype(np.int32) \
            if len(split_reqs) else np.zeros(0, dtype=np.int32)
        out.append({"bm": bm, "work": work[order].reshape(-1), "n_work": T, "n_slots": int(is_split.sum()),
                    "tile_info": tile_info.reshape(-1), "req_tile0": req_tile0, "comb": comb})
    return out


@dataclass
class ClassPlan:
    bm: int
    n_work: int = 0                             # grid size (includes padding items)
    work: Optional[torch.Tensor] = None        # int32 [n_work * 8]
    n_slots: int = 0                            # partial slots to provide
    req_tile0: Optional[torch.Tensor] = None
    tile_info: Optional[torch.Tensor] = None
    comb_tokens: Optional[torch.Tensor] = None  # None: every token of the batch
    n_comb: int = 0


class AttentionPlans:
    """Per-step cache of plans, keyed by (G, window, Hkv); owns the device copies."""

    def __init__(self, device):
        self.device = device
        self._plans = {}
        self._bufs = {}          # key -> (pinned, device) int32 buffers, grow-only
        self.generation = 0      # bumped whenever a device buffer moves

    def reset(self):
        self._plans = {}

    def keys_built(self):
        return list(self._plans)

    def _buffers(self, key, n):
        from .batch import PinnedRing
        b = self._bufs.get(key)
        if b is None or b[1].numel() < n:
            cap = max(1024, 2 * n)
            b = (PinnedRing(cap, torch.int32, self.device), torch.empty(cap, dtype=torch.int32, device=self.device))
            self._bufs[key] = b
            self.generation += 1
        return b

    def get(self, ctx, G, window, Hkv, fixed=False) -> List[Optional[ClassPlan]]:
        """fixed=True (a decode-only batch under a CUDA graph): the 16-row list is padded to
        `item_capacity` items and the merge visits every token, so that the launch shapes
        depend on the number of requests only."""
        key = (G, window, Hkv)
        if key in self._plans:
            return self._plans[key]
        host = build_host(ctx.h_q_len, ctx.h_pos0, G, window, Hkv)
        R = len(ctx.h_q_len)
        if fixed:
            h = host[0]
            if h is None or host[1] is not None:
                raise ValueError("a fixed-shape plan needs a batch of decoded tokens only")
            cap = item_capacity(R, Hkv)
            if h["n_work"] > cap:
                raise ValueError("attention plan exceeds its fixed capacity")
            padded = np.zeros(cap * 8, dtype=np.int32)
            padded[:h["work"].size] = h["work"]
            h["work"], h["n_work"], h["n_slots"] = padded, cap, cap
        arrays = []
        for h in host:
            if h is not None:
                arrays += [h["work"], h["tile_info"], h["req_tile0"], h["comb"]]
        total = sum(a.size for a in arrays)
        ring, dev = self._buffers(key, total)
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
            for name in ("work", "tile_info", "req_tile0", "comb"):
                views.append(dev[o:o + h[name].size])
                o += h[name].size
            cp = ClassPlan(h["bm"], h["n_work"], views[0], h["n_slots"])
            cp.tile_info, cp.req_tile0 = views[1], views[2]
            if fixed:
                cp.comb_tokens, cp.n_comb = None, ctx.n_tokens
            else:
                cp.comb_tokens, cp.n_comb = views[3], int(h["comb"].size)
            plans.append(cp)
        self._plans[key] = plans
        return plans
