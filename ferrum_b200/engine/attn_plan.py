"""Work lists of the tensor-core attention kernel for one step.

Every request's rows (tokens x query heads of one KV group) are cut into tiles, and a
tile's key range may be cut into splits so that a step with few requests and long contexts
still fills the GPU.  The plan depends on the batch (lengths, positions), on the group size
G = Hq / Hkv and on the window, not on the layer, so it is built once per step and used by
every layer with the same (G, window).

Requests with at most 16 rows (decoded tokens) go to the 16-row kernel, the others to the
64-row kernel; each class has its own work list.  A work item is
[request, first row, key begin, key end, number of splits, partial slot, 0, 0].
Split boundaries are multiples of 64 keys counted from the tile's first key, and the splits
are merged in order, so a row's result does not depend on the other requests in the batch
beyond the choice of the split length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

N_SMS = 148
CLASSES = (16, 64)
MIN_SPLIT_KEYS = {16: 256, 64: 1024}


@dataclass
class ClassPlan:
    bm: int
    n_work: int = 0
    work: Optional[torch.Tensor] = None        # int32 [n_work * 8]
    n_slots: int = 0                            # partial slots (work items that are splits)
    req_tile0: Optional[torch.Tensor] = None
    tile_info: Optional[torch.Tensor] = None
    comb_tokens: Optional[torch.Tensor] = None
    n_comb: int = 0


def build_host(q_len, pos0, G, window, Hkv):
    """numpy description of both classes: list of dicts with int32 arrays."""
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
        # enough work items to fill the GPU about twice over, never splits shorter than the minimum
        target = max(1, (2 * N_SMS + Hkv - 1) // Hkv)
        chunk = int(max(MIN_SPLIT_KEYS[bm], -(-int(length.sum()) // target)))
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
        first_slot = np.where(n_splits > 1, np.cumsum(np.where(n_splits > 1, n_splits, 0)) - np.where(n_splits > 1, n_splits, 0), 0)
        tile_info = np.stack([first_slot, n_splits], axis=1).astype(np.int32)
        req_tile0 = np.zeros(R, dtype=np.int32)
        req_tile0[sel] = (np.cumsum(n_tiles) - n_tiles).astype(np.int32)
        split_reqs = np.unique(req_of_tile[n_splits > 1])
        comb = np.concatenate([np.arange(q_start[r], q_start[r + 1]) for r in split_reqs]).astype(np.int32) \
            if len(split_reqs) else np.zeros(0, dtype=np.int32)
        out.append({"bm": bm, "work": work[order].reshape(-1), "n_work": T, "n_slots": int(is_split.sum()),
                    "tile_info": tile_info.reshape(-1), "req_tile0": req_tile0, "comb": comb})
    return out


class AttentionPlans:
    """Per-step cache of plans, keyed by (G, window, Hkv); owns the device copies."""

    def __init__(self, device):
        self.device = device
        self._plans = {}
        self._host = None
        self._dev = None

    def reset(self):
        self._plans = {}

    def get(self, ctx, G, window, Hkv) -> List[Optional[ClassPlan]]:
        key = (G, window, Hkv)
        if key in self._plans:
            return self._plans[key]
        host = build_host(ctx.h_q_len, ctx.h_pos0, G, window, Hkv)
        arrays = []
        for h in host:
            if h is not None:
                arrays += [h["work"], h["tile_info"], h["req_tile0"], h["comb"]]
        total = sum(a.size for a in arrays)
        pinned = torch.empty(max(total, 1), dtype=torch.int32).pin_memory()
        dev = torch.empty(max(total, 1), dtype=torch.int32, device=self.device)
        np.concatenate(arrays, out=pinned.numpy()[:total]) if arrays else None
        dev[:total].copy_(pinned[:total], non_blocking=True)
        ctx.h2d_bytes += total * 4
        self._keep = getattr(self, "_keep", []) + [pinned]      # alive until the copy has run
        if len(self._keep) > 8:
            self._keep = self._keep[-8:]
        plans, o = [], 0
        for h in host:
            if h is None:
                plans.append(None)
                continue
            def take(a):
                nonlocal o
                v = dev[o:o + a.size]
                o += a.size
                return v
            cp = ClassPlan(h["bm"], h["n_work"], take(h["work"]), h["n_slots"])
            cp.tile_info, cp.req_tile0, cp.comb_tokens = take(h["tile_info"]), take(h["req_tile0"]), take(h["comb"])
            cp.n_comb = int(h["comb"].size)
            plans.append(cp)
        self._plans[key] = plans
        return plans
