"""Device memory of the cache, laid out for the groups the model's layers form.

`CacheLayout` reads a model's schedule: runs whose mixers keep paged keys/values with the
same (kv heads, head size, window) form a group; each writing run gets a plane of its own in
the group's pool, a run with `cache_of` shares the plane of the run it names.  Runs whose
mixers keep a fixed-size state get a state array [max_requests, ...] indexed by slot id.

`CacheStorage` allocates one pool per group, [planes, pages, 2 (K, V), kv heads, page_size,
head size] in the compute dtype, the state arrays, and the native `CacheManager` that owns
the page and slot numbers.  Page size and page counts are parameters (the pool is sized for
the tokens the caller wants resident, or for a fraction of the free HBM).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import host


@dataclass
class LayerCache:
    """What one run of a layer may touch."""
    group: Optional[int]            # index into ctx.block_tables, None when the mixer keeps no pages
    plane: Optional[torch.Tensor]   # [pages, 2, Hkv, page_size, D]
    page_stride: int                # elements from one page to the next
    page_size: int
    writes: bool                    # False: reads the plane another run wrote
    state: Optional[torch.Tensor]   # [max_requests, ...] or None


class CacheLayout:
    def __init__(self, model):
        self.needs = model.cache_needs()
        self.schedule = model.schedule
        self.group_keys: List[tuple] = []
        self.group_planes: List[int] = []
        self.run_group: List[Optional[int]] = []
        self.run_plane: List[Optional[int]] = []
        self.run_state: List[Optional[int]] = []
        self.state_needs = []
        for k, (run, need) in enumerate(zip(self.schedule, self.needs)):
            if run.cache_of is not None:
                j = run.cache_of
                if (need.paged is None) != (self.needs[j].paged is None) or (
                        need.paged is not None and need.paged != self.needs[j].paged):
                    raise ValueError(f"run {k} cannot read the cache of run {j}: their needs differ")
                self.run_group.append(self.run_group[j])
                self.run_plane.append(self.run_plane[j])
                self.run_state.append(self.run_state[j])
                continue
            if need.paged is not None:
                key = (need.paged.n_kv_heads, need.paged.head_dim, need.paged.window)
                if key not in self.group_keys:
                    self.group_keys.append(key)
                    self.group_planes.append(0)
                g = self.group_keys.index(key)
                self.run_group.append(g)
                self.run_plane.append(self.group_planes[g])
                self.group_planes[g] += 1
            else:
                self.run_group.append(None)
                self.run_plane.append(None)
            if need.state is not None:
                self.run_state.append(len(self.state_needs))
                self.state_needs.append(need.state)
            else:
                self.run_state.append(None)

    def bytes_per_token(self, dtype) -> int:
        size = torch.empty((), dtype=dtype).element_size()
        return sum(2 * h * d * planes * size for (h, d, _), planes in zip(self.group_keys, self.group_planes))


class CacheStorage:
    def __init__(self, model, dtype, device, page_size=16, num_pages=None, max_requests=64, max_model_len=None,
                 max_tokens=None):
        """num_pages: pages per group (int or list); or max_tokens: tokens to keep resident,
        from which the page count follows (every group gets enough pages for them)."""
        self.layout = CacheLayout(model)
        self.dtype, self.device, self.page_size = dtype, device, int(page_size)
        n_groups = len(self.layout.group_keys)
        max_model_len = int(max_model_len or 4096)
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("give num_pages or max_tokens")
            num_pages = (int(max_tokens) + self.page_size - 1) // self.page_size
        pages = list(num_pages) if isinstance(num_pages, (list, tuple)) else [int(num_pages)] * n_groups
        self.table_width = (max_model_len + self.page_size - 1) // self.page_size
        specs = [host.module().GroupSpec(self.page_size, key[2], pages[g], self.table_width)
                 for g, key in enumerate(self.layout.group_keys)]
        if not specs:   # a model without paged layers still needs slots and lengths: pages without memory
            specs = [host.module().GroupSpec(self.page_size, 0, int(max_requests) * self.table_width, self.table_width)]
            self._dummy_group = True
        else:
            self._dummy_group = False
        self.manager = host.module().CacheManager(specs, int(max_requests))
        self.max_requests = int(max_requests)
        self.pools = []
        for g, (hkv, d, _w) in enumerate(self.layout.group_keys):
            self.pools.append(torch.empty((self.layout.group_planes[g], pages[g], 2, hkv, self.page_size, d),
                                          dtype=dtype, device=device))
        self.states = [torch.zeros((self.max_requests,) + tuple(n.shape), dtype=n.dtype, device=device)
                       for n in self.layout.state_needs]
        self._views = [self._make_view(k) for k in range(len(self.layout.schedule))]

    def _make_view(self, k):
        lay = self.layout
        g, p, s = lay.run_group[k], lay.run_plane[k], lay.run_state[k]
        plane = self.pools[g][p] if g is not None else None
        stride = plane.stride(0) if plane is not None else 0
        return LayerCache(group=g, plane=plane, page_stride=stride, page_size=self.page_size,
                          writes=lay.schedule[k].cache_of is None, state=self.states[s] if s is not None else None)

    @staticmethod
    def bytes_per_token_of(model, dtype) -> int:
        return CacheLayout(model).bytes_per_token(dtype)

    def layer_cache(self, k) -> LayerCache:
        return self._views[k]

    @property
    def n_groups(self):
        return len(self.pools)

    # ---- requests
    def open(self) -> int:
        slot = self.manager.open()
        for s in self.states:
            s[slot].zero_()          # a new request starts from an all-zero state
        return slot

    def close(self, slot: int) -> None:
        self.manager.close(slot)
