"""The description of one step's batch, on the device, and the scratch memory of a step.

A step is a list of entries (request slot, first position, its next tokens, which of them
want logits).  The reference's step takes one sequence per call
(`forward(token_ids, position0, slot, logits_out)`, crates/core-types/src/model.rs:200-206);
here all entries are flattened into one batch: per token its id, its position and its
request's index; per request its first token's index, the number of cached positions, its
slot id and one block-table row per cache group.  Everything travels in one pinned buffer
and one host-to-device copy per step (plus one per cache group for the block tables).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    pos0: int
    tokens: Sequence[int]
    want: Sequence[int] = ()       # indices into `tokens` whose logits are wanted


CANARY = 0x7FC0BEEF      # bit pattern of the guard words (a quiet NaN when read as float32)


class Scratch:
    """Named device buffers that live across steps and only ever grow, so that a buffer
    keeps its address from step to step.

    guard > 0 (FERRUM_CANARY=1 sets 64): debugging mode.  Every buffer is allocated to the exact
    size asked for plus `guard` 4-byte words behind it that hold a fixed pattern; `check()` names
    the buffers whose guard words a kernel has overwritten.  A buffer is then reallocated whenever
    its size changes, so steps run without CUDA graphs in this mode."""

    def __init__(self, device, guard=None):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._guards: Dict[str, torch.Tensor] = {}
        self.generation = 0      # bumped whenever a buffer is (re)allocated and so may have moved
        self.guard = int(os.environ.get("FERRUM_CANARY", "0") == "1") * 64 if guard is None else int(guard)

    def get(self, name, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        t = self._bufs.get(name)
        if self.guard:
            if t is None or t.dtype != dtype or t.numel() != max(n, 1):
                esize = torch.empty((), dtype=dtype).element_size()
                nbytes = (max(n, 1) * esize + 3) // 4 * 4
                raw = torch.empty(nbytes + 4 * self.guard, dtype=torch.uint8, device=self.device)
                words = raw[nbytes:].view(torch.int32)
                words.fill_(CANARY)
                t = raw[:max(n, 1) * esize].view(dtype)
                self._bufs[name], self._guards[name] = t, words
                self.generation += 1
            return t[:n].view(*shape)
        if t is None or t.dtype != dtype or t.numel() < n:
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = t
            self.generation += 1
        return t[:n].view(*shape)

    def check(self):
        """Names of the buffers whose guard words no longer hold the pattern (guard mode only)."""
        return [name for name, words in self._guards.items() if not bool((words == CANARY).all())]

    def bytes(self):
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


class PinnedRing:
    """A few pinned host buffers used in turn for host-to-device copies.  A buffer is
    rewritten only after the copy that last read it has run, so the host may run several
    steps ahead of the GPU without tearing a step's inputs."""

    def __init__(self, numel, dtype, device, depth=4):
        self.cuda = str(device) != "cpu"
        mk = (lambda: torch.empty(numel, dtype=dtype).pin_memory()) if self.cuda else (lambda: torch.empty(numel, dtype=dtype))
        self.bufs = [mk() for _ in range(depth)]
        self.events = [None] * depth
        self.i = 0

    def next(self):
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[self.i] is not None:
            self.events[self.i].synchronize()
        return self.bufs[self.i]

    def sent(self):
        """Call right after enqueueing the copy out of the current buffer."""
        if self.cuda:
            if self.events[self.i] is None:
                self.events[self.i] = torch.cuda.Event()
            self.events[self.i].record()


class PlanStore:
    """Staging for work lists that a part builds on the host every step: per key a ring of pinned
    buffers and one device buffer that keeps its address while it is large enough (a captured
    graph reads it at that address).  `generation` counts the times a device buffer moved."""

    def __init__(self, device):
        self.device = device
        self._bufs = {}
        self.generation = 0

    def buffers(self, key, n):
        """(PinnedRing, int32 device buffer) of at least n elements for `key`."""
        b = self._bufs.get(key)
        if b is None or b[1].numel() < n:
            cap = max(1024, 2 * n)
            b = (PinnedRing(cap, torch.int32, self.device), torch.empty(cap, dtype=torch.int32, device=self.device))
            self._bufs[key] = b
            self.generation += 1
        return b


class StepContext:
    """Built once per runner; `fill` rewrites it for each step.

    For parts that plan on the host: `step_cache` is a dict that is emptied at every `fill` (a
    part keeps there what it worked out for this batch, under a key of its own choosing, so that
    all layers of one shape share it), and `plan_store` hands out buffers that keep their
    addresses from step to step."""

    def __init__(self, device, max_tokens, max_requests, table_widths: List[int], err=None):
        """err: an int32 device tensor of one element to use as the kernels' error flag (the
        engine puts it next to the sampled ids so that both reach the host in one copy)."""
        self.device = device
        self.max_tokens, self.max_requests = int(max_tokens), int(max_requests)
        self.table_widths = list(table_widths)
        self.scratch = Scratch(device)
        self.err = err if err is not None else torch.zeros(1, dtype=torch.int32, device=device)
        n_small = 4 * self.max_tokens + 3 * self.max_requests + 1
        self._host = PinnedRing(n_small, torch.int32, device)
        self._dev = torch.empty(n_small, dtype=torch.int32, device=device)
        self.token_store = self._dev       # a step's token ids are its first entries
        self._bt_host = [PinnedRing(self.max_requests * w, torch.int32, device) for w in self.table_widths]
        self._bt_dev = [torch.empty((self.max_requests, w), dtype=torch.int32, device=device) for w in self.table_widths]
        self._splitk_counters = torch.zeros(4096, dtype=torch.int32, device=device)
        self.step_cache: Dict[object, object] = {}
        self.plan_store = PlanStore(device)
        self.n_tokens = self.n_reqs = self.n_want = 0
        self.fixed_shapes = False     # True while a decode-only batch runs under a CUDA graph
        # A residual product of a few tokens may stay in partials until the next norm adds it
        # (one kernel less on the critical path): (residual tensor, ops.Partials) or None.
        self.pending_residual = None
        self.defer_residuals = True
        self.defer_swiglu = True
        self.h2d_bytes = 0            # bytes copied to the device by the last fill
        self.token_capacity = self.want_capacity = 0

    # ------------------------------------------------------------------ per step
    def fill(self, entries: List[StepEntry], tables, token_capacity=None, keep_token_ids=False):
        """tables: the native CacheManager whose block tables the entries' slots index, or
        explicit rows, tables[g][r] being the row of entry r in group g.  keep_token_ids: the
        device already holds the first so many token ids of this step (`token_store`, written by an
        earlier kernel of the stream); the entries' own ids are placeholders there and are not
        uploaded."""
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        if R > self.max_requests or T > self.max_tokens:
            raise ValueError(f"batch of {T} tokens / {R} requests exceeds the runner's limits "
                             f"({self.max_tokens} / {self.max_requests})")
        W = sum(len(e.want) for e in entries)
        host = self._host.next()
        h = host.numpy()
        tok, pos, req, want = h[0:T], h[T:2 * T], h[2 * T:3 * T], h[3 * T:3 * T + W]
        o = 3 * T + W
        qstart, pos0, slots = h[o:o + R + 1], h[o + R + 1:o + 2 * R + 1], h[o + 2 * R + 1:o + 3 * R + 1]
        if T == R and W in (0, R):
            # one token per request (decoding): whole-array assignments
            self.h_q_start, self.h_q_len = list(range(R)), [1] * R
            self.h_pos0, self.h_slots = [e.pos0 for e in entries], [e.slot for e in entries]
            tok[:] = [e.tokens[0] for e in entries]
            pos[:] = self.h_pos0
            req[:] = qstart[:R] = self.h_q_start
            pos0[:] = self.h_pos0
            slots[:] = self.h_slots
            if W:
                if any(tuple(e.want) != (0,) for e in entries):
                    raise ValueError("wanted index is outside the entry's 1 tokens")
                want[:] = self.h_q_start
        else:
            t = w = 0
            self.h_q_start, self.h_q_len, self.h_pos0, self.h_slots = [], [], [], []
            for r, e in enumerate(entries):
                n = len(e.tokens)
                tok[t:t + n] = np.asarray(e.tokens, dtype=np.int32)
                pos[t:t + n] = np.arange(e.pos0, e.pos0 + n, dtype=np.int32)
                req[t:t + n] = r
                if len(set(e.want)) != len(e.want):
                    # (a row's pending residual product is added when the row is gathered: once only)
                    raise ValueError("a wanted index appears twice in one entry")
                for i in e.want:
                    if not 0 <= i < n:
                        raise ValueError(f"wanted index {i} is outside the entry's {n} tokens")
                    want[w] = t + i
                    w += 1
                qstart[r], pos0[r], slots[r] = t, e.pos0, e.slot
                self.h_q_start.append(t); self.h_q_len.append(n); self.h_pos0.append(e.pos0); self.h_slots.append(e.slot)
                t += n
        qstart[R] = T
        total = o + 3 * R + 1
        first = min(int(keep_token_ids), T)
        self._dev[first:total].copy_(host[first:total], non_blocking=True)
        self._host.sent()
        self.h2d_bytes = (total - first) * 4
        d = self._dev
        self.token_ids, self.positions, self.req_of_token = d[0:T], d[T:2 * T], d[2 * T:3 * T]
        self.want_rows = d[3 * T:3 * T + W]
        self.q_start, self.pos0, self.slots = d[o:o + R + 1], d[o + R + 1:o + 2 * R + 1], d[o + 2 * R + 1:o + 3 * R + 1]
        self.block_tables = []
        explicit = isinstance(tables, (list, tuple))
        for g in range(len(self.table_widths)):
            w = self.table_widths[g]
            bhost = self._bt_host[g].next()
            if explicit:
                bh = bhost.numpy().reshape(self.max_requests, w)
                for r, row in enumerate(tables[g]):
                    bh[r, :len(row)] = row
            else:
                from .. import host as host_module
                host_module.module().copy_tables(tables, g, self.h_slots, bhost.data_ptr(), w)
            self._bt_dev[g][:R].copy_(bhost[:R * w].view(R, w), non_blocking=True)
            self._bt_host[g].sent()
            self.h2d_bytes += R * self.table_widths[g] * 4
            self.block_tables.append(self._bt_dev[g][:R])
        self.n_tokens, self.n_reqs, self.n_want = T, R, W
        self.token_capacity = int(token_capacity or T)
        self.want_capacity = max(W, 1)
        self.max_q_len = max(self.h_q_len) if R else 0
        self.max_kv_len = max((p + n for p, n in zip(self.h_pos0, self.h_q_len)), default=0)
        self.step_cache = {}
        self.pending_residual = None

    def buffers_generation(self):
        """Changes whenever a buffer that kernels read may have moved (a captured graph is stale then)."""
        return (self.scratch.generation, self.plan_store.generation)

    # ------------------------------------------------------------------ pending residual sum
    def take_pending_residual(self, h):
        """For a norm about to read `h`: the partials it must add first, or None.  Partials
        pending for another tensor are added to that tensor now."""
        p = self.pending_residual
        if p is None:
            return None
        if p[0].data_ptr() == h.data_ptr():
            self.pending_residual = None
            return p[1]
        self.flush_residual()
        return None

    def flush_residual(self):
        """Adds a pending residual product to its tensor (for consumers that do not know
        about partials, and before the product workspace is used again)."""
        p = self.pending_residual
        if p is not None:
            from ..ops import lib as ops
            self.pending_residual = None
            ops.residual_reduce(p[0], self.n_tokens, p[1])

    # ------------------------------------------------------------------ scratch
    def buf(self, name, shape, dtype):
        return self.scratch.get(name, shape, dtype)

    def gemm_scratch(self, M, N, K, dual):
        """(float32 workspace, zeroed int32 tile counters) for the tensor-core product."""
        from ..ops import lib as ops
        floats, tiles = ops.gemm_tc_workspace(M, N, K, dual)
        if tiles > self._splitk_counters.numel():
            self._splitk_counters = torch.zeros(2 * tiles, dtype=torch.int32, device=self.device)
        return self.scratch.get("gemm_partials", (floats,), torch.float32), self._splitk_counters
