"""Next-token choice on the device for a batch of logits rows.

Greedy is the reference's argmax (crates/core-types/src/model.rs:44-62: lowest index wins a
tie, NaN is skipped).  With a temperature the kernel draws from softmax(logits / T) by the
Gumbel-max trick with a counter-based hash keyed by (seed, tokens generated so far,
vocabulary index): a request's draw does not depend on the batch it shares a step with.  The
reference's `SamplingParams` (crates/core-types/src/schedule.rs:16-40) also carries `top_p`;
like the reference this engine accepts only 1.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import lib as ops


class Ticket:
    """A launched sampling whose ids have not been read yet."""
    __slots__ = ("n", "host", "event")

    def __init__(self, n, host, event):
        self.n, self.host, self.event = n, host, event


class DeviceSampler:
    """Owns the small pinned and device buffers a step's sampling needs; one instance per engine.

    `launch` enqueues the kernel and the copy of its ids to the host and returns at once;
    `collect` waits for that copy.  Two samplings may be in flight (the engine queues the next
    step before it reads this one), so the pinned buffers are rings.  The kernel can write the
    ids to a second place on the device as well (`also_to`): the token buffer of a step that is
    queued behind this one.  The kernels' error flag lives behind the ids (`err`)."""

    DEPTH = 4

    def __init__(self, max_rows: int, device="cuda"):
        from ..engine.batch import PinnedRing
        n = int(max_rows)
        self.device = device
        dev = lambda dt: torch.empty(n + 1, dtype=dt, device=device)
        self._inv_t = (PinnedRing(n + 1, torch.float32, device, self.DEPTH), dev(torch.float32))
        self._seeds = (PinnedRing(n + 1, torch.int64, device, self.DEPTH), dev(torch.int64))
        self._counters = (PinnedRing(n + 1, torch.int32, device, self.DEPTH), dev(torch.int32))
        self._ids_host = [torch.empty(n + 1, dtype=torch.int32).pin_memory() for _ in range(self.DEPTH)]
        self._events = [torch.cuda.Event() for _ in range(self.DEPTH)]
        self._turn = 0
        self.max_rows = n
        self.ids_device = dev(torch.int32)
        self.ids_device.zero_()
        # the kernels' error flag sits behind the ids, so that one copy brings both to the host
        self.err = self.ids_device[n:n + 1]
        self.d2h_bytes = 0

    def launch(self, logits, rows, also_to=None) -> Ticket:
        """rows: objects with `temperature`, `seed`, `counter`, one per row of `logits`.  The ids
        and the error flag (`self.err`, which the step's kernels must have been given) travel to
        the host in one copy.  also_to: an int32 device tensor that receives the ids as well."""
        n, err = len(rows), self.err
        if n > self.max_rows:
            raise ValueError(f"{n} rows to sample, the sampler was made for {self.max_rows}")
        ids_d = self.ids_device
        if any(r.temperature > 0 for r in rows):
            (it_r, it_d), (sd_r, sd_d), (ct_r, ct_d) = self._inv_t, self._seeds, self._counters
            it_h, sd_h, ct_h = it_r.next(), sd_r.next(), ct_r.next()
            for i, r in enumerate(rows):
                it_h[i] = float(np.float32(1.0 / r.temperature)) if r.temperature > 0 else 0.0
                sd_h[i] = int(np.uint64(r.seed).astype(np.int64))
                ct_h[i] = r.counter
            for ring, h, d in ((it_r, it_h, it_d), (sd_r, sd_h, sd_d), (ct_r, ct_h, ct_d)):
                d[:n].copy_(h[:n], non_blocking=True)
                ring.sent()
            ops.sample(logits, n, ids_d, err, it_d[:n], sd_d[:n], ct_d[:n], also_to=also_to)
        else:
            ops.sample(logits, n, ids_d, err, also_to=also_to)
        self._turn = (self._turn + 1) % self.DEPTH
        host, event = self._ids_host[self._turn], self._events[self._turn]
        host.copy_(ids_d, non_blocking=True)
        event.record()
        self.d2h_bytes = 4 * (self.max_rows + 1)
        return Ticket(n, host, event)

    @staticmethod
    def collect(ticket: Ticket):
        """(ids, device error code) of a launch; the wait for its copy is the step's only
        synchronisation."""
        ticket.event.synchronize()
        out = ticket.host.tolist()
        return out[:ticket.n], out[-1]

    def sample(self, logits, rows):
        """launch + collect."""
        return self.collect(self.launch(logits, rows))
