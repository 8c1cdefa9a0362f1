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


class DeviceSampler:
    """Owns the small pinned and device buffers a step's sampling needs; one instance per engine."""

    def __init__(self, max_rows: int, device="cuda"):
        n = int(max_rows)
        pin = lambda dt: torch.empty(n + 1, dtype=dt).pin_memory()
        dev = lambda dt: torch.empty(n + 1, dtype=dt, device=device)
        self._inv_t = (pin(torch.float32), dev(torch.float32))
        self._seeds = (pin(torch.int64), dev(torch.int64))
        self._counters = (pin(torch.int32), dev(torch.int32))
        self._ids = (pin(torch.int32), dev(torch.int32))
        self.d2h_bytes = 0

    def sample(self, logits, rows, err):
        """rows: objects with `temperature`, `seed`, `counter`, one per row of `logits`.
        Returns (ids, device error code): the ids and the error flag travel to the host in
        one copy, followed by the only synchronisation of the step."""
        n = len(rows)
        ids_h, ids_d = self._ids
        if any(r.temperature > 0 for r in rows):
            (it_h, it_d), (sd_h, sd_d), (ct_h, ct_d) = self._inv_t, self._seeds, self._counters
            for i, r in enumerate(rows):
                it_h[i] = float(np.float32(1.0 / r.temperature)) if r.temperature > 0 else 0.0
                sd_h[i] = int(np.uint64(r.seed).astype(np.int64))
                ct_h[i] = r.counter
            for h, d in (self._inv_t, self._seeds, self._counters):
                d[:n].copy_(h[:n], non_blocking=True)
            ops.sample(logits, n, ids_d, err, it_d[:n], sd_d[:n], ct_d[:n])
        else:
            ops.sample(logits, n, ids_d, err)
        ids_d[n:n + 1].copy_(err)
        ids_h[:n + 1].copy_(ids_d[:n + 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes = 4 * (n + 1)
        out = ids_h[:n + 1].tolist()
        return out[:n], out[n]
