"""Trace replay session: the loop behind `bin/trace_run`.

It owns nothing of its own: the model comes from the registry and the loader, the cache from
`CacheStorage`, and every step goes through `ModelRunner.step`, the same objects that
generation uses.  The reference's nearest relative is the teacher-forced
`forward(tokens, 0, slot, logits)` of its acceptance test (tests/accept/tests/m4_forward.rs:
158-166); a trace generalises it to several requests, cut into steps anywhere.
"""
from __future__ import annotations

import json
import os

from ..cache import CacheStorage
from .api import load_model
from .batch import StepEntry
from .runner import ModelRunner


class TraceSession:
    def __init__(self, model_dir, dtype, max_tokens, page_size=16, max_requests=8):
        max_tokens = max(int(max_tokens), page_size)
        # every live request's length is rounded up to whole pages
        self.model, self.dtype = load_model(model_dir, dtype, max_positions=max_tokens)
        self.cache = CacheStorage(self.model, self.dtype, "cuda", page_size=page_size, max_tokens=max_tokens,
                                  max_requests=max_requests, max_model_len=max_tokens)
        self.runner = ModelRunner(self.model, self.cache, max_batch_tokens=max_tokens,
                                  max_batch_requests=max_requests)
        self.slots = {}

    def run_step(self, rec):
        """rec: {"step", "entries": [{"id", "tokens", "want"}], "end": [...]}.  Returns the
        float32 logits [wanted, vocab] on the device, or None."""
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in self.slots:
                self.slots[rid] = self.cache.open()
            slot = self.slots[rid]
            entries.append(StepEntry(slot, self.cache.manager.seq_len(slot), list(e["tokens"]),
                                     list(e.get("want", []))))
        logits = self.runner.step(entries) if entries else None
        for rid in rec.get("end", []):
            if rid in self.slots:
                self.cache.close(self.slots.pop(rid))
        return logits

    def run_stream(self, lines, out_dir, log):
        os.makedirs(out_dir, exist_ok=True)
        for line in lines:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            logits = self.run_step(rec)
            if logits is not None and logits.shape[0] > 0:
                logits.detach().to("cpu").numpy().astype("<f4").tofile(os.path.join(out_dir, f"{rec['step']}.f32"))
            log.write(f"done {rec['step']}\n")
            log.flush()
