"""The Python entry point: load a model, submit requests, step, generate.

`Engine` is the composition root, as the reference's CLI is for its crates
(docs/ARCHITECTURE.md:15-26): registry -> model -> cache -> runner -> scheduler -> sampler.
Request fields and their meanings follow the reference's `SubmitRequest` and
`SamplingParams` (crates/core-types/src/schedule.rs:16-49): prompt_tokens, max_new_tokens,
temperature (0 = greedy), top_p (kept for the interface, must be 1), seed, stop_tokens.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import host
from ..cache import CacheStorage
from ..config import registry
from ..errors import ConfigError, InvalidRequest
from ..ops import lib as ops
from ..sampling import DeviceSampler
from ..weights import init_random, load_weights
from .batch import StepEntry
from .runner import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
          "f16": torch.float16, "half": torch.float16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}
FINISH_REASONS = {0: "stop", 1: "length", 2: "cancelled"}


def parse_dtype(name):
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ConfigError(f"unsupported dtype {name!r}; choose bfloat16, float16 or float32") from None


def load_model(path, dtype="bfloat16", device="cuda", max_positions=None, random_seed=None):
    """(model, torch dtype) from a model folder.  With random_seed the folder needs only
    config.json and the weights are drawn on the device."""
    ops.require_cuda()
    td = parse_dtype(dtype)
    arch, cfg = registry.read_config(path)
    model = arch.build(cfg, td, device, max_positions=max_positions)
    if random_seed is not None:
        init_random(model, random_seed, device)
    else:
        rename = arch.hf_names(cfg) if arch.hf_names and not str(path).endswith(".gguf") else None
        load_weights(model, path, rename, device)
    return model, td


@dataclass
class SamplingParams:
    """crates/core-types/src/schedule.rs:16-29."""
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    @staticmethod
    def greedy():
        return SamplingParams()


@dataclass
class StepEvent:
    """`token` events carry a token id; `finished` events a reason (stop, length, cancelled)."""
    kind: str
    id: int
    token: Optional[int] = None
    reason: Optional[str] = None


_NOTHING_SAMPLED = object()      # stands for the ticket of a batch without sampled rows


class Engine:
    def __init__(self, model_path=None, dtype="bfloat16", random_weights=False, seed=0, page_size=16,
                 num_pages=None, max_batch_tokens=2048, max_batch_seqs=64, chunk_size=0, max_model_len=None,
                 gpu_memory_fraction=0.85, device="cuda", model=None, plan_ahead=True, profile=False):
        ops.require_cuda()
        if model is None:
            model, td = load_model(model_path, dtype, device, max_positions=max_model_len,
                                   random_seed=seed if random_weights else None)
        else:
            td = model.dtype
        self.model, self.dtype, self.device = model, td, device
        cfg = model.config
        self.max_model_len = int(max_model_len or getattr(cfg, "n_ctx_train", 4096))
        if num_pages is None:
            layout_bytes = CacheStorage.bytes_per_token_of(model, td)
            free, _total = torch.cuda.mem_get_info()
            budget = int(free * gpu_memory_fraction) - 2 * (1 << 30)
            num_pages = max(16, min(budget // max(layout_bytes * page_size, 1),
                                    (self.max_model_len * max_batch_seqs + page_size - 1) // page_size))
        self.cache = CacheStorage(model, td, device, page_size=page_size, num_pages=num_pages,
                                  max_requests=max_batch_seqs, max_model_len=self.max_model_len)
        self.sampler = DeviceSampler(max_batch_seqs, device)
        self.runner = ModelRunner(model, self.cache, max_batch_tokens=max_batch_tokens,
                                  max_batch_requests=max_batch_seqs, err=self.sampler.err)
        sc = host.module().SchedulerConfig()
        sc.max_batch_tokens, sc.max_batch_seqs, sc.chunk_size = int(max_batch_tokens), int(max_batch_seqs), int(chunk_size)
        sc.max_model_len, sc.n_vocab = self.max_model_len, model.n_vocab
        eos = getattr(cfg, "eos_token_ids", None)
        if eos is None:
            one = getattr(cfg, "eos_token_id", None)
            eos = () if one is None else (one,)
        sc.eos_token_ids = [int(t) for t in eos]
        self.scheduler = host.module().Scheduler(self.cache.manager, sc)
        self._next_id = 0
        self.plan_ahead = bool(plan_ahead)
        self._in_flight = None       # the sampling ticket of a batch that is on the GPU's queue
        if profile:
            # every launch is timed on its own: no CUDA graphs, one step at a time
            self.runner.use_graphs = False
            self.plan_ahead = False
            ops.profile_begin()

    # ------------------------------------------------------------------ requests
    def submit(self, prompt_tokens: Sequence[int], max_new_tokens: int, sampling: SamplingParams = None,
               stop_tokens: Sequence[int] = (), request_id: Optional[int] = None, temperature=None, seed=None) -> int:
        sp = sampling or SamplingParams()
        if temperature is not None:
            sp = SamplingParams(float(temperature), sp.top_p, sp.seed)
        if seed is not None:
            sp = SamplingParams(sp.temperature, sp.top_p, int(seed))
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid) + 1
        self.scheduler.submit(rid, [int(t) for t in prompt_tokens], int(max_new_tokens), float(sp.temperature),
                              float(sp.top_p), int(sp.seed) & 0xFFFFFFFFFFFFFFFF, [int(t) for t in stop_tokens])
        return rid

    def cancel(self, request_id: int) -> None:
        self.scheduler.cancel(int(request_id))

    # ------------------------------------------------------------------ one step
    def step(self) -> List[StepEvent]:
        """Plan a batch, run it, sample on the device, read the ids back, commit.

        While the GPU runs the batch the scheduler is asked for the one after it
        (`plan_ahead`); if that is decided already, it is queued behind the running one (the ids
        that this step draws are on the device already: its sampling kernel writes them where the
        next step reads its first tokens; portions of prompts that follow come from the host),
        and the next call finds it in flight.  The events returned are always those of one step."""
        if self._in_flight is None:
            plan = self.scheduler.plan()
            if not plan:
                return self._events(self.scheduler.commit([]))
            try:
                self._in_flight = self._launch(plan)
            except Exception:
                self.scheduler.abandon()
                raise
        ticket, self._in_flight = self._in_flight, None
        following = None
        try:
            if self.plan_ahead and ticket is not _NOTHING_SAMPLED:
                ahead = self.scheduler.plan_ahead()
                if ahead:
                    following = self._launch(ahead, ahead_of_commit=True)
            ids = []
            if ticket is not _NOTHING_SAMPLED:
                ids, code = self.sampler.collect(ticket)
                if code:
                    self.runner.check_device_errors()
        except Exception:
            self.scheduler.abandon()
            raise
        events = self.scheduler.commit(ids)
        self._in_flight = following
        return self._events(events)

    def _launch(self, plan, ahead_of_commit=False):
        """Queues the batch and its sampling on the GPU; returns the sampling's ticket."""
        entries, rows = [], []
        for p in plan:
            n = len(p.tokens)
            entries.append(StepEntry(p.slot, p.pos0, p.tokens, [n - 1] if p.sample else []))
            if p.sample:
                rows.append(p)
        # (a batch planned ahead starts with the rows whose token the step before it is still drawing)
        logits = self.runner.step(entries, commit=False, check=False, ahead_of_commit=ahead_of_commit,
                                  tokens_on_device=sum(1 for p in plan if p.from_device))
        # the ids also go where a step queued behind this one looks for its tokens
        return self.sampler.launch(logits, rows, also_to=self.runner.ctx.token_store) if rows else _NOTHING_SAMPLED

    @staticmethod
    def _events(raw):
        return [StepEvent("token", e.id, token=e.token) if e.kind == 0 else
                StepEvent("finished", e.id, reason=FINISH_REASONS[e.reason]) for e in raw]

    # ------------------------------------------------------------------ whole generations
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens=16, temperature=0.0, seed=0,
                 stop_tokens: Sequence[int] = ()) -> List[List[int]]:
        """Generates for every prompt (token ids in, token ids out), batching them continuously."""
        ids = [self.submit(p, max_new_tokens, SamplingParams(temperature, 1.0, seed), stop_tokens) for p in prompts]
        out: Dict[int, List[int]] = {i: [] for i in ids}
        live = set(ids)
        while live:
            for ev in self.step():
                if ev.id not in out:
                    continue
                if ev.kind == "token":
                    out[ev.id].append(ev.token)
                else:
                    live.discard(ev.id)
        return [out[i] for i in ids]

    def step_raw(self, entries, commit=True):
        """The step function itself, below the scheduler: `entries` is a list of
        `StepEntry(slot, pos0, tokens, want)` on slots taken with `self.cache.open()` (given back with
        `self.cache.close(slot)`); returns the float32 logits [wanted, vocab] on the device, or None.
        For replay and tests.  It shares the cache with `submit()` / `step()` but not their
        bookkeeping: use it on an engine that has no requests in flight."""
        if self._in_flight is not None or not self.scheduler.idle():
            raise RuntimeError("step_raw: the engine has requests in flight")
        return self.runner.step(list(entries), commit=commit)

    def profile_report(self):
        """Rows of `ops.profile_report` for everything launched since the engine was made with
        profile=True: per kernel its launches, milliseconds, share and, for the products, GB/s and
        TFLOP/s against the measured peaks of this machine where a MEASURED_PEAKS.json gives them."""
        import json
        peaks = None
        for folder in (os.getcwd(), os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))):
            try:
                with open(os.path.join(folder, "MEASURED_PEAKS.json")) as f:
                    d = json.load(f)
                peaks = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}
                break
            except (OSError, ValueError, KeyError, TypeError):
                continue
        return ops.profile_report(peaks)

    def stats(self) -> dict:
        s = self.scheduler.stats()
        m = self.cache.manager
        return {"steps": s.steps, "prompt_tokens": s.prompt_tokens, "decode_tokens": s.decode_tokens,
                "preemptions": s.preemptions, "finished": s.finished, "queued": self.scheduler.queued(),
                "active": self.scheduler.active(),
                "pages_used": [m.used_pages(g) for g in range(m.n_groups)],
                "pages_free": [m.free_pages(g) for g in range(m.n_groups)]}
