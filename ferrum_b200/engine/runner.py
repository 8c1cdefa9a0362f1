"""The step function: runs one batch of (request, its next tokens) through the model.

It runs only the tokens it is given, as one batch, against the cache that earlier steps
left, and returns the logits at the wanted places.  The reference's contract is kept per
entry: the first position must equal the number of positions the request already holds
(crates/model/src/llama.rs:353-361), and a step that fails leaves the lengths untouched
(:368-377; here the cache manager's lengths only advance in `commit`).
"""
from __future__ import annotations

from typing import List

import torch

from ..cache import CacheStorage
from ..errors import CacheError, FerrumError, InvalidRequest, KernelError
from ..ops import lib as ops
from ..models.decoder import NVTX
from .batch import StepContext, StepEntry

_DEVICE_ERRORS = {
    1: "a token id is outside the vocabulary", 2: "a position is outside the rotary table",
    3: "a position is beyond the block table", 4: "a token's page is missing from the block table",
    5: "attention reached a position whose page is missing", 6: "a row of logits is all NaN",
    10: "tensor-core product: the producer timed out", 11: "tensor-core product: the matrix unit timed out",
    12: "tensor-core product: the epilogue timed out", 13: "tensor-core product: the accumulator was not released in time",
    14: "tensor-core product: partial tiles did not arrive in time",
    20: "tensor-core attention: the producer timed out", 22: "tensor-core attention: the queries did not arrive in time",
    23: "tensor-core attention: keys or values did not arrive in time", 24: "tensor-core attention: the weights were not ready in time",
    25: "tensor-core attention: the scores were not ready in time", 26: "tensor-core attention: the output was not ready in time",
    27: "tensor-core attention: a product did not finish in time", 28: "tensor-core attention: the last values did not arrive in time",
}


class _CapturedStep:
    def __init__(self, graph, logits, generation, n_launches):
        self.graph, self.logits, self.generation = graph, logits, generation
        self.n_launches = n_launches      # kernels one replay launches


class ModelRunner:
    def __init__(self, model, cache: CacheStorage, max_batch_tokens=2048, max_batch_requests=None, use_graphs=True,
                 err=None):
        """use_graphs: steps that bring one token per request (decoding) are captured in a
        CUDA graph per (requests, wanted rows) the second time that shape is seen, and
        replayed afterwards; every other step is launched kernel by kernel."""
        ops.require_cuda()
        self.model, self.cache = model, cache
        self.device = cache.device
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_batch_requests = int(max_batch_requests or cache.max_requests)
        widths = [cache.table_width] * cache.n_groups
        self.ctx = StepContext(self.device, self.max_batch_tokens, self.max_batch_requests, widths, err=err)
        self.ctx.cache = cache
        # (guarded scratch buffers move whenever their size changes: no graphs then)
        self._graphs_possible = model.all_graph_safe() and not self.ctx.scratch.guard
        self.use_graphs = bool(use_graphs)
        self._graphs = {}
        self._seen = {}
        self.graph_replays = 0

    @property
    def use_graphs(self):
        """Whether decode-only steps are captured and replayed.  Never with a part that is not
        graph-safe, nor with guarded scratch buffers (they move when a size changes, and a captured
        graph would keep writing to where they were)."""
        return self._use_graphs and self._graphs_possible

    @use_graphs.setter
    def use_graphs(self, on):
        self._use_graphs = bool(on)

    def step(self, entries: List[StepEntry], commit=True, check=True, ahead_of_commit=False, tokens_on_device=False):
        """Returns float32 logits [n_wanted, V] on the device (a view that the next step
        overwrites), in the order of the entries and of their `want` lists; None when no
        logits are wanted.  With commit=False the caller advances the cache lengths itself.

        ahead_of_commit: the step is queued before the one ahead of it has been committed, so an
        entry starts past its request's committed length, where that step ends (the caller
        vouches for it).  tokens_on_device: the first so many entries bring one token each whose id
        is already in `ctx.token_store` (an earlier kernel of the stream leaves them there, in this
        order); those entries carry placeholders.  True stands for every entry."""
        mgr = self.cache.manager
        if not entries:
            return None
        seen = set()
        for e in entries:
            if len(e.tokens) == 0:
                raise InvalidRequest("a step entry has no tokens")
            if e.slot in seen:
                raise InvalidRequest("a request appears twice in one step")
            seen.add(e.slot)
            have = mgr.seq_len(e.slot)
            if e.pos0 != have and not (ahead_of_commit and e.pos0 > have):
                raise CacheError(f"position0 {e.pos0} does not match sequence length {have}")
            mgr.grow(e.slot, e.pos0 + len(e.tokens))      # no-op when the scheduler already reserved
            if e.pos0 == 0:
                for s in self.cache.states:
                    s[e.slot].zero_()                      # a request starts from an all-zero state
        decode_only = self.use_graphs and all(len(e.tokens) == 1 for e in entries)
        self.ctx.fixed_shapes = decode_only
        n_dev = len(entries) if tokens_on_device is True else int(tokens_on_device)
        if n_dev > len(entries) or any(len(e.tokens) != 1 for e in entries[:n_dev]):
            raise InvalidRequest("tokens on the device stand for one token per entry, first in the batch")
        self.ctx.fill(entries, mgr if self.cache.n_groups else [], keep_token_ids=n_dev)
        if NVTX:
            torch.cuda.nvtx.range_push(f"step tokens={self.ctx.n_tokens} requests={self.ctx.n_reqs}")
        logits = self._run_decode() if decode_only else self.model.forward(self.ctx, self.cache)
        if NVTX:
            torch.cuda.nvtx.range_pop()
        if check:
            self.check_device_errors()       # raises before anything is committed: the lengths stay as they were
        if commit:
            for e in entries:
                mgr.commit(e.slot, e.pos0 + len(e.tokens))
        return logits[:self.ctx.n_want] if logits is not None else None

    def _generation(self):
        return self.ctx.buffers_generation()

    def _run_decode(self):
        """A decode-only batch: replay its graph, or run it kernel by kernel and capture."""
        ctx = self.ctx
        key = (ctx.n_reqs, ctx.n_want)
        cap = self._graphs.get(key)
        if cap is not None and cap.generation == self._generation():
            self.model.plan(ctx, self.cache)     # this step's work lists, into the buffers the graph reads
            if cap.generation == self._generation():
                cap.graph.replay()
                self.graph_replays += 1
                ops.launches += cap.n_launches
                return cap.logits
        logits = self.model.forward(ctx, self.cache)
        self._seen[key] = self._seen.get(key, 0) + 1
        if self._seen[key] >= 2:
            # every buffer exists now and the plans of this step are cached: capturing
            # launches nothing and allocates nothing
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            with torch.cuda.graph(graph):
                captured = self.model.forward(ctx, self.cache)
            n_launches, ops.launches = ops.launches - before, before      # captured, not launched
            self._graphs[key] = _CapturedStep(graph, captured, self._generation(), n_launches)
            if len(self._graphs) > 96:
                self._graphs.pop(next(iter(self._graphs)))
        return logits

    def check_device_errors(self):
        """Synchronises and raises if a kernel raised the error flag, or (in the debugging mode with
        guarded scratch buffers) wrote past the end of one."""
        code = int(self.ctx.err.item())
        if code:
            self.ctx.err.zero_()
            raise KernelError(f"device error {code}: {_DEVICE_ERRORS.get(code, 'unknown')}")
        if self.ctx.scratch.guard:
            bad = self.ctx.scratch.check()
            if bad:
                raise KernelError("a kernel wrote past the end of: " + ", ".join(bad))
