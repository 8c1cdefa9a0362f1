"""Interfaces of the parts a model is put together from.

A layer is a norm, a mixer, a norm and a feed-forward arranged by a block; a model is an
embedding, a list of blocks, a run order, a final norm and an output head.  Every part
takes its sizes and constants as constructor parameters and knows nothing about the
model it sits in.  The reference has one of each, wired by hand inside
`forward_one_token` (crates/model/src/llama.rs:150-293); the seams here are what another
mixer, feed-forward, norm or position encoding has to offer:

Part            named parameters (`params`), children (`children`), `finalize` after loading.
Norm            `forward(h, ctx, rows=None) -> x`: float32 rows in, compute-dtype rows out.
Mixer           `cache_need()` says what it keeps per request (paged keys/values and/or a
                fixed-size state); `forward(x, ctx, cache, residual)` adds its output to the
                float32 `residual` in place.  `cache` is a `LayerCache`: the page plane and
                the state rows this run of the layer may use.  A mixer whose kernels read
                work lists made on the host brings its planner with it: `plan(ctx, cache)`
                builds the lists of this step (see `Mixer.plan`).
FeedForward     `forward(x, ctx, residual)` adds its output to `residual` in place.
PositionEncoding `rotary()` returns the table a rotating mixer needs, or None;
                `on_embedding(h, ctx)` may add to the embedded tokens.
Block           `forward(h, ctx, cache)` runs its parts on the residual stream `h`.

A built-in part may leave its residual sum pending in `ctx` (StepContext.pending_residual)
for the next norm to add; whoever reads or writes `residual` by other means calls
`ctx.flush_residual()` first (PreNormBlock does so before every mixer and feed-forward).

`ctx` is the `StepContext` of the batch (engine/batch.py): which token belongs to which
request, positions, block tables, and the scratch allocator.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    shape: Tuple[int, ...]
    kind: str = "matrix"          # "matrix": compute dtype; "vector": float32; "table": int32
    init: object = "normal"       # random-weights mode: "normal" N(0, .02), "ones_normal" 1 + N(0, .02), another name
                                  # registered in weights/random_init.py, or a function (shape, generator, device, std)
    optional: bool = False        # may be absent from the file (e.g. a tied output matrix)


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of `n_kv_heads` x `head_dim` per position; `window` 0 keeps all keys."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per request (shape without the request dimension)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    paged: Optional[PagedKVNeed] = None
    state: Optional[StateNeed] = None


class Part:
    """Base of every part: a tree of named parameters."""

    # True when `forward` only enqueues work on the current stream with launch shapes that
    # depend on the batch's sizes alone (no host synchronisation, no data-dependent
    # allocation): such a part may be captured in a CUDA graph.  Parts say so themselves.
    graph_safe = False

    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(c.all_graph_safe() for _, c in self.children())

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def children(self) -> List[Tuple[str, "Part"]]:
        """(prefix, part) pairs; a child's parameters are named prefix + its own names."""
        return []

    def named_specs(self, prefix: str = "") -> Iterator[Tuple[str, ParamSpec, "Part", str]]:
        for local, spec in self.param_specs().items():
            yield prefix + local, spec, self, local
        for cp, child in self.children():
            yield from child.named_specs(prefix + cp)

    def assign(self, local_name: str, tensor: torch.Tensor) -> None:
        setattr(self, "w_" + local_name.replace(".", "_"), tensor)

    def finalize(self) -> None:
        """Called once after every parameter was assigned (fuse, precompute)."""
        for _, child in self.children():
            child.finalize()


class Norm(Part):
    def forward(self, h, ctx, rows=None, n_rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self):
        return None

    def on_embedding(self, h, ctx) -> None:
        return None


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def plan(self, ctx, cache) -> None:
        """Optional: build what this step's kernels need from the host (work lists, split
        tables) and send it to the device.  `forward` may call it itself; the runner calls it
        for every run of the schedule before it replays a captured graph, whose kernels read
        the lists at fixed addresses.  So: keep a step's result in `ctx.step_cache` under a key
        of the part's own (it is emptied for every batch; layers of one shape then share the
        work), put the lists into buffers from `ctx.plan_store` (they keep their addresses),
        and while `ctx.fixed_shapes` is set make grid sizes depend on the batch's sizes only."""
        return None

    def forward(self, x, ctx, cache, residual) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx, residual) -> None:
        raise NotImplementedError
