"""Causal grouped-query attention over the paged cache.

q, k, v projections (one fused matrix), rotary encoding of q and k fused with the cache
write, attention of every token over its request's pages, output projection added to the
residual stream (crates/model/src/llama.rs:185-257).  Query head h reads KV head
h / (Hq/Hkv); the score scale is 1/sqrt(head_dim) unless given.  `window` > 0 keeps the last
`window` keys only; the reference has no window.
"""
from __future__ import annotations

import math

import torch

from ..ops import lib as ops
from . import attention_plan
from .base import CacheNeed, Mixer, PagedKVNeed, ParamSpec
from .linear import RESIDUAL, STORE, linear, linear_deferred


# Up to this many tokens in a step the attention kernel lets the kernels after it start early
# (see attention_flash.cu); with more, their waiting blocks cost more than the overlap gains.
EARLY_TRIGGER_MAX_TOKENS = 16


# The CUDA-core attention cuts a row's keys among CTAs while the step has fewer rows than this many
# per SM (a CTA slot is a third of an SM: under some 2.7 waves of whole rows the last wave idles
# too much); with more rows, tokens of a request that follow each other share their key tiles.
GENERIC_SPLIT_BELOW = 8


class PagedAttention(Mixer):
    @property
    def graph_safe(self):
        """Decoded tokens run under a CUDA graph when one token's rows (the query heads of a KV
        head) fit the 16-row tile of the tensor-core kernel, whose padded work list has a shape
        that depends on the number of requests only; larger groups take the 64-row class, whose
        grid follows the context lengths.  The generic kernel has no work lists at all."""
        if not ops.attention_flash_supported(self.dtype, self.D):
            return True
        return self.Hq // self.Hkv <= 16

    def __init__(self, width, n_head, n_head_kv, head_dim, position, dtype, window=0, scale=None):
        if n_head % n_head_kv:
            raise ValueError("head count is not divisible by kv head count")
        self.width, self.Hq, self.Hkv, self.D = width, n_head, n_head_kv, head_dim
        self.position, self.dtype, self.window = position, dtype, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.w_q_weight = self.w_k_weight = self.w_v_weight = self.w_output_weight = None
        self.w_qkv = None
        self._tc_tokens = {}     # cache shape -> tokens per tile of the tcgen05 kernel (0: not applicable)

    def param_specs(self):
        q, kv = self.Hq * self.D, self.Hkv * self.D
        return {"q.weight": ParamSpec((q, self.width)), "k.weight": ParamSpec((kv, self.width)),
                "v.weight": ParamSpec((kv, self.width)), "output.weight": ParamSpec((self.width, q))}

    def finalize(self):
        self.w_qkv = torch.cat([self.w_q_weight, self.w_k_weight, self.w_v_weight], dim=0).contiguous()
        self.w_q_weight = self.w_k_weight = self.w_v_weight = None

    def cache_need(self):
        return CacheNeed(paged=PagedKVNeed(self.Hkv, self.D, self.window))

    def forward(self, x, ctx, cache, residual):
        T, Hq, Hkv, D = ctx.n_tokens, self.Hq, self.Hkv, self.D
        qw = Hq * D
        qkv = ctx.buf("attn_qkv", (ctx.token_capacity, (Hq + 2 * Hkv) * D), self.dtype)
        w = self.w_qkv if cache.writes else self.w_qkv[:qw]   # a run that reads another run's cache needs q only
        part = linear_deferred(x, w, ctx, T) if ctx.defer_residuals else None
        if part is None:
            linear(x, w, qkv, STORE, ctx, M=T)
        rot = self.position.rotary() if self.position is not None else None
        table = ctx.block_tables[cache.group]
        ops.rope_cache_write(qkv, T, ctx.positions, ctx.req_of_token, table,
                             rot.cos_sin if rot is not None else None, cache.plane, cache.page_stride,
                             cache.page_size, Hq, Hkv, D, rot.rope_dim if rot is not None else 0,
                             rot.pairing if rot is not None else 0, cache.writes, ctx.err, partials=part)
        out = ctx.buf("attn_out", (ctx.token_capacity, qw), self.dtype)
        if ops.attention_flash_supported(self.dtype, D):
            self._flash(qkv, out, ctx, cache, table)
        else:
            self._generic(qkv, out, ctx, cache, table)
        linear(out, self.w_output_weight, residual, RESIDUAL, ctx, M=T)

    def _generic(self, qkv, out, ctx, cache, table):
        """CUDA-core path.  With enough rows to fill the GPU (a prompt portion) every row walks its
        keys alone; with few (decoding) the keys of a row are cut into splits among CTAs.  Which of
        the two runs depends on the number of tokens only, and so does the number of split slots
        while a CUDA graph is being captured or replayed (then it covers the longest context the
        cache can hold)."""
        T, Hq, Hkv, D = ctx.n_tokens, self.Hq, self.Hkv, self.D
        rows = T * Hkv * -(-(Hq // Hkv) // 4)
        part, slots = None, 0
        if rows < GENERIC_SPLIT_BELOW * attention_plan.sm_count():
            split = ops.attention_generic_split()
            longest = table.shape[1] * cache.page_size if ctx.fixed_shapes else ctx.max_kv_len
            if self.window > 0:
                longest = min(longest, self.window + split)       # a window of w keys touches at most w / split + 2 splits
            slots = longest // split + 2
            part = ctx.buf("attn_generic_part", (T * Hq * slots * (D + 2),), torch.float32)
        ops.attention_generic(qkv, out, T, ctx.positions, ctx.req_of_token, table, cache.plane, cache.page_stride,
                              cache.page_size, Hq, Hkv, D, self.scale, self.window, ctx.err, part, slots,
                              q_start=ctx.q_start, n_reqs=ctx.n_reqs)

    def plan(self, ctx, cache):
        """The step's work lists of the tensor-core kernels for this layer's shape (None on the
        generic path, which has none)."""
        if not ops.attention_flash_supported(self.dtype, self.D):
            return None
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        shape_key = (cache.page_size, cache.page_stride, cache.plane.dtype, cache.plane.dim())
        tc_tokens = self._tc_tokens.get(shape_key)
        if tc_tokens is None:
            tc_tokens = self._tc_tokens[shape_key] = ops.attention_tc_tokens(D, Hq // Hkv, cache.page_size, cache.plane,
                                                                             cache.page_stride)
        return attention_plan.plans_for(ctx, Hq // Hkv, self.window, Hkv, tc_tokens)

    def _flash(self, qkv, out, ctx, cache, table):
        """Tensor-core path: one launch per row-tile class of the step's plan, plus a merge
        launch where key ranges were split."""
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        for plan in self.plan(ctx, cache):
            if plan is None:
                continue
            part_o = part_ml = None
            if plan.n_slots:
                part_o = ctx.buf("attn_part_o", (plan.n_slots * plan.bm * D,), torch.float32)
                part_ml = ctx.buf("attn_part_ml", (plan.n_slots * plan.bm * 2,), torch.float32)
            if plan.kind == "tc":
                ops.attention_tc(qkv, out, cache.plane, cache.page_stride, cache.page_size, table, ctx.q_start, ctx.pos0,
                                 plan.work, plan.n_work, part_o, part_ml, Hq, Hkv, D, self.scale, self.window, ctx.err)
            else:
                ops.attention_flash(qkv, out, cache.plane, cache.page_stride, cache.page_size, table, ctx.q_start,
                                    ctx.pos0, plan.work, plan.n_work, part_o, part_ml, Hq, Hkv, D, self.scale,
                                    self.window, plan.bm, ctx.err, plan.cta_items, plan.n_ctas,
                                    trigger_early=ctx.n_tokens <= EARLY_TRIGGER_MAX_TOKENS)
            if plan.n_comb:
                ops.attention_combine(out, part_o, part_ml, ctx.q_start, ctx.req_of_token, plan.req_tile0,
                                      plan.tile_info, plan.comb_tokens, plan.n_comb, Hq, Hkv, D, plan.bm, plan.comb_warps)
