"""A pre-norm block: h += mixer(norm1(h)); h += ffn(norm2(h)).

The reference's order (crates/model/src/llama.rs:183-285; docs/ARCHITECTURE.md "Forward
pass").  The two residual sums happen inside the parts' last kernels, in float32.
"""
from __future__ import annotations

from .base import FeedForward, Mixer, Norm, Part


class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward,
                 names=("attn_norm.", "attn_", "ffn_norm.", "ffn_")):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self._names = names

    def children(self):
        return list(zip(self._names, (self.norm1, self.mixer, self.norm2, self.ffn)))

    def forward(self, h, ctx, cache):
        x = self.norm1.forward(h, ctx)
        ctx.flush_residual()            # no-op when the norm took the pending sum itself
        self.mixer.forward(x, ctx, cache, h)
        x = self.norm2.forward(h, ctx)
        ctx.flush_residual()
        self.ffn.forward(x, ctx, h)
