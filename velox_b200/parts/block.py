"""Arrangements of a layer's parts.

`PreNormBlock`, the reference's decoder layer (src/paged/qwen3.rs:932-939):
    h = norm1(x); x = x + mixer(h); h = norm2(x); x = x + feed_forward(h)

The residual stream x is float32.  A sublayer's output is not added at once:
it travels as `delta` to the next norm, whose kernel forms x + delta in float32,
stores it and norms it in one pass.  A block therefore takes (residual, delta)
and returns (residual, delta); the model adds the last delta in its final norm.
"""
from __future__ import annotations

from .base import Block


class PreNormBlock(Block):
    norm_names = ("mixer", "feed_forward")

    def forward(self, residual, delta, ctx, cache):
        h = self.norms["mixer"].add_norm(residual, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norms["feed_forward"].add_norm(residual, a)
        f = self.feed_forward.forward(h, ctx)
        return residual, f
