"""Block arrangements: how norms, mixer and feed-forward sit on the residual stream.

"pre_norm" is the reference's block (serve/model.py:146-149):
x = x + mixer(norm1(x)); x = x + ffn(norm2(x)). The residual stream x is
float32; each sub-layer's output is handed on as a pending delta and added
inside the next norm kernel.
"""
from __future__ import annotations

from .base import Block, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    wants = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(x, a, ctx)
        f = self.feed_forward.forward(h, ctx)
        return x, f
