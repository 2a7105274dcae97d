"""Block arrangements: how norms, mixer and feed-forward sit on the residual stream.

"pre_norm" is the reference's block (serve/model.py:146-149):
x = x + mixer(norm1(x)); x = x + ffn(norm2(x)). The residual stream x is
float32; each sub-layer's output is handed on as a pending delta and added
inside the next norm kernel.
"""
from __future__ import annotations

from .base import Block, build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, runtime, layer_spec=None):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.feed_forward_norm = build_part("norm", layer_spec.feed_forward_norm, runtime)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, runtime)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(x, a, ctx)
        f = self.feed_forward.forward(h, ctx)
        return x, f
