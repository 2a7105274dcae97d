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

    def fused_description(self, cache):
        """This arrangement with its parts' own descriptions, for kernels that run whole layers at once; None if a part
        has no description to give (such a layer runs part by part)."""
        out = {"kind": "pre_norm"}
        for name in self.wants:
            describe = getattr(getattr(self, name), "fused_description", None)
            if describe is None:
                return None
            out[name] = describe(cache) if name == "mixer" else describe()
        return out

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(x, a, ctx)
        f = self.feed_forward.forward(h, ctx)
        return x, f
