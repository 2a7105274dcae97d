"""RMS normalisation, fused with the residual addition that precedes it.

Reference formula (serve/model.py:63-68): y = x32 * rsqrt(mean(x32^2) + eps),
cast to the model dtype, times weight. Here the residual stream itself is kept
in float32, the pending delta of the previous sub-layer is added in the same
kernel (model.py:147-148 do it as a separate op), and the product with the
weight is taken in float32 before the single rounding to the activation dtype.
"""
from __future__ import annotations

from .base import Norm, TensorDecl, register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """params: size, eps, weight_name (relative to prefix, default "weight")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight_name = self.prefix + spec.params.get("weight_name", "weight")
        self.weight = None

    def tensor_decls(self):
        return [TensorDecl(self.weight_name, (self.size,), role="vector", init="norm")]

    def load(self, tensors):
        self.weight = tensors[self.weight_name]

    def fused_description(self):
        """What a kernel that runs whole layers at once needs to know of this norm."""
        return dict(kind="rms", size=self.size, eps=self.eps, weight=self.weight)

    def forward(self, x, delta, ctx):
        out = self.rt.empty_act((x.shape[0], self.size))
        self.rt.kernels.add_rmsnorm(x, delta, self.weight, self.eps, out)
        return out

    def forward_rows(self, x, delta, rows, ctx):
        out = self.rt.empty_act((rows.shape[0], self.size))
        self.rt.kernels.add_rmsnorm_rows(x, delta, rows, self.weight, self.eps, out)
        return out
