"""Dense gated feed-forward (SwiGLU): down( silu(gate x) * (up x) ).

Reference: serve/model.py:80-85 (w1 = gate, w3 = up, w2 = down, no biases).
Gate and up weights are fused at load into one [2*I, hidden] matrix so that one
matrix product feeds the activation kernel.
"""
from __future__ import annotations

import torch

from .base import FeedForward, TensorDecl, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden, intermediate, names (gate/up/down tensor names relative to prefix)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.intermediate = int(p["intermediate"])
        names = p.get("names", {})
        self.gate_name = self.prefix + names.get("gate", "gate_proj.weight")
        self.up_name = self.prefix + names.get("up", "up_proj.weight")
        self.down_name = self.prefix + names.get("down", "down_proj.weight")
        self.w_gate_up = None
        self.w_down = None

    def tensor_decls(self):
        return [
            TensorDecl(self.gate_name, (self.intermediate, self.hidden)),
            TensorDecl(self.up_name, (self.intermediate, self.hidden)),
            TensorDecl(self.down_name, (self.hidden, self.intermediate)),
        ]

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.gate_name], tensors[self.up_name]], dim=0).contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def fused_description(self):
        """What a kernel that runs whole layers at once needs to know of this feed-forward."""
        return dict(kind="swiglu", hidden=self.hidden, intermediate=self.intermediate, w_gate_up=self.w_gate_up, w_down=self.w_down)

    def forward(self, h, ctx):
        rt = self.rt
        t = h.shape[0]
        act = rt.empty_act((t, self.intermediate))
        rt.kernels.gate_up_swiglu(h, self.w_gate_up, act)
        out = rt.empty_act((t, self.hidden))
        rt.kernels.linear(act, self.w_down, out)
        return out
