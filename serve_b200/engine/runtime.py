"""What every part is handed at construction: the kernels, the device and the dtypes."""
from __future__ import annotations

import torch


class _NoKernels:
    """Stands where a model is only described (tensor names and shapes), never run."""

    def check_attention_shape(self, heads, kv_heads, head_dim):
        return None

    def __getattr__(self, name):
        raise RuntimeError(f"this runtime only describes a model; kernel {name!r} cannot run")


class Runtime:
    def __init__(self, kernels, device, act_dtype: torch.dtype):
        self.kernels = kernels
        self.device = torch.device(device)
        self.act_dtype = act_dtype
        self.constants = {}      # device tensors that parts with equal parameters share (keyed by those parameters)

    @classmethod
    def describe_only(cls) -> "Runtime":
        return cls(_NoKernels(), "cpu", torch.float32)

    def empty_act(self, shape):
        return torch.empty(shape, dtype=self.act_dtype, device=self.device)
