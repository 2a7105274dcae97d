"""Rotary position encoding: frequencies, optional llama3 scaling, pairing style.

Frequencies follow serve/model.py:276, freq_j = 1 / base^(2j/D), and the llama3
rule of serve/model.py:247-266 per frequency. The reference rotates interleaved
pairs (2i, 2i+1) of weights it permuted at conversion
(serve/hf_utils/convert_hf_checkpoint.py:115-118); with the weight file's own
row order that is the rotation of pairs (j, j + D/2), which is the "half"
pairing here. "interleaved" is there for weights laid out the other way.
Angles (position x frequency) are formed in float32 inside the kernel.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part

PAIRING_HALF = 0
PAIRING_INTERLEAVED = 1


def rotary_inv_freq(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 [rotary_dim/2] inverse frequencies, scaled per frequency if asked.

    ``scaling`` is None or a mapping with factor, low_freq_factor,
    high_freq_factor, original_max_position_embeddings.
    """
    freqs = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2)[: rotary_dim // 2].float() / rotary_dim))
    if scaling is None:
        return freqs
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    old_len = float(scaling["original_max_position_embeddings"])
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    out = []
    for f in freqs:  # element-wise in float32, as the reference does
        wavelen = 2 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / factor)
        else:
            smooth = (old_len / wavelen - low) / (high - low)
            out.append((1 - smooth) * f / factor + smooth * f)
    return torch.stack([torch.as_tensor(v, dtype=torch.float32) for v in out]).to(torch.float32)


@register_part("position", "rotary")
class Rotary(PositionEncoding):
    """params: rotary_dim, theta, scaling (mapping or None), pairing ("half"|"interleaved")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.rotary_dim = int(p["rotary_dim"])
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        self.theta = float(p["theta"])
        self.scaling = p.get("scaling")
        pairing = p.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is not known (half, interleaved)")
        self.pairing = PAIRING_HALF if pairing == "half" else PAIRING_INTERLEAVED
        # layers with the same frequencies share one tensor: what a step derives from it is then made once, not per layer
        key = ("rotary_inv_freq", self.rotary_dim, self.theta, tuple(sorted(self.scaling.items())) if self.scaling else None)
        constants = getattr(runtime, "constants", None)
        if constants is None or key not in constants:
            made = rotary_inv_freq(self.rotary_dim, self.theta, self.scaling).to(runtime.device)
            if constants is None:
                constants = {}
            constants[key] = made
        self.inv_freq = constants[key]


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position signal in the mixer (rotary_dim 0)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.rotary_dim = 0
        self.pairing = PAIRING_HALF
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=runtime.device)
