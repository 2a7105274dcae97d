"""Choosing the next token from float32 logits: greedy, or temperature sampling.

Greedy is the largest logit, the lowest index on ties. With a temperature the
reference draws argmax(softmax(l/T) / q), q ~ Exp(1) from torch's global
generator (serve/run.py:47-60); here the same distribution is drawn as
argmax(l/T - log q) with q from a counter-based hash of (seed, request id,
index of the generated token, vocabulary index), so a request's draws do not
depend on what else is in the batch or on how its prompt was cut. ``top_p`` is
a parameter the reference accepts and ignores (run.py:55); it is not built.
"""
from __future__ import annotations

from typing import Sequence

import torch


class Sampler:
    def __init__(self, kernels, device, seed: int = 0):
        self.kernels = kernels
        self.device = torch.device(device)
        self.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        self._pin = self.device.type == "cuda"

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], request_ids: Sequence[int],
               token_indices: Sequence[int]) -> torch.Tensor:
        """logits [L, V] float32 -> int32 [L] on the device (one token per row)."""
        n = logits.shape[0]
        if not (len(temperatures) == len(request_ids) == len(token_indices) == n):
            raise ValueError("one temperature, request id and token index per row of logits is needed")
        if any(t < 0 for t in temperatures):
            raise ValueError("temperature must not be negative")
        meta_f = torch.tensor(list(temperatures), dtype=torch.float32, pin_memory=self._pin).to(self.device, non_blocking=True)
        meta_i = torch.tensor([list(request_ids), list(token_indices)], dtype=torch.int32, pin_memory=self._pin).to(
            self.device, non_blocking=True)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        self.kernels.sample(logits, meta_f, meta_i[0], meta_i[1], self.seed, out)
        return out
