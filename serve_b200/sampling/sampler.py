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
        self._host = None     # pinned staging [3, cap] int32: temperatures (as float bits), request ids, token indices
        self._dev = None
        self._event = None

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], request_ids: Sequence[int],
               token_indices: Sequence[int], slots: Sequence[int] = None, last_token: torch.Tensor = None,
               out: torch.Tensor = None) -> torch.Tensor:
        """logits [L, V] float32 -> int32 [L] on the device (one token per row).

        ``out``, if given, receives the tokens instead of a new device tensor; it may be pinned host memory (the
        kernel then writes the tokens straight to the host, and no copy back is needed once the kernel has ended).

        With ``slots`` and ``last_token`` the token of row r is also left in last_token[slots[r]] on the device, where
        the next step's embedding finds it (FROM_DEVICE) without a trip through the host."""
        n = logits.shape[0]
        if not (len(temperatures) == len(request_ids) == len(token_indices) == n):
            raise ValueError("one temperature, request id and token index per row of logits is needed")
        if any(t < 0 for t in temperatures):
            raise ValueError("temperature must not be negative")
        if self._host is None or self._host.shape[1] < n:
            cap = max(64, 1 << (n - 1).bit_length())
            self._host = torch.empty((4, cap), dtype=torch.int32, pin_memory=self._pin)
            self._dev = torch.empty((4, cap), dtype=torch.int32, device=self.device)
        if self._event is not None:
            self._event.synchronize()       # the copy that last used the staging buffer has finished
        h = self._host.numpy()
        h[0, :n].view("float32")[:] = temperatures
        h[1, :n] = request_ids
        h[2, :n] = token_indices
        feed_back = slots is not None and last_token is not None
        if feed_back:
            h[3, :n] = slots
        self.kernels.fetch_ints(self._host, self._dev, self._host.numel())
        if self._pin:
            if self._event is None:
                self._event = torch.cuda.Event()
            self._event.record()
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=self.device)
        elif out.dtype != torch.int32 or out.numel() < n:
            raise ValueError("out must hold one int32 per row of logits")
        self.kernels.sample(logits, self._dev[0, :n].view(torch.float32), self._dev[1, :n], self._dev[2, :n], self.seed, out,
                            self._dev[3, :n] if feed_back else None, last_token if feed_back else None)
        return out
