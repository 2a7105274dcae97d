"""Run-time limits of an engine instance; nothing here describes the model.

The reference keeps these as module constants: page size 64 (serve/run.py:247),
at most 4000 live requests (run.py:13), 2048 prompt tokens a step (run.py:265),
60 % of free memory for the pool (serve/model.py:172), admission up to 90 % of
the pool (run.py:277). Here they are fields with those values as defaults.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

from .base import ConfigError


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"              # "bfloat16" | "float32"
    page_size: int = 64                  # tokens in a cache page
    num_pages: Optional[Union[int, Sequence[int]]] = None   # pages of every cache group, or one count per group; None: from memory_fraction
    memory_fraction: float = 0.6         # share of free device memory for the pools when num_pages is None
    max_slots: int = 256                 # live requests at most
    max_tokens_per_step: int = 2048      # token budget of a step
    max_context: Optional[int] = None    # longest sequence; None: the model's max position
    prefill_chunk: Optional[int] = None  # longest portion of one prompt in a step; None: the budget
    reserve_full: bool = False           # admit only when prompt+max_new fits (the reference's rule)
    admission_fraction: float = 0.9      # with reserve_full: share of the pool admission may promise
    use_cuda_graphs: bool = True         # replay pure-decode steps from captured graphs
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype {self.dtype!r} is not supported (bfloat16, float32)")
        if self.page_size <= 0:
            raise ConfigError("page_size must be positive")
        if self.num_pages is not None:
            counts = [self.num_pages] if isinstance(self.num_pages, int) else list(self.num_pages)
            if not counts or any(int(n) <= 0 for n in counts):
                raise ConfigError("num_pages must be positive")
        if not (0.0 < self.memory_fraction <= 1.0):
            raise ConfigError("memory_fraction must be in (0, 1]")
        if self.max_slots <= 0 or self.max_tokens_per_step <= 0:
            raise ConfigError("max_slots and max_tokens_per_step must be positive")
        if self.prefill_chunk is not None and self.prefill_chunk <= 0:
            raise ConfigError("prefill_chunk must be positive")


def normalize_dtype(name) -> str:
    """'bf16', 'bfloat16', torch.bfloat16 ... -> 'bfloat16' | 'float32'."""
    s = str(name).replace("torch.", "").lower()
    if s in ("bf16", "bfloat16"):
        return "bfloat16"
    if s in ("fp32", "float32", "float", "f32"):
        return "float32"
    raise ConfigError(f"dtype {name!r} is not supported (bfloat16, float32)")
