"""An engine instance: a model with its weights, its cache and its step function.

The reference spreads this over ``load_model`` (serve/utils.py:41-78),
``LlamaModel.create_kv_cache`` (serve/model.py:168-194) and the top of
``generate`` (serve/run.py:246-249). Here ``Engine.from_folder`` reads a model
folder, ``Engine.from_config`` makes seeded random weights on the device, and
both end with a cache pool sized either by ``num_pages`` or by a share of the
free device memory.
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import torch

from .. import models  # noqa: F401  (registers architectures)
from .. import parts  # noqa: F401  (registers parts)
from ..cache import CacheManager
from ..config.base import ModelConfig, build_spec, load_config
from ..config.engine import EngineConfig, normalize_dtype
from ..models.decoder import DecoderModel
from ..weights.loader import load_from_source, load_weights
from ..weights.random_init import random_tensor
from .runtime import Runtime
from .step import StepEntry, Stepper

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _head_dims_of(spec) -> Sequence[int]:
    dims = set()
    for layer in spec.layers:
        for part in layer.parts.values():
            hd = part.params.get("head_dim")
            if hd:
                dims.add(int(hd))
    return sorted(dims)


class Engine:
    def __init__(self, config: ModelConfig, engine_config: Optional[EngineConfig] = None, kernels=None, spec=None):
        """Builds the model's parts; weights come through ``load_folder`` / ``load_random``.

        ``kernels`` defaults to the CUDA kernels of the engine's device (built at
        first use); tests pass a stand-in. ``spec`` overrides the layer
        description the architecture's builder would give.
        """
        self.config = config
        self.engine_config = engine_config or EngineConfig()
        self.engine_config.dtype = normalize_dtype(self.engine_config.dtype)
        self.engine_config.validate()
        self.spec = spec if spec is not None else build_spec(config)
        self.dtype = _TORCH_DTYPE[self.engine_config.dtype]
        if kernels is None:
            from ..kernels import load_kernels

            kernels = load_kernels(self.engine_config.device, _head_dims_of(self.spec))
        self.kernels = kernels
        device = getattr(kernels, "device", None) or self.engine_config.device
        self.rt = Runtime(kernels, device, self.dtype)
        self.model = DecoderModel(self.spec, self.rt)
        self.cache: Optional[CacheManager] = None
        self.stepper: Optional[Stepper] = None
        self.max_context = min(self.engine_config.max_context or self.spec.max_position, self.spec.max_position)

    # ---- construction -------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, engine_config: Optional[EngineConfig] = None, kernels=None) -> "Engine":
        eng = cls(load_config(model_dir), engine_config, kernels)
        load_weights(eng.model, model_dir, eng.dtype, eng.rt.device)
        eng._make_cache()
        return eng

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, engine_config: Optional[EngineConfig] = None, kernels=None,
                    std: float = 0.02, norm_std: float = 0.0, spec=None) -> "Engine":
        """Random weights made on the engine's device (no folder is written)."""
        eng = cls(config, engine_config, kernels, spec=spec)
        dev = eng.rt.device
        load_from_source(eng.model, lambda d: random_tensor(d, seed, std, norm_std, torch.float32, dev), eng.dtype, dev)
        eng._make_cache()
        return eng

    def _make_cache(self) -> None:
        ec = self.engine_config
        needs = self.model.cache_needs()
        cache_of = [e.cache_of for e in self.model.schedule]
        num_pages = ec.num_pages
        if num_pages is None:
            # Every group is sized to the same share of the most it could ever use (every slot at full context, or,
            # behind a window, what a slot can hold at a time), so that no group runs out long before the others;
            # the share is what the memory fraction pays for, at most all of it.
            keys = CacheManager.group_keys(needs)
            per_page = CacheManager.bytes_per_page(needs, ec.page_size, self.dtype.itemsize)
            most = [ec.max_slots * CacheManager.most_pages_of_a_request(key[2], ec.page_size, self.max_context, ec.max_tokens_per_step)
                    for key in keys]
            share = 1.0
            if self.rt.device.type == "cuda" and keys:
                free, _total = torch.cuda.mem_get_info(self.rt.device)
                share = min(1.0, free * ec.memory_fraction / max(1, sum(m * b for m, b in zip(most, per_page))))
            num_pages = [max(1, int(m * share)) for m in most]
        self.cache = CacheManager(needs, cache_of, ec.page_size, num_pages, ec.max_slots, self.max_context,
                                  device=self.rt.device, kv_dtype=self.dtype)
        self.num_pages = num_pages
        self.stepper = Stepper(self.model, self.cache, self.rt, ec.max_tokens_per_step, ec.use_cuda_graphs)

    # ---- the step -----------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]):
        """Run one batch (see Stepper.step); float32 logits [wanted, vocab] or None.

        The returned tensor may be overwritten by the next step: use or copy it first."""
        return self.stepper.step(entries)

    def end(self, rid: Hashable) -> None:
        """The request is finished: its pages and its slot are given back."""
        if self.cache.is_open(rid):
            self.cache.close(rid)

    def length(self, rid: Hashable) -> int:
        return self.cache.length(rid) if self.cache.is_open(rid) else 0
