"""Random weights from a configuration and a seed, by tensor name.

``write_random_model`` writes a model folder (config.json, model.safetensors)
that the ordinary loader reads back, so tests and measurements need no
download. Values: matrices N(0, std); norm weights 1, or 1 + N(0, norm_std).
Every tensor draws from its own generator seeded by (seed, name), so a value
does not depend on which other tensors exist or in which order they are made.
The reference has no such mode (it always downloads, serve/utils.py:41-53).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..parts.base import TensorDecl


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(decl: TensorDecl, seed: int, std: float = 0.02, norm_std: float = 0.0,
                  dtype: torch.dtype = torch.float32, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, decl.name))
    if decl.role == "table":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "norm":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
        if norm_std:
            t = t + norm_std * torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device)
        return t.to(dtype)
    t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * std
    return t.to(dtype)


def model_tensor_decls(config) -> Dict[str, TensorDecl]:
    """Declared tensors of the model that ``config`` describes (no device, no kernels)."""
    from ..config.base import build_spec
    from ..engine.runtime import Runtime
    from ..models.decoder import DecoderModel

    model = DecoderModel(build_spec(config), Runtime.describe_only())
    return model.tensor_decls()


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Write config.json and model.safetensors for ``config`` with seeded random weights."""
    from .safetensors_io import write_safetensors

    os.makedirs(model_dir, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    tensors = {n: random_tensor(decl, seed, std, norm_std, dtype) for n, decl in model_tensor_decls(config).items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
