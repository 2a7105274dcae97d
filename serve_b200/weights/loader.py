"""Weights by tensor name, from a model folder into the parts of a model.

A folder holds ``model.safetensors`` or shards listed in
``model.safetensors.index.json`` (the reference locates files the same way,
serve/hf_utils/convert_hf_checkpoint.py:70-96). The model's parts declare which
names and shapes they want; this module compares that with what the files hold
and raises ONE error that lists every missing tensor, every unexpected tensor
and every wrong shape. The reference renames into private names, permutes q/k
rows and stores a converted checkpoint (convert_hf_checkpoint.py:98-161); here
tensors keep their names and row order, and parts fuse what they want fused.

Kept dtypes: matrices become the compute dtype (bfloat16, or float32 for the
32-bit path); a vector stored in 32-bit stays 32-bit; integer tables become int32.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Optional

import torch

from ..parts.base import TensorDecl
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The weight files do not hold what the model needs."""


def _open_files(model_dir: str) -> Dict[str, SafetensorsFile]:
    """tensor name -> open file holding it."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    files: Dict[str, SafetensorsFile] = {}
    where: Dict[str, SafetensorsFile] = {}
    if os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
        for name, fname in weight_map.items():
            if fname not in files:
                path = os.path.join(model_dir, fname)
                if not os.path.isfile(path):
                    raise WeightError(f"{index} names {fname}, which is not in the folder")
                files[fname] = SafetensorsFile(path)
        for f in files.values():
            for name in f.keys():
                where[name] = f
    elif os.path.isfile(single):
        f = SafetensorsFile(single)
        for name in f.keys():
            where[name] = f
    else:
        raise WeightError(f"{model_dir!r} holds neither model.safetensors nor model.safetensors.index.json")
    return where


def kept_dtype(decl: TensorDecl, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if decl.role == "table":
        return torch.int32
    if decl.role == "vector" and stored == torch.float32:
        return torch.float32
    return compute


def load_weights(model, model_dir: str, compute_dtype: torch.dtype, device) -> None:
    """Fill ``model`` (a DecoderModel) from the folder, or raise WeightError."""
    try:
        where = _open_files(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    decls = model.tensor_decls()
    ignorable = set(model.ignorable_tensors())
    missing = sorted(n for n in decls if n not in where)
    unexpected = sorted(n for n in where if n not in decls and n not in ignorable)
    wrong = []
    for n, d in decls.items():
        if n in where:
            _, shape = where[n].info(n)
            if tuple(shape) != tuple(d.shape):
                wrong.append(f"{n}: file has {list(shape)}, model wants {list(d.shape)}")
    if missing or unexpected or wrong:
        lines = [f"weights in {model_dir!r} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(lines))
    tensors = {}
    for n, d in decls.items():
        t = where[n].tensor(n)
        tensors[n] = t.to(device=device, dtype=kept_dtype(d, t.dtype, compute_dtype)).contiguous()
    model.load(tensors)


def load_from_source(model, source: Callable[[TensorDecl], torch.Tensor], compute_dtype: torch.dtype, device) -> None:
    """Fill ``model`` from a function that makes each declared tensor (random-weights mode)."""
    tensors = {}
    for n, d in model.tensor_decls().items():
        t = source(d)
        tensors[n] = t.to(device=device, dtype=kept_dtype(d, t.dtype, compute_dtype)).contiguous()
    model.load(tensors)
