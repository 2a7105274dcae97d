"""Reading and writing the safetensors container without any other package.

File layout: 8 bytes little-endian header length N, N bytes of JSON mapping
tensor name -> {dtype, shape, data_offsets:[begin,end]} (plus an optional
"__metadata__" entry), then the raw little-endian tensor bytes. Tensors are
returned as torch views over a memory map, so nothing is copied until a tensor
is moved to the device.

The reference reads the same files through ``safetensors.torch.load_file``
(serve/hf_utils/convert_hf_checkpoint.py:9,123).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One open file: ``keys()``, ``info(name)`` (dtype, shape) and ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file size {size} (truncated?)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        header.pop("__metadata__", None)
        self._base = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dtype = _DTYPES[e["dtype"]]
                shape = tuple(int(s) for s in e["shape"])
                begin, end = (int(v) for v in e["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: entry {name!r} is malformed or has an unsupported dtype: {e!r}") from None
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * dtype.itemsize or begin < 0 or self._base + end > size:
                raise SafetensorsError(f"{path}: entry {name!r} has offsets [{begin},{end}) that do not match its shape/dtype or the file size")
            self._entries[name] = (dtype, shape, begin, end)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def keys(self) -> Iterable[str]:
        return self._entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self._entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._mm)[self._base + begin : self._base + end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # read-only buffer: the tensor is only ever copied from
            t = torch.frombuffer(buf, dtype=dtype)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors handed out may still view the map; it is released with them
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write CPU tensors (made contiguous) under their names."""
    header = {}
    offset = 0
    order = list(tensors.keys())
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(blob) % 8) % 8
    blob += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
