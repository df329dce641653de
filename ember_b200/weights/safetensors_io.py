"""Reading and writing the safetensors container.

Format (as the reference reads it, src/model/safetensors.cpp:54-82): 8 bytes of
little-endian header length, a JSON header mapping tensor names to ``dtype``,
``shape`` and ``data_offsets`` (relative to the end of the header), then raw
little-endian data.  ``__metadata__`` is skipped.  Sharded models list their files in
``model.safetensors.index.json`` under ``weight_map`` (safetensors.cpp:90-102).

Tensors are returned as CPU torch tensors that view the memory-mapped file.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too small to be a safetensors file")
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > size - 8 or header_len > _MAX_HEADER:
            raise SafetensorsError(f"{path}: invalid header length {header_len}")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from None
        self._data_start = 8 + header_len
        data_size = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: unsupported tensor dtype {dt} for {name}")
            dtype, esize = _DTYPES[dt]
            shape = tuple(int(x) for x in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            if begin > end or end > data_size:
                raise SafetensorsError(f"{path}: tensor {name} lies outside the file")
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * esize:
                raise SafetensorsError(f"{path}: tensor {name} has {end - begin} bytes for shape {list(shape)}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def get(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        # the mapping is read-only; torch warns about non-writable buffers, the tensors are never written
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=dtype)
        return t.reshape(shape)


class SafetensorsDir:
    """All tensors of a model folder (one file, or the shards its index names)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                idx = json.load(f)
            shards = sorted(set(idx["weight_map"].values()))
            paths = [os.path.join(model_dir, s) for s in shards]
        else:
            paths = [os.path.join(model_dir, "model.safetensors")]
        for p in paths:
            if not os.path.isfile(p):
                raise SafetensorsError(f"{model_dir}: {os.path.basename(p)} not found")
        self.files = [SafetensorsFile(p) for p in paths]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                if n in self._where:
                    raise SafetensorsError(f"tensor {n} appears in more than one file")
                self._where[n] = f

    def names(self) -> List[str]:
        return list(self._where)

    def has(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].entries[name][0]

    def get(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise SafetensorsError(f"the model has no tensor named {name}")
        return self._where[name].get(name)


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] = None) -> None:
    """Writes ``tensors`` (CPU, contiguous) as one safetensors file; names in sorted order."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor {name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
