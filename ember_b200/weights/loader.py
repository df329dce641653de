"""Weights by tensor name, with one error that lists everything that is wrong.

A ``WeightStore`` wraps a source of named tensors (a model folder, or tensors made in
memory).  Parts *declare* what they need (``take(name, shape)``); every problem —
a missing tensor, a wrong shape, a tensor nobody asked for — is collected, and
``finish()`` raises a single ``WeightError`` that lists them all.  Tensors nobody asked
for are listed in that error whenever something else is wrong; when they are the only
finding the load goes on with a warning that lists them (the reference looks tensors up
by name and never sees the rest, src/backend/cpu/cpu_backend.cpp:50-75, and published
files do carry extra buffers), unless the store is ``strict``.

Stored precision is kept: bfloat16 stays bfloat16, float32 stays float32, float16 is
converted to bfloat16 (the serving precision), integer tables become int32.  The
float32 path widens everything to float32 when it builds its device copies; that is
the parts' business, not the store's.
"""
from __future__ import annotations

import fnmatch
import warnings
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsDir


class WeightError(ValueError):
    """Raised once per load; ``missing``, ``unexpected`` and ``wrong_shape`` hold the details."""

    def __init__(self, source: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"the weights in {source} do not fit the model:"]

        def clip(items, fmt):
            shown = [fmt(i) for i in items[:12]]
            if len(items) > 12:
                shown.append(f"... and {len(items) - 12} more")
            return shown

        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += ["    " + s for s in clip(self.missing, str)]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += ["    " + s for s in clip(
                self.wrong_shape, lambda t: f"{t[0]} has shape {list(t[1])}, expected {list(t[2])}")]
        if self.wrong_dtype:
            lines.append(f"  unsupported dtypes ({len(self.wrong_dtype)}):")
            lines += ["    " + s for s in clip(self.wrong_dtype, lambda t: f"{t[0]} is {t[1]}")]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += ["    " + s for s in clip(self.unexpected, str)]
        super().__init__("\n".join(lines))


class UnexpectedTensorsWarning(UserWarning):
    """The model folder holds tensors that no part of the model asked for."""


class _DictSource:
    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self._t = dict(tensors)

    def names(self):
        return list(self._t)

    def has(self, name):
        return name in self._t

    def shape(self, name):
        return tuple(self._t[name].shape)

    def dtype(self, name):
        return self._t[name].dtype

    def get(self, name):
        return self._t[name]


_FLOATS = (torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int8, torch.uint8, torch.int32, torch.int64)


class WeightStore:
    def __init__(self, source, description: str = "memory", strict: bool = False):
        self._src = source
        self.description = description
        self.strict = bool(strict)         # True: a tensor nobody asked for is an error of its own
        self._taken = set()
        self._missing: List[str] = []
        self._wrong_shape = []
        self._wrong_dtype = []
        self._ignored_patterns: List[str] = []

    # -------------------------------------------------------------- constructors
    @classmethod
    def from_dir(cls, model_dir: str, strict: bool = False) -> "WeightStore":
        return cls(SafetensorsDir(model_dir), description=model_dir, strict=strict)

    @classmethod
    def from_tensors(cls, tensors: Mapping[str, torch.Tensor], description: str = "memory",
                     strict: bool = False) -> "WeightStore":
        return cls(_DictSource(tensors), description=description, strict=strict)

    # ------------------------------------------------------------------- queries
    def has(self, name: str) -> bool:
        return self._src.has(name)

    def allow_unused(self, pattern: str) -> None:
        """Names matching ``pattern`` (fnmatch) may be present without being used."""
        self._ignored_patterns.append(pattern)

    def take(self, name: str, shape: Sequence[int], integer: bool = False) -> Optional[torch.Tensor]:
        """The tensor ``name`` with the stored precision kept, or None if it is missing or has
        the wrong shape (the problem is recorded for ``finish``)."""
        shape = tuple(int(s) for s in shape)
        self._taken.add(name)
        if not self._src.has(name):
            self._missing.append(name)
            return None
        have = tuple(self._src.shape(name))
        if have != shape:
            self._wrong_shape.append((name, have, shape))
            return None
        dt = self._src.dtype(name)
        if integer:
            if dt not in _INTS:
                self._wrong_dtype.append((name, str(dt)))
                return None
            return self._src.get(name).to(torch.int32)
        if dt not in _FLOATS:
            self._wrong_dtype.append((name, str(dt)))
            return None
        t = self._src.get(name)
        if dt == torch.float16:
            t = t.to(torch.bfloat16)
        return t

    def finish(self) -> None:
        """Raises ``WeightError`` if anything was missing or misshapen (the error lists left-over tensors too);
        left-over tensors alone give a warning, or the error if the store is strict."""
        unexpected = []
        for n in self._src.names():
            if n in self._taken:
                continue
            if any(fnmatch.fnmatchcase(n, p) for p in self._ignored_patterns):
                continue
            unexpected.append(n)
        if unexpected and not (self._missing or self._wrong_shape or self._wrong_dtype or self.strict):
            shown = ", ".join(sorted(unexpected)[:12]) + (f", ... and {len(unexpected) - 12} more" if len(unexpected) > 12 else "")
            warnings.warn(f"the weights in {self.description} hold {len(unexpected)} tensor(s) the model does not use: {shown}",
                          UnexpectedTensorsWarning, stacklevel=2)
            return
        if self._missing or self._wrong_shape or self._wrong_dtype or unexpected:
            raise WeightError(self.description, sorted(self._missing), sorted(unexpected),
                              sorted(self._wrong_shape), sorted(self._wrong_dtype))
