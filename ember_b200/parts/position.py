"""Position encodings.

Rotary, rotate-half layout (src/backend/cpu/cpu_backend.cpp:85-88, 263-272):
inv_freq_i = 1 / powf(float(theta), float(2i) / float(rotary_dim)) computed in fp32; the angle
float(pos) * inv_freq_i and its sine and cosine are fp32; pairs are (x_i, x_{i + rotary_dim/2}).
The rotation itself runs inside the mixer's fused norm + rotation + cache-write kernel; this
part owns the frequency table, so an encoding with other frequencies (or none) is another
part with the same interface.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config.spec import ConfigError
from .base import PositionEncoding, Runtime
from .registry import register_part


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self._table = None

    def inv_freq(self) -> np.ndarray:
        r = self.spec.rotary_dim
        i = np.arange(r // 2, dtype=np.float32)
        exponent = (np.float32(2.0) * i) / np.float32(r)                      # float(2i) / float(D)
        return (np.float32(1.0) / np.power(np.float32(self.spec.theta), exponent, dtype=np.float32)).astype(np.float32)

    def rotary_table(self, rt: Runtime):
        if self._table is None or self._table.device != rt.device:
            self._table = torch.from_numpy(self.inv_freq()).to(rt.device)
        return self._table, self.spec.rotary_dim

    def table_key(self):
        return (self.spec.rotary_dim, float(self.spec.theta))        # equal frequencies: one table a step


class NoPosition(PositionEncoding):
    graph_safe = True


register_part("position", "rope", RotaryEmbedding)
register_part("position", "none", NoPosition)
