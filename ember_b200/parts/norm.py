"""RMSNorm: out = weight * (x * rsqrt(mean(x^2) + eps)), statistics in fp32.

Formula: src/backend/cpu/cpu_backend.cpp:34-39 (the weight multiplies after the scaling; it
is the plain weight, not 1 + weight).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Norm, Runtime, WeightDecl
from .registry import register_part


class RMSNorm(Norm):
    graph_safe = True

    def weight_decls(self) -> List[WeightDecl]:
        return [WeightDecl(self.prefix + "weight", (self.spec.size,), init="norm")]

    def load(self, store, rt: Runtime) -> None:
        w = store.take(self.prefix + "weight", (self.spec.size,))
        self.weight = rt.to_device(w, torch.float32) if w is not None else None

    def scale_output(self, scale: float) -> None:
        if self.weight is not None:
            self.weight = self.weight * scale

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, self.spec.eps, out, n_rows, rows=rows, stream=ctx.stream)


register_part("norm", "rmsnorm", RMSNorm)
