"""Gated feed-forward (SwiGLU): h += down( silu(gate(x)) * up(x) ), no biases.

Formula: src/backend/cpu/cpu_backend.cpp:204-211 with silu(g) = g / (1 + exp(-g)).
Device layout: gate and up rows are interleaved (even rows gate, odd rows up) into one
[2 * intermediate, hidden] matrix, so one product yields adjacent (gate, up) pairs and the
activation is the product's epilogue.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import FeedForward, Runtime, WeightDecl
from .linear import Linear
from .registry import register_part


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        if spec.activation != "silu":
            raise ConfigError(f"activation {spec.activation!r} is not supported (silu only)")

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        return [WeightDecl(p + "gate_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightDecl(p + "up_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightDecl(p + "down_proj.weight", (s.hidden_size, s.intermediate_size))]

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        gate = store.take(p + "gate_proj.weight", (s.intermediate_size, s.hidden_size))
        up = store.take(p + "up_proj.weight", (s.intermediate_size, s.hidden_size))
        down = store.take(p + "down_proj.weight", (s.hidden_size, s.intermediate_size))
        if gate is None or up is None or down is None:
            return
        wd = rt.weight_dtype(torch.result_type(gate, up))
        gu = torch.stack([rt.to_device(gate, wd), rt.to_device(up, wd)], dim=1)   # [I, 2, H]
        self.gate_up = Linear(gu.reshape(2 * s.intermediate_size, s.hidden_size).contiguous())
        self.down = Linear.from_host(down, rt)

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor) -> None:
        s = self.spec
        act = ctx.buf("gated_mlp.act", (ctx.max_tokens, s.intermediate_size), self.rt.dtype)
        self.gate_up(ctx, x, act, ctx.T, ops.EPI_SILU_MUL)
        self.down(ctx, act, residual, ctx.T, ops.EPI_ADD_F32)


register_part("feed_forward", "gated_mlp", GatedMLP)
