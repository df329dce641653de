"""Arrangements: how a layer's parts are put around the residual stream.

"prenorm" (src/backend/cpu/cpu_backend.cpp:139-213): h += mixer(norm_a(h)); h += ffn(norm_b(h)).
The residual stream is fp32; mixers and feed-forwards add into it through the epilogue of
their last product.
"""
from __future__ import annotations

from typing import List

import torch

from .base import Runtime, WeightDecl
from .registry import build_part, register_part


class PreNormBlock:
    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, layer_spec.mixer_norm_prefix)
        self.mixer = build_part("mixer", layer_spec.mixer, layer_spec.mixer_prefix)
        self.feed_forward_norm = build_part("norm", layer_spec.feed_forward_norm, layer_spec.feed_forward_norm_prefix)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, layer_spec.feed_forward_prefix)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def weight_decls(self) -> List[WeightDecl]:
        return [d for p in self.parts() for d in p.weight_decls()]

    def load(self, store, rt: Runtime) -> None:
        self.rt = rt
        for p in self.parts():
            p.load(store, rt)

    def forward(self, ctx, h: torch.Tensor, cache, owns_cache: bool = True) -> None:
        x = ctx.buf("block.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
        self.mixer_norm.forward(ctx, h, x, ctx.T)
        self.mixer.forward(ctx, x, h, cache, owns_cache)
        self.feed_forward_norm.forward(ctx, h, x, ctx.T)
        self.feed_forward.forward(ctx, x, h)


register_part("arrangement", "prenorm", PreNormBlock)
