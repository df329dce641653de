"""What every part is: a spec, the tensors it declares, device copies, and a forward.

A part is built from its spec alone (no device needed), so a model's tensor names and
shapes can be listed — for loading, for the error that lists what is missing, and for the
random-weights mode — before anything touches a GPU.  ``load`` makes the device copies.

Interfaces (what a new part must provide):

* ``Norm``:          ``forward(ctx, x_f32[rows, size], out[n_rows, size], n_rows, rows=None)``
* ``PositionEncoding``: ``rotary_table(rt) -> (inv_freq_f32[rotary/2] | None, rotary_dim)``; encodings that
  act elsewhere may instead override ``on_embedding(ctx, h)``.  ``table_key()`` says which layers' frequencies are
  the same (they share the step's angle table that ``cos_sin`` makes from ``rotary_table``).
* ``Norm`` may also provide ``scale_output(scale)`` (needed only as the final norm of a model with a logit scale).
* ``Mixer``:         ``cache_need() -> CacheNeed | None`` and
  ``forward(ctx, x[T, hidden], residual_f32[T, hidden], cache: LayerCache | None, owns_cache: bool)``;
  it *adds* its result to ``residual``.
* ``FeedForward``:   ``forward(ctx, x[T, hidden], residual_f32[T, hidden])``; it adds its result.

No part knows which model it is in: sizes and constants come from its spec, weights from the
names under the prefix it is given.  A part whose ``forward`` only launches kernels that read the step's
indices on the device sets ``graph_safe = True``; decode steps of a model are captured into CUDA graphs only if
every part of it says so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class WeightDecl:
    """A tensor a part reads: its full name, shape, and how the random-weights mode fills it."""

    name: str
    shape: Tuple[int, ...]
    init: str = "linear"      # "linear": N(0, std) | "norm": 1 + N(0, norm_std) | "zeros"
    optional: bool = False    # may be absent from the file (the part then does without)


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache manager, per layer.

    kind "full":   pages holding every key/value of the request.
    kind "window": pages holding the last ``window`` keys; older pages are given back.
    kind "state":  no pages; one slot of ``state_shape`` elements of ``state_dtype`` per request.
    Layers whose needs are equal share a group (one block table, one page pool per group).
    """

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"


@dataclass
class Runtime:
    """Where and how a model computes."""

    device: torch.device
    dtype: torch.dtype                 # activations and cache: torch.bfloat16 (serving) or torch.float32
    page_tokens: int = 16

    def weight_dtype(self, stored: torch.dtype) -> torch.dtype:
        """Matrix weights: widened to float32 on the float32 path, stored precision kept otherwise."""
        if self.dtype == torch.float32:
            return torch.float32
        return torch.float32 if stored == torch.float32 else torch.bfloat16

    def to_device(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        return t.to(device=self.device, dtype=dtype).contiguous()


class Part:
    family = ""
    # Whether ``forward`` may be captured into a CUDA graph and replayed for later steps: true only if it does
    # nothing but launch work on ``ctx.stream`` whose indices (positions, slots, block tables, run offsets) are
    # read on the device from the step's uploaded arrays.  A part that reads the step's host views
    # (``ctx.query_start_host``, ``ctx.state_slots_host``, ...) or synchronises bakes one step's values into the
    # graph, so the default is False and a model with such a part decodes without graphs.
    graph_safe = False

    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec = spec
        self.prefix = prefix

    def weight_decls(self) -> List[WeightDecl]:
        return []

    def load(self, store, rt: Runtime) -> None:
        """Takes the declared tensors from ``store`` and makes device copies."""

    def workspace_need(self, max_tokens: int, rt: Runtime) -> None:
        return None


class Norm(Part):
    family = "norm"

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def scale_output(self, scale: float) -> None:
        """After ``load``: makes the norm's output ``scale`` times what it was (a model's logit scale is applied
        this way to its final norm).  A norm that ends in a weight folds the factor into it."""
        raise NotImplementedError(f"{type(self).__name__} cannot scale its output")


class PositionEncoding(Part):
    family = "position"

    def rotary_table(self, rt: Runtime):
        """(inv_freq float32 device tensor of rotary_dim/2, rotary_dim), or (None, 0) for no rotation."""
        return None, 0

    def on_embedding(self, ctx, h: torch.Tensor) -> None:
        """Hook for encodings that are added to the embedded tokens; rotary ones do nothing here."""

    def table_key(self):
        """What tells this part's frequencies from another's: layers whose keys are equal share a step's angle
        table.  Unknown parts share nothing."""
        return id(self)

    def cos_sin(self, ctx, rt: Runtime) -> torch.Tensor:
        """[rotary / 4, tokens, 4]: (cos, cos, sin, sin) of float(position) * inv_freq for pairs of frequencies (the
        layout of ``ops.rope_table``), made once per step for the products that rotate in their epilogue and kept
        in the step's memo."""
        from .. import ops
        inv, _ = self.rotary_table(rt)
        key = ("rope.cos_sin", self.table_key())
        got = ctx.memo.get(key)
        if got is None:
            half = inv.numel()
            got = ctx.buf(f"rope.cos_sin.{key[1]}", (half // 2, ctx.max_tokens, 4), torch.float32)
            ops.rope_table(ctx.positions, inv, ctx.T, got, stream=ctx.stream)
            ctx.memo[key] = got
        return got


class Mixer(Part):
    family = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, cache, owns_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    family = "feed_forward"

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError
