"""Arrangements: how a layer's parts are put around the residual stream.

An arrangement is a registered class (family "arrangement") built from a ``LayerSpec``.  It decides which *roles*
the layer's parts play, which family each role belongs to and in what order they run; the model above it only
asks it for its tensors, for what its mixers need of the cache, and to run.  ``Arrangement`` does the common work
(building the parts of the declared roles, declaring and loading their tensors, listing the mixers' cache needs); a
subclass states ``ROLES`` and ``forward``.

"prenorm" (src/backend/cpu/cpu_backend.cpp:139-213): h += mixer(norm_a(h)); h += ffn(norm_b(h)).
The residual stream is fp32; mixers and feed-forwards add into it through the epilogue of
their last product.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..config.spec import ConfigError
from .base import CacheNeed, Runtime, WeightDecl
from .registry import build_part, register_part


class Arrangement:
    """Base of arrangements.  ``ROLES`` maps every role the arrangement understands to its part family, in the
    order the parts are listed; ``OPTIONAL`` names roles a layer may leave out.

    A mixer's cache is known to the model by a *sub-id*: "" if the arrangement has a single mixer role, else the
    role's name.  ``forward`` receives ``caches``, a mapping from sub-id to the ``LayerCache`` of this layer (or of
    the layer whose cache the schedule tells this run to use)."""

    ROLES: Mapping[str, str] = {}
    OPTIONAL: frozenset = frozenset()

    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.parts: Dict[str, object] = {}
        for role, spec, prefix in layer_spec.parts:
            family = self.ROLES.get(role)
            if family is None:
                raise ConfigError(f"arrangement {layer_spec.arrangement!r} has no role {role!r} "
                                  f"(its roles: {', '.join(self.ROLES)})")
            self.parts[role] = build_part(family, spec, prefix)
        missing = [r for r in self.ROLES if r not in self.parts and r not in self.OPTIONAL]
        if missing:
            raise ConfigError(f"arrangement {layer_spec.arrangement!r} needs parts in the roles: {', '.join(missing)}")
        mixer_roles = [r for r, f in self.ROLES.items() if f == "mixer" and r in self.parts]
        self.mixers: Dict[str, object] = {("" if len(mixer_roles) == 1 else r): self.parts[r] for r in mixer_roles}

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step through this block may be captured into a CUDA graph: every part must allow it
        (an arrangement whose own ``forward`` reads host views overrides this with False)."""
        return all(getattr(p, "graph_safe", False) for p in self.parts.values())

    def weight_decls(self) -> List[WeightDecl]:
        return [d for p in self.parts.values() for d in p.weight_decls()]

    def load(self, store, rt: Runtime) -> None:
        self.rt = rt
        for p in self.parts.values():
            p.load(store, rt)

    def cache_needs(self) -> Dict[str, Optional[CacheNeed]]:
        """What each mixer of the block asks of the cache manager, by sub-id."""
        return {sub: m.cache_need() for sub, m in self.mixers.items()}

    def tile_requests(self):
        """Attention tile shapes the block's mixers will ask the step context for."""
        keys = []
        for m in self.mixers.values():
            fn = getattr(m, "tile_requests", None)
            for k in (fn() if fn else ()):
                if k not in keys:
                    keys.append(k)
        return keys

    def forward(self, ctx, h: torch.Tensor, caches: Mapping[str, object], owns_cache: bool = True) -> None:
        raise NotImplementedError


class PreNormBlock(Arrangement):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, layer_spec):
        super().__init__(layer_spec)
        self.mixer_norm, self.mixer = self.parts["mixer_norm"], self.parts["mixer"]
        self.feed_forward_norm, self.feed_forward = self.parts["feed_forward_norm"], self.parts["feed_forward"]

    def forward(self, ctx, h: torch.Tensor, caches, owns_cache: bool = True) -> None:
        x = ctx.buf("block.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
        self.mixer_norm.forward(ctx, h, x, ctx.T)
        self.mixer.forward(ctx, x, h, caches[""], owns_cache)
        self.feed_forward_norm.forward(ctx, h, x, ctx.T)
        self.feed_forward.forward(ctx, x, h)


register_part("arrangement", "prenorm", PreNormBlock)
