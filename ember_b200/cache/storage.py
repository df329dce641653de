"""Device memory behind the cache manager's ids.

Per paged group one tensor [layers_in_group, 2 (key, value), pages, kv_heads, page_tokens,
head_dim] in the compute dtype, zero-filled so that a slot never written holds no NaN (the
reference zero-fills too: src/backend/cuda/cuda_backend.cu:757-780).  Per state group one
tensor [layers_in_group, slots, *state_shape].  A ``LayerCache`` is the view one layer's mixer
gets.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .manager import CacheManager


@dataclass
class LayerCache:
    group: int
    page_tokens: int
    k: Optional[torch.Tensor] = None        # [pages, kv_heads, page_tokens, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None    # [slots, *state_shape]


def cache_bytes_per_token(needs, dtype: torch.dtype) -> int:
    """Bytes of device memory one cached token takes over all paged groups (every group's pool is made for the
    same number of tokens): keys and values of every layer of the group.  ``needs`` is what
    ``CausalLM.cache_needs`` returns."""
    elem = torch.empty(0, dtype=dtype).element_size()
    return sum(2 * n.num_kv_heads * n.head_dim * elem for n in needs.values() if n is not None and n.kind in ("full", "window"))


def state_bytes_per_request(needs) -> int:
    """Bytes of fixed-size state one request's slot takes over all state groups."""
    total = 0
    for n in needs.values():
        if n is not None and n.kind == "state":
            size = torch.empty(0, dtype=getattr(torch, n.state_dtype)).element_size()
            for d in n.state_shape:
                size *= int(d)
            total += size
    return total


class CacheStorage:
    def __init__(self, manager: CacheManager, device: torch.device, dtype: torch.dtype):
        self.manager = manager
        self.device = device
        self.dtype = dtype
        self._paged: Dict[int, torch.Tensor] = {}
        self._state: Dict[int, torch.Tensor] = {}
        for g in manager.groups:
            if g.paged:
                n = g.need
                self._paged[g.index] = torch.zeros(
                    (len(g.layers), 2, max(1, g.pool.n_pages), n.num_kv_heads, g.page_tokens, n.head_dim),
                    dtype=dtype, device=device)
            else:
                sd = getattr(torch, g.need.state_dtype)
                self._state[g.index] = torch.zeros((len(g.layers), manager.max_requests) + tuple(g.need.state_shape),
                                                   dtype=sd, device=device)

    def layer(self, layer) -> Optional[LayerCache]:
        """The cache of one mixer, by cache id (a layer index, or (layer, sub-id)); None if it owns none."""
        gi = self.manager.layer_group.get(layer)
        if gi is None:
            return None
        g = self.manager.groups[gi]
        li = g.layers.index(layer)
        if g.paged:
            t = self._paged[gi]
            return LayerCache(group=gi, page_tokens=g.page_tokens, k=t[li, 0], v=t[li, 1])
        return LayerCache(group=gi, page_tokens=g.page_tokens, state=self._state[gi][li])

    def reset_slot(self, slot: int) -> None:
        """Zeroes a request's fixed-size state in every state group (at admission)."""
        for t in self._state.values():
            t[:, slot].zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self._paged.values()) + list(self._state.values()))
