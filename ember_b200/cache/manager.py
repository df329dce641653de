"""Host-side bookkeeping of the cache: pages, block tables, groups, state slots.

Keys and values live in pages of ``page_tokens`` tokens.  Layers whose needs are equal
(``CacheNeed``: all keys, or a window of them, with the same head geometry) form a *group*;
every group has its own page pool and every request has one block table per group.  Pages are
given back when a request ends, when it is preempted, and — in a window group — as soon as
every key on them is older than the window; freed pages are handed out again (most recently
freed first).  Beside the pages, every admitted request holds one *slot* for state of fixed
size; mixers of kind "state" keep their per-request tensors there.

The books themselves are kept natively (``ember_b200/runtime/cache_core.cpp``, as the reference
keeps its own in C++: src/kvcache/block_manager.{hpp,cpp}, src/engine/engine.cpp:176-184; groups,
windows and slots have no counterpart there).  This module is their Python face: it names
requests by any hashable key, groups layers by need, and turns return codes into ``CacheError``.
The manager owns no device memory: ``ember_b200.cache.storage`` allocates the tensors the ids
point into.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int32
from dataclasses import dataclass
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from ..parts.base import CacheNeed
from ..runtime import library

_KINDS = {"full": 0, "window": 1, "state": 2}


class CacheError(RuntimeError):
    pass


def _message(fn, handle) -> str:
    buf = ctypes.create_string_buffer(256)
    fn(handle, buf, 256)
    return buf.value.decode("utf-8", "replace")


class PagePool:
    """Ids 0..n-1; low ids first from a fresh pool, then most recently freed first."""

    def __init__(self, n_pages: int, _native=None, _owner=None):
        if n_pages < 0:
            raise CacheError("a pool cannot have a negative number of pages")
        self._lib = library()
        self.n_pages = int(n_pages)
        self._owner = _owner                 # a pool inside a manager lives and dies with it
        self._own = _native is None
        self._p = _native if _native is not None else self._lib.ember_pool_create(self.n_pages)

    def __del__(self):
        if getattr(self, "_own", False) and self._p:
            self._lib.ember_pool_destroy(self._p)
            self._p = None

    @property
    def available(self) -> int:
        return self._lib.ember_pool_available(self._p)

    @property
    def used(self) -> int:
        return self.n_pages - self.available

    def allocate(self) -> int:
        return self._lib.ember_pool_allocate(self._p)

    def release(self, page: int) -> None:
        code = self._lib.ember_pool_release(self._p, int(page))
        if code == 1:
            raise CacheError(f"page {page} is outside the pool of {self.n_pages}")
        if code == 2:
            raise CacheError(f"page {page} is freed twice")

    def is_held(self, page: int) -> bool:
        return bool(self._lib.ember_pool_is_held(self._p, int(page)))

    def check(self) -> str:
        return _message(self._lib.ember_pool_check, self._p)


@dataclass
class CacheGroup:
    index: int
    need: CacheNeed
    layers: List[object]           # cache ids: layer indices, or (layer, sub-id) pairs
    page_tokens: int
    pool: Optional[PagePool]       # None for kind "state"

    @property
    def paged(self) -> bool:
        return self.need.kind in ("full", "window")


class RequestCache:
    """What one admitted request holds: a view of the native record."""

    __slots__ = ("_m", "handle", "slot", "tokens")

    def __init__(self, manager: "CacheManager", handle: int, slot: int):
        self._m = manager
        self.handle = handle
        self.slot = slot
        self.tokens = 0                # tokens whose keys are in the cache (kept in step by the manager)

    def table_array(self, group: int) -> np.ndarray:
        """The group's block table as an int32 array (a copy): physical page of each logical page, -1 once
        given back."""
        ptr = POINTER(c_int32)()
        n = self._m._lib.ember_cache_table(self._m.core, self.handle, group, ctypes.byref(ptr))
        if n <= 0:
            return np.zeros(0, dtype=np.int32)
        return np.ctypeslib.as_array(ptr, shape=(n,)).copy()

    @property
    def tables(self) -> List[List[int]]:
        return [self.table_array(g).tolist() for g in range(len(self._m.groups))]

    @property
    def first_live(self) -> List[int]:
        return [self._m._lib.ember_cache_first_live(self._m.core, self.handle, g) for g in range(len(self._m.groups))]


def _cache_id_order(cache_id):
    """Cache ids are layer indices, or (layer, sub-id) for a layer with several mixers: ordered by layer."""
    return (cache_id, "") if isinstance(cache_id, int) else (cache_id[0], str(cache_id[1]))


def group_needs(needs: Mapping[object, Optional[CacheNeed]]) -> List[Tuple[CacheNeed, List[object]]]:
    """Groups caches (one per layer, or per mixer of a layer that has several) by equal need, in order of first
    appearance."""
    out: List[Tuple[CacheNeed, List[object]]] = []
    for layer in sorted(needs, key=_cache_id_order):
        n = needs[layer]
        if n is None:
            continue
        for need, layers in out:
            if need == n:
                layers.append(layer)
                break
        else:
            out.append((n, [layer]))
    return out


class CacheManager:
    def __init__(self, needs: Mapping[int, Optional[CacheNeed]], page_tokens: int, capacity_tokens: int,
                 max_requests: int, pages_per_group: Optional[Sequence[int]] = None):
        if page_tokens <= 0:
            raise CacheError("page_tokens must be positive")
        self._lib = library()
        self.page_tokens = page_tokens
        self.max_requests = max_requests
        grouped = group_needs(needs)
        kinds, windows, pages = [], [], []
        for gi, (need, _) in enumerate(grouped):
            if need.kind not in _KINDS:
                raise CacheError(f"unknown cache need {need.kind!r}")
            n = 0
            if need.kind != "state":
                n = int(pages_per_group[gi] if pages_per_group is not None else capacity_tokens // page_tokens)
                if n < 0:
                    raise CacheError("a pool cannot have a negative number of pages")
            kinds.append(_KINDS[need.kind])
            windows.append(int(getattr(need, "window", 0) or 0))
            pages.append(n)
        G = len(grouped)
        arr = lambda v: (c_int32 * max(G, 1))(*v)          # noqa: E731
        self.core = self._lib.ember_cache_create(G, arr(kinds), arr(windows), arr(pages), int(page_tokens), int(max_requests))
        if not self.core:
            raise CacheError("the cache core could not be created")
        self.groups: List[CacheGroup] = []
        for gi, (need, layers) in enumerate(grouped):
            pool = None
            if need.kind != "state":
                pool = PagePool(pages[gi], _native=self._lib.ember_cache_pool(self.core, gi), _owner=self)
            self.groups.append(CacheGroup(gi, need, layers, page_tokens, pool))
        self.layer_group: Dict[object, int] = {l: g.index for g in self.groups for l in g.layers}
        self._requests: Dict[Hashable, RequestCache] = {}

    def __del__(self):
        core, self.core = getattr(self, "core", None), None
        if core:
            self._lib.ember_cache_destroy(core)

    # ---------------------------------------------------------------- requests
    def has(self, request: Hashable) -> bool:
        return request in self._requests

    def get(self, request: Hashable) -> RequestCache:
        try:
            return self._requests[request]
        except KeyError:
            raise CacheError(f"request {request!r} holds no cache") from None

    def handle_of(self, request: Hashable) -> int:
        """The native handle of an admitted request (what the step packer passes back to the core)."""
        return self.get(request).handle

    def admit(self, request: Hashable) -> Optional[RequestCache]:
        """Gives the request a state slot and empty block tables; None if no slot is free."""
        if request in self._requests:
            raise CacheError(f"request {request!r} is admitted twice")
        h = self._lib.ember_cache_admit(self.core)
        if h < 0:
            return None
        rc = RequestCache(self, h, self._lib.ember_cache_slot(self.core, h))
        self._requests[request] = rc
        return rc

    def pages_needed(self, request: Hashable, upto_tokens: int) -> List[int]:
        rc = self.get(request)
        want = (upto_tokens + self.page_tokens - 1) // self.page_tokens
        return [max(0, want - self._lib.ember_cache_table(self.core, rc.handle, g.index, None)) if g.paged else 0
                for g in self.groups]

    def ensure(self, request: Hashable, upto_tokens: int) -> bool:
        """Makes sure pages exist for tokens [0, upto_tokens) in every paged group (all or nothing)."""
        return self._lib.ember_cache_ensure(self.core, self.get(request).handle, int(upto_tokens)) == 1

    def advance(self, request: Hashable, tokens: int) -> int:
        """Records that ``tokens`` tokens are now cached; gives back window pages no later query
        can see.  Returns how many pages were freed."""
        rc = self.get(request)
        rc.tokens = int(tokens)
        return self._lib.ember_cache_advance(self.core, rc.handle, rc.tokens)

    def release(self, request: Hashable) -> None:
        """Gives back everything the request holds (pages in reverse order, then its slot)."""
        rc = self._requests.pop(request, None)
        if rc is None:
            raise CacheError(f"request {request!r} is released but holds nothing")
        self._lib.ember_cache_release(self.core, rc.handle)

    def reset(self, request: Hashable) -> None:
        """Preemption: pages go back, the slot stays with the request."""
        rc = self.get(request)
        self._lib.ember_cache_reset(self.core, rc.handle)
        rc.tokens = 0

    # ------------------------------------------------------------------ queries
    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def free_slots(self) -> int:
        return self._lib.ember_cache_free_slots(self.core)

    def available_pages(self) -> List[int]:
        return [g.pool.available if g.paged else 0 for g in self.groups]

    def used_pages(self) -> List[int]:
        return [g.pool.used if g.paged else 0 for g in self.groups]

    def capacity_tokens(self) -> int:
        paged = [g.pool.n_pages * self.page_tokens for g in self.groups if g.paged and g.need.kind == "full"]
        return min(paged) if paged else 1 << 30

    def check(self) -> str:
        """Audit: every page is free or held by exactly one request; every slot likewise; and the
        requests known here are the ones the core holds."""
        msg = _message(self._lib.ember_cache_check, self.core)
        if msg:
            return msg
        if len(self._requests) + self.free_slots() != self.max_requests:
            return "the requests known to the manager and the slots held in the core differ"
        return ""
