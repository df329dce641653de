"""Host-side bookkeeping of the cache: pages, block tables, groups, state slots.

Keys and values live in pages of ``page_tokens`` tokens.  Layers whose needs are equal
(``CacheNeed``: all keys, or a window of them, with the same head geometry) form a *group*;
every group has its own page pool and every request has one block table per group.  Pages are
given back when a request ends, when it is preempted, and — in a window group — as soon as
every key on them is older than the window; freed pages are handed out again (most recently
freed first).  Beside the pages, every admitted request holds one *slot* for state of fixed
size; mixers of kind "state" keep their per-request tensors there.

The manager owns no memory: ``ember_b200.cache.storage`` allocates the device tensors the ids
point into.  (Page accounting in the reference: src/kvcache/block_manager.{hpp,cpp},
src/engine/engine.cpp:176-184; groups, windows and slots have no counterpart there.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from ..parts.base import CacheNeed


class CacheError(RuntimeError):
    pass


class PagePool:
    """Ids 0..n-1; low ids first from a fresh pool, then most recently freed first."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise CacheError("a pool cannot have a negative number of pages")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return self.n_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            return -1
        p = self._free.pop()
        self._held[p] = True
        return p

    def release(self, page: int) -> None:
        if not (0 <= page < self.n_pages):
            raise CacheError(f"page {page} is outside the pool of {self.n_pages}")
        if not self._held[page]:
            raise CacheError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> str:
        seen = set()
        for p in self._free:
            if p in seen:
                return f"page {p} is on the free list twice"
            seen.add(p)
            if self._held[p]:
                return f"page {p} is both free and held"
        held = sum(self._held)
        if held + len(self._free) != self.n_pages:
            return f"{held} held + {len(self._free)} free != {self.n_pages} pages (a page is lost)"
        return ""


@dataclass
class CacheGroup:
    index: int
    need: CacheNeed
    layers: List[int]
    page_tokens: int
    pool: Optional[PagePool]       # None for kind "state"

    @property
    def paged(self) -> bool:
        return self.need.kind in ("full", "window")


@dataclass
class RequestCache:
    slot: int
    tables: List[List[int]]        # per group: physical page of each logical page, -1 once given back
    first_live: List[int]          # per group: first logical page still held
    tokens: int = 0                # tokens whose keys are in the cache
    arrays: List[np.ndarray] = field(default_factory=list)   # per group: int32 mirror of `tables` (grown by doubling)
    addrs: List[int] = field(default_factory=list)           # per group: address of the mirror (for the native packer)

    def table_array(self, group: int) -> np.ndarray:
        """The group's block table as an int32 array (a view: valid until the table changes)."""
        n = len(self.tables[group])
        return self.arrays[group][:n]

    def _mirror_append(self, group: int, page: int) -> None:
        n = len(self.tables[group])          # the list already holds the new page at n - 1
        a = self.arrays[group]
        if n > a.shape[0]:
            b = np.full(max(16, 2 * a.shape[0]), -1, dtype=np.int32)
            b[:a.shape[0]] = a
            self.arrays[group] = a = b
            self.addrs[group] = a.ctypes.data
        a[n - 1] = page


def group_needs(needs: Mapping[int, Optional[CacheNeed]]) -> List[Tuple[CacheNeed, List[int]]]:
    """Groups layers by equal need, in order of first appearance."""
    out: List[Tuple[CacheNeed, List[int]]] = []
    for layer in sorted(needs):
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
        self.page_tokens = page_tokens
        self.max_requests = max_requests
        self.groups: List[CacheGroup] = []
        for gi, (need, layers) in enumerate(group_needs(needs)):
            if need.kind not in ("full", "window", "state"):
                raise CacheError(f"unknown cache need {need.kind!r}")
            pool = None
            if need.kind != "state":
                n = pages_per_group[gi] if pages_per_group is not None else capacity_tokens // page_tokens
                pool = PagePool(int(n))
            self.groups.append(CacheGroup(gi, need, layers, page_tokens, pool))
        self.layer_group: Dict[int, int] = {l: g.index for g in self.groups for l in g.layers}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, RequestCache] = {}

    # ---------------------------------------------------------------- requests
    def has(self, request: Hashable) -> bool:
        return request in self._requests

    def get(self, request: Hashable) -> RequestCache:
        try:
            return self._requests[request]
        except KeyError:
            raise CacheError(f"request {request!r} holds no cache") from None

    def admit(self, request: Hashable) -> Optional[RequestCache]:
        """Gives the request a state slot and empty block tables; None if no slot is free."""
        if request in self._requests:
            raise CacheError(f"request {request!r} is admitted twice")
        if not self._free_slots:
            return None
        arrays = [np.full(16, -1, dtype=np.int32) for _ in self.groups]
        rc = RequestCache(slot=self._free_slots.pop(), tables=[[] for _ in self.groups],
                          first_live=[0 for _ in self.groups], arrays=arrays,
                          addrs=[a.ctypes.data for a in arrays])
        self._requests[request] = rc
        return rc

    def pages_needed(self, request: Hashable, upto_tokens: int) -> List[int]:
        rc = self.get(request)
        want = (upto_tokens + self.page_tokens - 1) // self.page_tokens
        return [max(0, want - len(rc.tables[g.index])) if g.paged else 0 for g in self.groups]

    def ensure(self, request: Hashable, upto_tokens: int) -> bool:
        """Makes sure pages exist for tokens [0, upto_tokens) in every paged group (all or nothing)."""
        rc = self.get(request)
        need = self.pages_needed(request, upto_tokens)
        for g, n in zip(self.groups, need):
            if g.paged and g.pool.available < n:
                return False
        for g, n in zip(self.groups, need):
            for _ in range(n):
                page = g.pool.allocate()
                rc.tables[g.index].append(page)
                rc._mirror_append(g.index, page)
        return True

    def advance(self, request: Hashable, tokens: int) -> int:
        """Records that ``tokens`` tokens are now cached; gives back window pages no later query
        can see.  Returns how many pages were freed."""
        rc = self.get(request)
        rc.tokens = tokens
        freed = 0
        for g in self.groups:
            if g.need.kind != "window":
                continue
            # the next query is at position >= tokens and sees keys > position - window
            first_key = max(0, tokens - g.need.window + 1)
            dead = first_key // self.page_tokens
            table = rc.tables[g.index]
            for i in range(rc.first_live[g.index], min(dead, len(table))):
                if table[i] >= 0:
                    g.pool.release(table[i])
                    table[i] = -1
                    rc.arrays[g.index][i] = -1
                    freed += 1
            rc.first_live[g.index] = max(rc.first_live[g.index], min(dead, len(table)))
        return freed

    def release(self, request: Hashable) -> None:
        """Gives back everything the request holds (pages in reverse order, then its slot)."""
        rc = self._requests.pop(request, None)
        if rc is None:
            raise CacheError(f"request {request!r} is released but holds nothing")
        for g in self.groups:
            if not g.paged:
                continue
            for p in reversed(rc.tables[g.index]):
                if p >= 0:
                    g.pool.release(p)
        self._free_slots.append(rc.slot)

    def reset(self, request: Hashable) -> None:
        """Preemption: pages go back, the slot stays with the request."""
        rc = self.get(request)
        for g in self.groups:
            if g.paged:
                for p in reversed(rc.tables[g.index]):
                    if p >= 0:
                        g.pool.release(p)
            rc.tables[g.index] = []
            rc.first_live[g.index] = 0
        rc.tokens = 0

    # ------------------------------------------------------------------ queries
    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def available_pages(self) -> List[int]:
        return [g.pool.available if g.paged else 0 for g in self.groups]

    def used_pages(self) -> List[int]:
        return [g.pool.used if g.paged else 0 for g in self.groups]

    def capacity_tokens(self) -> int:
        paged = [g.pool.n_pages * self.page_tokens for g in self.groups if g.paged and g.need.kind == "full"]
        return min(paged) if paged else 1 << 30

    def check(self) -> str:
        """Audit: every page is free or held by exactly one request; every slot likewise."""
        for g in self.groups:
            if not g.paged:
                continue
            msg = g.pool.check()
            if msg:
                return f"group {g.index}: {msg}"
            owners: Dict[int, Hashable] = {}
            for req, rc in self._requests.items():
                for p in rc.tables[g.index]:
                    if p < 0:
                        continue
                    if p in owners:
                        return f"group {g.index}: page {p} is held by {owners[p]!r} and {req!r}"
                    owners[p] = req
                    if not g.pool.is_held(p):
                        return f"group {g.index}: page {p} of {req!r} is on the free list"
            if len(owners) != g.pool.used:
                return f"group {g.index}: {g.pool.used} pages are out but requests hold {len(owners)}"
        slots = [rc.slot for rc in self._requests.values()]
        if len(set(slots)) != len(slots):
            return "a state slot is held twice"
        if set(slots) & set(self._free_slots):
            return "a state slot is both held and free"
        if len(slots) + len(self._free_slots) != self.max_requests:
            return "a state slot is lost"
        return ""
