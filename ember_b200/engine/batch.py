"""The ragged batch of one step, on the host and on the device.

A step holds S runs; run s is ``n`` consecutive new tokens of one request at consecutive
absolute positions — a portion of a prompt, one decoded token, or anything between (the
reference's StepBatch: src/backend/backend.hpp:56-76).  ``StepBatch`` is the host form built
from (request, tokens, wanted rows) entries and the cache manager's tables; ``StepContext`` is
its device form plus the step's scratch buffers, handed to every part.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager


class BatchError(ValueError):
    pass


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    requests: List[Hashable]
    tokens: np.ndarray            # [T] int32
    positions: np.ndarray         # [T] int32 absolute position of each token
    seq_of: np.ndarray            # [T] int32 run index of each token
    query_start: np.ndarray       # [S+1] int32
    context_len: np.ndarray       # [S] int32 tokens cached after this step
    block_tables: List[np.ndarray]  # per cache group [S, max_blocks_g] int32 (-1 = none / given back)
    state_slots: np.ndarray       # [S] int32
    logit_rows: np.ndarray        # [R] int32 token indices in output order

    @property
    def T(self) -> int:
        return int(self.tokens.shape[0])

    @property
    def S(self) -> int:
        return int(self.context_len.shape[0])

    @property
    def R(self) -> int:
        return int(self.logit_rows.shape[0])


def build_batch(entries: Sequence[StepEntry], cache: CacheManager, vocab_size: int,
                max_positions: Optional[int] = None) -> StepBatch:
    """Checks the entries, reads each request's cached length and tables from ``cache`` (pages
    for the new tokens must already be ensured) and lays the batch out."""
    if not entries:
        raise BatchError("a step needs at least one entry")
    seen = set()
    tokens: List[int] = []
    positions: List[int] = []
    seq_of: List[int] = []
    query_start = [0]
    context_len: List[int] = []
    slots: List[int] = []
    rows: List[int] = []
    tables: List[List[List[int]]] = [[] for _ in cache.groups]
    for s, e in enumerate(entries):
        if e.request in seen:
            raise BatchError(f"request {e.request!r} appears twice in one step")
        seen.add(e.request)
        n = len(e.tokens)
        if n == 0:
            raise BatchError(f"request {e.request!r} brings no tokens")
        rc = cache.get(e.request)
        start = rc.tokens
        if max_positions is not None and start + n > max_positions:
            raise BatchError(f"request {e.request!r} would reach position {start + n}; the model's limit is {max_positions}")
        for g in cache.groups:
            if g.paged and len(rc.tables[g.index]) * cache.page_tokens < start + n:
                raise BatchError(f"request {e.request!r} has no pages for tokens up to {start + n}")
        for i, t in enumerate(e.tokens):
            t = int(t)
            if not (0 <= t < vocab_size):
                raise BatchError(f"token id {t} is out of range (vocabulary {vocab_size})")
            tokens.append(t)
            positions.append(start + i)
            seq_of.append(s)
        for w in e.want:
            w = int(w)
            if not (0 <= w < n):
                raise BatchError(f"request {e.request!r} wants row {w} of {n} tokens")
            rows.append(query_start[-1] + w)
        query_start.append(query_start[-1] + n)
        context_len.append(start + n)
        slots.append(rc.slot)
        for g in cache.groups:
            tables[g.index].append(rc.tables[g.index])
    bt = []
    for g in cache.groups:
        width = max(1, max(len(t) for t in tables[g.index]))
        arr = np.full((len(entries), width), -1, dtype=np.int32)
        for s, t in enumerate(tables[g.index]):
            if t:
                arr[s, :len(t)] = t
        bt.append(arr)
    return StepBatch(
        requests=[e.request for e in entries],
        tokens=np.asarray(tokens, dtype=np.int32), positions=np.asarray(positions, dtype=np.int32),
        seq_of=np.asarray(seq_of, dtype=np.int32), query_start=np.asarray(query_start, dtype=np.int32),
        context_len=np.asarray(context_len, dtype=np.int32), block_tables=bt,
        state_slots=np.asarray(slots, dtype=np.int32), logit_rows=np.asarray(rows, dtype=np.int32))


def pad_tables(batch: StepBatch, widths: Sequence[int]) -> StepBatch:
    """The same batch with every group's block table padded (with -1) to the given width."""
    tables = []
    for t, w in zip(batch.block_tables, widths):
        if t.shape[1] < w:
            t = np.concatenate([t, np.full((t.shape[0], w - t.shape[1]), -1, dtype=np.int32)], axis=1)
        tables.append(t)
    return StepBatch(batch.requests, batch.tokens, batch.positions, batch.seq_of, batch.query_start,
                     batch.context_len, tables, batch.state_slots, batch.logit_rows)


def attention_tiles(batch: StepBatch, tile_q: int, kind: str = "all") -> np.ndarray:
    """Cuts runs into tiles of at most ``tile_q`` consecutive queries:
    rows of (run, first token row, queries, position of the first query).
    ``kind`` selects the runs: "all", "multi" (two or more new tokens) or "single" (one)."""
    out = []
    for s in range(batch.S):
        a, b = int(batch.query_start[s]), int(batch.query_start[s + 1])
        if (kind == "multi" and b - a < 2) or (kind == "single" and b - a != 1):
            continue
        for r in range(a, b, tile_q):
            out.append((s, r, min(tile_q, b - r), int(batch.positions[r])))
    return np.asarray(out, dtype=np.int32).reshape(-1, 4)


class Workspace:
    """Named device buffers that live across steps (no allocation inside a step once warm)."""

    def __init__(self, device: torch.device):
        self.device = device
        self._fixed: Dict[Tuple, torch.Tensor] = {}
        self._dyn: Dict[Tuple, torch.Tensor] = {}
        self.version = 0          # grows whenever a buffer is (re)allocated: captured graphs hold the old pointers

    def fixed(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._fixed.get(key)
        if t is None:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._fixed[key] = t
            self.version += 1
        return t

    def dynamic(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype)
        t = self._dyn.get(key)
        if t is None or t.numel() < numel:
            t = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._dyn[key] = t
            self.version += 1
        return t

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self._fixed.values()) + list(self._dyn.values()))

    def pinned_ints(self, numel: int):
        """A pinned int32 staging buffer from a small ring; the caller records ``event`` after its
        copy so the buffer is not rewritten while the copy is still queued."""
        if not hasattr(self, "_ring"):
            self._ring, self._ring_pos = [[None, None] for _ in range(4)], 0
        self._ring_pos = (self._ring_pos + 1) % len(self._ring)
        slot = self._ring[self._ring_pos]
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < numel:
            slot[0] = torch.empty(max(numel, 1024), dtype=torch.int32, pin_memory=True)
        if slot[1] is None:
            slot[1] = torch.cuda.Event()
        return slot[0], slot[1]


class StepContext:
    """Device form of a step: index arrays (one host-to-device copy), scratch, stream."""

    def __init__(self, batch: StepBatch, workspace: Workspace, device: torch.device, max_tokens: int,
                 err: Optional[torch.Tensor] = None, tile_sizes: Sequence[int] = (),
                 max_context: Optional[int] = None, upload: bool = True):
        self.batch = batch
        self.workspace = workspace
        self.device = device
        self.max_tokens = max_tokens
        self.T, self.S, self.R = batch.T, batch.S, batch.R
        if self.T > max_tokens:
            raise BatchError(f"the step has {self.T} tokens; the limit is {max_tokens}")
        # an upper bound of the cached length may be given (graph replays are built for a bucket)
        self.max_context = int(max_context) if max_context is not None else int(batch.context_len.max())
        self.err = err
        self.stream = torch.cuda.current_stream(device).cuda_stream
        # host views parts may read (toy mixers, planners)
        self.query_start_host = batch.query_start
        self.positions_host = batch.positions
        self.state_slots_host = batch.state_slots
        # tile_sizes: (tile_q, kind) pairs the model's mixers asked for ahead of time
        self._tiles_host = {key: attention_tiles(batch, key[0], key[1]) for key in tile_sizes}
        # one packed upload
        parts = [batch.tokens, batch.positions, batch.seq_of, batch.query_start, batch.context_len,
                 batch.state_slots, batch.logit_rows] + [t.reshape(-1) for t in batch.block_tables] + \
                [t.reshape(-1) for t in self._tiles_host.values()]
        offs, total = [], 0
        for p in parts:
            offs.append(total)
            total += (p.size + 7) // 8 * 8          # keep every array 32-byte aligned
        total = max(total, 8)
        dev = workspace.dynamic("step.ints", max(total, 1 << 16), torch.int32)
        self.ints = dev
        if upload:
            host, event = workspace.pinned_ints(total)
            hn = host.numpy()
            for p, o in zip(parts, offs):
                hn[o:o + p.size] = p
            dev[:total].copy_(host[:total], non_blocking=True)
            event.record()

        def view(i, shape=None):
            p = parts[i]
            v = dev[offs[i]:offs[i] + p.size]
            return v.view(shape) if shape is not None else v

        self.tokens, self.positions, self.seq_of = view(0), view(1), view(2)
        self.query_start, self.context_len, self.state_slots, self.logit_rows = view(3), view(4), view(5), view(6)
        ng = len(batch.block_tables)
        self._tables = [view(7 + g, batch.block_tables[g].shape) for g in range(ng)]
        self._tiles = {key: (view(7 + ng + i, (-1, 4)) if self._tiles_host[key].size else None,
                             int(self._tiles_host[key].shape[0]))
                       for i, key in enumerate(self._tiles_host)}

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    def attention_tiles(self, tile_q: int, kind: str = "all"):
        """(device tensor [n, 4] or None, n) for tiles of up to ``tile_q`` queries over the runs of
        ``kind``.  Tile shapes a mixer announces through ``tile_requests`` travel with the step's one
        upload; others cost a copy of their own."""
        key = (tile_q, kind)
        got = self._tiles.get(key)
        if got is None:
            host = attention_tiles(self.batch, tile_q, kind)
            if host.size == 0:
                got = (None, 0)
            else:
                dev = self.workspace.dynamic(f"step.tiles.{tile_q}.{kind}", max(host.size, 4), torch.int32)
                dev[:host.size].copy_(torch.from_numpy(host.reshape(-1)), non_blocking=False)
                got = (dev[:host.size].view(-1, 4), int(host.shape[0]))
            self._tiles[key] = got
            self._tiles_host[key] = host
        return got

    def buf(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.fixed(name, shape, dtype)

    def buf_dyn(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.dynamic(name, numel, dtype)
