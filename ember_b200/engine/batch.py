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

from .. import transfers
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
    tok_parts, pos_parts = [], []
    counts: List[int] = []
    starts: List[int] = []
    slots: List[int] = []
    rows: List[int] = []
    tables: List[List[np.ndarray]] = [[] for _ in cache.groups]
    at = 0
    page = cache.page_tokens
    for e in entries:
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
            if g.paged and len(rc.tables[g.index]) * page < start + n:
                raise BatchError(f"request {e.request!r} has no pages for tokens up to {start + n}")
        tok_parts.append(np.asarray(e.tokens, dtype=np.int64))
        pos_parts.append(np.arange(start, start + n, dtype=np.int32))
        for w in e.want:
            w = int(w)
            if not (0 <= w < n):
                raise BatchError(f"request {e.request!r} wants row {w} of {n} tokens")
            rows.append(at + w)
        counts.append(n)
        starts.append(start)
        at += n
        slots.append(rc.slot)
        for g in cache.groups:
            tables[g.index].append(rc.table_array(g.index))
    tokens = np.concatenate(tok_parts) if len(tok_parts) > 1 else tok_parts[0]
    if tokens.size and (int(tokens.min()) < 0 or int(tokens.max()) >= vocab_size):
        bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
        raise BatchError(f"token id {bad} is out of range (vocabulary {vocab_size})")
    counts_a = np.asarray(counts, dtype=np.int32)
    query_start = np.zeros(len(entries) + 1, dtype=np.int32)
    np.cumsum(counts_a, out=query_start[1:])
    bt = []
    for g in cache.groups:
        width = max(1, max(len(t) for t in tables[g.index]))
        arr = np.full((len(entries), width), -1, dtype=np.int32)
        for s, t in enumerate(tables[g.index]):
            if t.shape[0]:
                arr[s, :t.shape[0]] = t
        bt.append(arr)
    return StepBatch(
        requests=[e.request for e in entries],
        tokens=tokens.astype(np.int32), positions=np.concatenate(pos_parts) if len(pos_parts) > 1 else pos_parts[0],
        seq_of=np.repeat(np.arange(len(entries), dtype=np.int32), counts_a), query_start=query_start,
        context_len=np.asarray(starts, dtype=np.int32) + counts_a, block_tables=bt,
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
    qs = batch.query_start
    lens = qs[1:] - qs[:-1]
    if kind == "multi":
        runs = np.nonzero(lens >= 2)[0]
    elif kind == "single":
        runs = np.nonzero(lens == 1)[0]
    else:
        runs = np.arange(batch.S)
    if runs.size == 0:
        return np.zeros((0, 4), dtype=np.int32)
    if int(lens[runs].max()) <= tile_q:                 # every selected run is one tile (all decode steps)
        first = qs[:-1][runs]
        return np.stack([runs.astype(np.int32), first, lens[runs], batch.positions[first]], axis=1).astype(np.int32)
    out = []
    for s in runs:
        a, b = int(qs[s]), int(qs[s + 1])
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

    def __init__(self, batch, workspace: Workspace, device: torch.device, max_tokens: int,
                 err: Optional[torch.Tensor] = None, tile_sizes: Sequence[Tuple[int, str]] = (),
                 max_context: Optional[int] = None, upload: bool = True, prev_ids: Optional[torch.Tensor] = None):
        """``batch`` is a ``StepBatch`` (packed here, with numpy) or a ``runtime.PackedStep`` (packed
        already, by the native packer, with the tile lists it was asked for)."""
        self.batch = batch
        self.workspace = workspace
        self.device = device
        self.max_tokens = max_tokens
        self.T, self.S, self.R = batch.T, batch.S, batch.R
        if self.T > max_tokens:
            raise BatchError(f"the step has {self.T} tokens; the limit is {max_tokens}")
        self.err = err
        self.prev_ids = prev_ids         # where the sampler left the step before's ids (tokens < 0 point there)
        self.stream = torch.cuda.current_stream(device).cuda_stream
        # host views parts may read (toy mixers, planners)
        self.query_start_host = batch.query_start
        self.positions_host = batch.positions
        self.state_slots_host = batch.state_slots
        self._packed = batch if hasattr(batch, "layout") else None
        if self._packed is not None:
            lay, S = batch.layout, batch.S
            longest = batch.max_context
            self._table_shapes = [(S, w) for w in batch.widths]
            self._tile_rows = {key: int(lay.n_tiles[i]) for i, key in enumerate(batch.tile_keys)}
            self._offs = [lay.tokens, lay.positions, lay.seq_of, lay.query_start, lay.context_len, lay.state_slots,
                          lay.logit_rows] + [lay.tables[g] for g in range(len(batch.widths))] + \
                         [lay.tiles[i] for i in range(len(batch.tile_keys))]
            self._sizes = [self.T, self.T, self.T, S + 1, S, S, self.R] + [S * w for w in batch.widths] + \
                          [4 * n for n in self._tile_rows.values()]
            self._parts, self._total = None, int(lay.total)
        else:
            longest = int(batch.context_len.max())
            # tile_sizes: (tile_q, kind) pairs the model's mixers asked for ahead of time
            tiles_host = {key: attention_tiles(batch, key[0], key[1]) for key in tile_sizes}
            self._table_shapes = [t.shape for t in batch.block_tables]
            self._tile_rows = {key: int(t.shape[0]) for key, t in tiles_host.items()}
            parts = [batch.tokens, batch.positions, batch.seq_of, batch.query_start, batch.context_len,
                     batch.state_slots, batch.logit_rows] + [t.reshape(-1) for t in batch.block_tables] + \
                    [t.reshape(-1) for t in tiles_host.values()]
            offs, total = [], 0
            for p in parts:
                offs.append(total)
                total += (p.size + 7) // 8 * 8          # keep every array 32-byte aligned
            self._parts, self._offs, self._total = parts, offs, max(total, 8)
            self._sizes = [p.size for p in parts]
        # an upper bound of the cached length may be given (graph replays are built for a bucket)
        self.max_context = int(max_context) if max_context is not None else longest
        # one packed upload; device views of its pieces are made only when a part asks for them
        # (a replayed graph needs the upload alone)
        self.ints = workspace.dynamic("step.ints", max(self._total, 1 << 16), torch.int32)
        self._ng = len(self._table_shapes)
        self._tiles = {}
        self.memo = {}                # what parts compute once per step and share between layers
        if upload:
            self.upload()

    _NAMES = {"tokens": 0, "positions": 1, "seq_of": 2, "query_start": 3, "context_len": 4, "state_slots": 5,
              "logit_rows": 6}

    def upload(self) -> None:
        staging = self._packed.staging if self._packed is not None else None
        if staging is not None:
            host, event = staging
        else:
            host, event = self.workspace.pinned_ints(self._total)
            hn = host.numpy()
            if self._packed is not None:
                hn[:self._total] = self._packed.buf[:self._total]
            else:
                for p, o in zip(self._parts, self._offs):
                    hn[o:o + p.size] = p
        self.ints[:self._total].copy_(host[:self._total], non_blocking=True)
        event.record()
        transfers.add_h2d(4 * self._total)

    def _view(self, i: int, shape=None) -> torch.Tensor:
        v = self.ints[self._offs[i]:self._offs[i] + self._sizes[i]]
        return v.view(shape) if shape is not None else v

    def __getattr__(self, name: str):
        # device views of the packed arrays, made on first use
        idx = StepContext._NAMES.get(name)
        if idx is None:
            raise AttributeError(name)
        v = self._view(idx)
        setattr(self, name, v)
        return v

    def block_table(self, group: int) -> torch.Tensor:
        return self._view(7 + group, self._table_shapes[group])

    def attention_tiles(self, tile_q: int, kind: str = "all"):
        """(device tensor [n, 4] or None, n) for tiles of up to ``tile_q`` queries over the runs of
        ``kind``.  Tile shapes a mixer announces through ``tile_requests`` travel with the step's one
        upload; others cost a copy of their own."""
        key = (tile_q, kind)
        got = self._tiles.get(key)
        if got is None and key in self._tile_rows:
            i = 7 + self._ng + list(self._tile_rows).index(key)
            n = self._tile_rows[key]
            got = (self._view(i, (-1, 4)) if n else None, n)
            self._tiles[key] = got
        if got is None:
            host = attention_tiles(self.batch, tile_q, kind)
            if host.size == 0:
                got = (None, 0)
            else:
                dev = self.workspace.dynamic(f"step.tiles.{tile_q}.{kind}", max(host.size, 4), torch.int32)
                dev[:host.size].copy_(torch.from_numpy(host.reshape(-1)), non_blocking=False)
                got = (dev[:host.size].view(-1, 4), int(host.shape[0]))
            self._tiles[key] = got
        return got

    def buf(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.fixed(name, shape, dtype)

    def buf_dyn(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.dynamic(name, numel, dtype)
