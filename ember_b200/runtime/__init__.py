"""Native host runtime: the per-step packing of a batch's integer arrays (C++, C ABI, ctypes).

``pack_step`` is what ``ModelRunner.step`` uses; ``engine.batch.build_batch`` states the same
layout with numpy and is what tests compare it with.  The library is compiled with the host
C++ compiler at first use (no CUDA needed) into the folder the kernels are built in.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from ctypes import c_int, c_int32, c_uint64, c_void_p, POINTER
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np

from ..csrc import build as kernel_build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lock = threading.Lock()
_lib = None

TILE_KINDS = {"all": 0, "multi": 1, "single": 2}


class StepLayout(ctypes.Structure):
    _fields_ = [("tokens", c_int32), ("positions", c_int32), ("seq_of", c_int32), ("query_start", c_int32),
                ("context_len", c_int32), ("state_slots", c_int32), ("logit_rows", c_int32),
                ("tables", c_int32 * 8), ("tiles", c_int32 * 8), ("n_tiles", c_int32 * 8), ("total", c_int32),
                ("T", c_int32), ("S", c_int32), ("R", c_int32), ("max_context", c_int32)]


class RuntimeBuildError(RuntimeError):
    pass


def _compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and shutil.which(cand):
            return cand
    raise RuntimeBuildError("no C++ compiler found (g++ / c++); the native host runtime cannot be built")


def library() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        srcs = [os.path.join(_HERE, n) for n in ("step_pack.cpp", "cache_core.cpp")]
        h = hashlib.sha256()
        for src in srcs:
            with open(src, "rb") as f:
                h.update(f.read())
        digest = h.hexdigest()[:16]
        so = os.path.join(kernel_build.build_dir(), "libember_runtime.so")
        stamp = so + ".stamp"
        current = os.path.isfile(so) and os.path.isfile(stamp) and open(stamp).read().strip() == digest
        if not current:
            print("[ember_b200] compiling the host runtime (step_pack.cpp, cache_core.cpp) ...", file=sys.stderr, flush=True)
            tmp = f"{so}.{os.getpid()}.tmp"
            proc = subprocess.run([_compiler(), "-O2", "-std=c++17", "-shared", "-fPIC", "-o", tmp] + srcs,
                                  capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeBuildError(f"the C++ compiler failed on the host runtime:\n{proc.stdout}{proc.stderr}")
            os.replace(tmp, so)
            with open(stamp, "w") as f:
                f.write(digest)
        lib = ctypes.CDLL(so)
        vp = c_void_p                 # addresses are passed as plain integers
        lib.ember_step_layout.restype = c_int
        lib.ember_step_layout.argtypes = [c_int, vp, vp, vp, vp, vp, c_int, vp, c_int, vp, vp, c_int, c_int,
                                          POINTER(StepLayout)]
        lib.ember_step_pack.restype = None
        lib.ember_step_pack.argtypes = [c_int, vp, vp, vp, vp, vp, vp, c_int, vp, vp, vp,
                                        c_int, vp, vp, POINTER(StepLayout), vp]
        # the cache core (cache_core.cpp)
        i32p, i64p, u64p = POINTER(c_int32), POINTER(ctypes.c_int64), POINTER(c_uint64)
        sigs = {
            "ember_pool_create": (c_void_p, [c_int]), "ember_pool_destroy": (None, [c_void_p]),
            "ember_pool_allocate": (c_int, [c_void_p]), "ember_pool_release": (c_int, [c_void_p, c_int]),
            "ember_pool_available": (c_int, [c_void_p]), "ember_pool_is_held": (c_int, [c_void_p, c_int]),
            "ember_pool_check": (c_int, [c_void_p, ctypes.c_char_p, c_int]),
            "ember_cache_create": (c_void_p, [c_int, i32p, i32p, i32p, c_int, c_int]),
            "ember_cache_destroy": (None, [c_void_p]), "ember_cache_pool": (c_void_p, [c_void_p, c_int]),
            "ember_cache_admit": (c_int, [c_void_p]), "ember_cache_slot": (c_int, [c_void_p, c_int]),
            "ember_cache_tokens": (ctypes.c_longlong, [c_void_p, c_int]),
            "ember_cache_first_live": (c_int, [c_void_p, c_int, c_int]),
            "ember_cache_table": (c_int, [c_void_p, c_int, c_int, POINTER(i32p)]),
            "ember_cache_ensure": (c_int, [c_void_p, c_int, ctypes.c_longlong]),
            "ember_cache_advance": (c_int, [c_void_p, c_int, ctypes.c_longlong]),
            "ember_cache_release": (c_int, [c_void_p, c_int]), "ember_cache_reset": (c_int, [c_void_p, c_int]),
            "ember_cache_free_slots": (c_int, [c_void_p]),
            "ember_cache_describe": (c_int, [c_void_p, c_int, vp, vp, vp, vp, vp]),
            "ember_cache_check": (c_int, [c_void_p, ctypes.c_char_p, c_int]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
        return lib


_ERRORS = {-1: "a step needs at least one entry", -2: "a request brings no tokens",
           -3: "a wanted row lies outside its request's tokens", -4: "a token id is out of range",
           -5: "too many cache groups or tile lists for one step"}


class PackedStep:
    """A step's integer arrays in one buffer, with the offsets of its pieces."""

    def __init__(self, requests, layout: StepLayout, buf: np.ndarray, widths: Sequence[int],
                 tile_keys: Sequence[Tuple[int, str]]):
        self.requests = requests
        self.layout = layout
        self.buf = buf
        self.widths = list(widths)
        self.tile_keys = list(tile_keys)
        self.T, self.S, self.R = layout.T, layout.S, layout.R
        self.max_context = layout.max_context
        self.total = layout.total
        self.staging = None          # (pinned tensor, event) when ``buf`` is a view of staging memory

    @property
    def block_tables(self):
        return [self.block_table(g) for g in range(len(self.widths))]

    def piece(self, offset: int, n: int) -> np.ndarray:
        return self.buf[offset:offset + n]

    @property
    def tokens(self):
        return self.piece(self.layout.tokens, self.T)

    @property
    def positions(self):
        return self.piece(self.layout.positions, self.T)

    @property
    def seq_of(self):
        return self.piece(self.layout.seq_of, self.T)

    @property
    def query_start(self):
        return self.piece(self.layout.query_start, self.S + 1)

    @property
    def context_len(self):
        return self.piece(self.layout.context_len, self.S)

    @property
    def state_slots(self):
        return self.piece(self.layout.state_slots, self.S)

    @property
    def logit_rows(self):
        return self.piece(self.layout.logit_rows, self.R)

    def block_table(self, group: int) -> np.ndarray:
        return self.piece(self.layout.tables[group], self.S * self.widths[group]).reshape(self.S, self.widths[group])

    def tiles(self, index: int) -> np.ndarray:
        return self.piece(self.layout.tiles[index], self.layout.n_tiles[index] * 4).reshape(-1, 4)


class StepPacker:
    """Packs steps through the native library.  Keeps its input arrays (and their addresses) across
    steps, so a step costs one pass over the entries and two calls into the library."""

    def __init__(self):
        self._lib = library()
        self._cap_runs = self._cap_tokens = self._cap_want = self._cap_tables = 0
        self._small = {}
        self._lay = None

    def _array(self, name: str, n: int, dtype=np.int32):
        got = self._small.get(name)
        if got is None or got[0].shape[0] < n:
            arr = np.zeros(max(16, 2 * n), dtype=dtype)
            got = (arr, arr.ctypes.data)
            self._small[name] = got
        return got

    def pack(self, entries, cache, vocab_size: int, max_positions: Optional[int] = None,
             tile_keys: Sequence[Tuple[int, str]] = (), widths: Optional[Sequence[int]] = None,
             min_widths: Optional[Sequence[int]] = None, alloc=None, n_prev: int = 0) -> PackedStep:
        """Checks the entries, reads cached lengths, slots and block tables from ``cache`` (pages for the
        new tokens must already be ensured) and packs the step.  ``widths`` sets the block tables' widths,
        ``min_widths`` only pads them (graph buckets); ``alloc(n)`` returns (int32 array to fill, its
        address) — pinned staging memory — else a new array is made.  With ``n_prev`` > 0 a token
        -(r + 1), r < n_prev, is allowed: the id sampled in row r of the step before."""
        from ..engine.batch import BatchError
        lib = self._lib
        S = len(entries)
        if S == 0:
            raise BatchError("a step needs at least one entry")
        groups = cache.groups
        G = len(groups)
        page = cache.page_tokens
        requests, counts, want_counts, handles = [], [], [], []
        tok_flat, want_flat = [], []
        handle_of = cache.handle_of
        for e in entries:
            requests.append(e.request)
            handles.append(handle_of(e.request))
            counts.append(len(e.tokens))
            want_counts.append(len(e.want))
            tok_flat += e.tokens
            if e.want:
                want_flat += e.want
        # cached lengths, slots and block tables of all entries in one native call
        d_i32, d_i32_at = self._array("describe.i32", S * (2 + G) + 8)
        d_i64, d_i64_at = self._array("describe.i64", S * (1 + G) + 8, np.int64)
        d_i32[:S] = handles
        bad = lib.ember_cache_describe(cache.core, S, d_i32_at, d_i64_at, d_i32_at + 4 * S, d_i64_at + 8 * S,
                                       d_i32_at + 8 * S)
        if bad >= 0:
            from ..cache.manager import CacheError
            raise CacheError(f"request {entries[bad].request!r} holds no cache")
        starts = d_i64[:S].tolist()
        slots = d_i32[S:2 * S].tolist()
        table_addr = d_i64[S:S + G * S].view(np.uint64).tolist()
        table_lens = d_i32[2 * S:2 * S + G * S].tolist()
        for s in range(S):
            n, start = counts[s], starts[s]
            if max_positions is not None and start + n > max_positions:
                raise BatchError(f"request {requests[s]!r} would reach position {start + n}; "
                                 f"the model's limit is {max_positions}")
            for g in groups:
                if g.paged and table_lens[g.index * S + s] * page < start + n:
                    raise BatchError(f"request {requests[s]!r} has no pages for tokens up to {start + n}")
        if len(set(requests)) != S:
            raise BatchError("a request appears twice in one step")
        if widths is None:
            widths = [max(1, max(table_lens[g * S:(g + 1) * S])) for g in range(G)]
            if min_widths is not None:
                widths = [max(w, m) for w, m in zip(widths, min_widths)]
        L = len(tile_keys)
        T, R = len(tok_flat), len(want_flat)
        # one int32 scratch array holds every small input; the table addresses have their own
        n_small = 4 * S + T + R + G + 2 * L
        ints, ints_at = self._array("ints", n_small + 8)
        try:
            ints[:n_small] = counts + starts + slots + want_counts + tok_flat + want_flat + list(widths) + \
                [k[0] for k in tile_keys] + [TILE_KINDS[k[1]] for k in tile_keys]
        except (OverflowError, ValueError, TypeError):
            raise BatchError("a token id or a wanted row is not a 32-bit integer") from None
        o_counts, o_starts, o_slots, o_wc = ints_at, ints_at + 4 * S, ints_at + 8 * S, ints_at + 12 * S
        o_tok = ints_at + 16 * S
        o_want = o_tok + 4 * T
        o_widths = o_want + 4 * R
        o_tq = o_widths + 4 * G
        o_tk = o_tq + 4 * L
        lay = StepLayout()
        lay_ref = ctypes.byref(lay)
        code = lib.ember_step_layout(S, o_counts, o_starts, o_wc, o_tok, o_want, G, o_widths, L, o_tq, o_tk,
                                     int(vocab_size), int(n_prev), lay_ref)
        if code != 0:
            raise BatchError(_ERRORS.get(code, f"the step could not be laid out (code {code})") +
                             f" (vocabulary {vocab_size})")
        if alloc is not None:
            buf, buf_at = alloc(lay.total)
        else:
            buf = np.empty(lay.total, dtype=np.int32)
            buf_at = buf.ctypes.data
        addr, addr_at = self._array("addr", G * S + 1, np.uint64)
        lens, lens_at = self._array("lens", G * S + 1)
        addr[:G * S] = table_addr
        lens[:G * S] = table_lens
        lib.ember_step_pack(S, o_counts, o_starts, o_slots, o_wc, o_tok, o_want, G, o_widths, addr_at, lens_at,
                            L, o_tq, o_tk, lay_ref, buf_at)
        return PackedStep(requests, lay, buf, widths, tile_keys)


_default_packer = None


def pack_step(entries, cache, vocab_size: int, max_positions: Optional[int] = None,
              tile_keys: Sequence[Tuple[int, str]] = (), widths: Optional[Sequence[int]] = None,
              min_widths: Optional[Sequence[int]] = None, alloc=None, n_prev: int = 0) -> PackedStep:
    """``StepPacker.pack`` with a packer shared by the process (not for concurrent use)."""
    global _default_packer
    if _default_packer is None:
        _default_packer = StepPacker()
    return _default_packer.pack(entries, cache, vocab_size, max_positions, tile_keys, widths, min_widths, alloc, n_prev)
