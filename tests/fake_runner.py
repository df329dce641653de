"""A stand-in for the model that needs no GPU and *reads the cache back*: it stores every
token it is given in fake pages through the block tables, and the "logits" of a row are a
one-hot at a hash of the context read back through those tables.  Any mistake in tables, page
accounting or positions changes the output (the idea of the reference's
tests/fake_backend.hpp:19-99).  With ``state=True`` the fake model is also recurrent: every token is folded, in
order, into the request's state slot, and the slot's value is folded into the output, so a slot that two requests
share, that is not zeroed when a preempted request is admitted again, or that is lost changes the tokens too."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ember_b200.cache.manager import CacheManager
from ember_b200.config.spec import ModelSpec
from ember_b200.engine.batch import build_batch
from ember_b200.parts.base import CacheNeed


def context_hash(tokens: List[int], vocab: int, state: int = 0) -> int:
    h = 0xCBF29CE484222325 ^ state
    for t in tokens:
        h = ((h ^ (t + 1)) * 0x100000001B3) & ((1 << 64) - 1)
    return int(h % vocab)


def fold_state(state: int, token: int) -> int:
    """The fake recurrent state after one more token."""
    return (state * 6364136223846793005 + token + 1442695040888963407) & ((1 << 61) - 1)


class _FakeSlots:
    """The part of ``CacheStorage`` the engine uses at admission: zeroing a request's state slot."""

    def __init__(self, n: int):
        self.values = [0] * n
        self.resets = 0

    def reset_slot(self, slot: int) -> None:
        self.values[slot] = 0
        self.resets += 1


class FakeSpec:
    def __init__(self, vocab_size=977, max_positions=4096, eos_ids=()):
        self.vocab_size, self.max_positions, self.eos_ids = vocab_size, max_positions, tuple(eos_ids)


class FakeRunner:
    def __init__(self, capacity_tokens: int, page_tokens: int = 16, max_requests: int = 64,
                 max_batch_tokens: int = 2048, vocab_size: int = 977, max_positions: int = 4096, eos_ids=(),
                 window: int = 0, state: bool = False):
        self.spec = FakeSpec(vocab_size, max_positions, eos_ids)
        need = CacheNeed(kind="window" if window else "full", num_kv_heads=1, head_dim=2, window=window)
        self.cache = CacheManager({0: need}, page_tokens, capacity_tokens, max_requests)
        # state=True: the engine zeroes the slot at every admission through this object, as it does with the real storage
        self.storage = _FakeSlots(max_requests) if state else None
        self.err_code = 0                  # what read_error() reports: tests inject a kernel's error word here
        self.resets_after_error = 0
        self.max_batch_tokens, self.max_requests = max_batch_tokens, max_requests
        self.pages = np.full((self.cache.groups[0].pool.n_pages, page_tokens), -1, dtype=np.int64)
        self.window = window
        self.steps = 0
        self.fail_next = False
        self.sampled_ids: List[int] = []
        self.speculated_steps = 0

    def set_sampled_ids(self, ids: List[int]) -> None:
        """What the sampler drew in the step before (the real runner keeps them on the device)."""
        self.sampled_ids = list(ids)

    def read_error(self) -> int:
        return self.err_code

    def reset_after_error(self) -> None:
        self.err_code = 0
        self.resets_after_error += 1

    def step(self, entries, n_prev: int = 0) -> Optional[torch.Tensor]:
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("injected step failure")
        if n_prev:
            from ember_b200.engine.batch import StepEntry
            self.speculated_steps += 1
            assert n_prev == len(self.sampled_ids)
            entries = [StepEntry(e.request, [self.sampled_ids[-t - 1] if t < 0 else t for t in e.tokens], e.want)
                       for e in entries]
        b = build_batch(entries, self.cache, self.spec.vocab_size, self.spec.max_positions)
        assert b.T <= self.max_batch_tokens
        page = self.cache.page_tokens
        table = b.block_tables[0]
        state_at = {}
        for t in range(b.T):                      # write first, as the model does
            s, pos = int(b.seq_of[t]), int(b.positions[t])
            blk = int(table[s, pos // page])
            assert blk >= 0
            self.pages[blk, pos % page] = int(b.tokens[t])
            if self.storage is not None:          # the recurrent part: tokens of a run in order, into the run's slot
                slot = int(b.state_slots[s])
                if pos == 0:
                    assert self.storage.values[slot] == 0, f"slot {slot} was not zeroed for a request that starts"
                self.storage.values[slot] = state_at[t] = fold_state(self.storage.values[slot], int(b.tokens[t]))
        rows = []
        for t in b.logit_rows:
            s, pos = int(b.seq_of[t]), int(b.positions[t])
            lo = max(0, pos - self.window + 1) if self.window else 0
            ctx = []
            for j in range(lo, pos + 1):
                blk = int(table[s, j // page])
                assert blk >= 0, f"position {j} of run {s} reads a page that was given back"
                ctx.append(int(self.pages[blk, j % page]))
            row = torch.zeros(self.spec.vocab_size)
            row[context_hash(ctx, self.spec.vocab_size, state_at.get(int(t), 0))] = 1.0
            rows.append(row)
        for s, req in enumerate(b.requests):
            self.cache.advance(req, int(b.context_len[s]))
        self.steps += 1
        return torch.stack(rows) if rows else None


def argmax_sampler(logits, params, counters):
    return [int(i) for i in torch.argmax(logits, dim=-1)]


def expected_generation(prompt: List[int], n: int, vocab: int, window: int = 0, state: bool = False) -> List[int]:
    toks, out = list(prompt), []
    st = 0
    if state:
        for t in toks:
            st = fold_state(st, t)
    for _ in range(n):
        ctx = toks[-window:] if window else toks
        t = context_hash(ctx, vocab, st)
        out.append(t)
        toks.append(t)
        if state:
            st = fold_state(st, t)
    return out
