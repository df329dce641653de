"""The native step packer against the numpy statement of the same layout (no GPU)."""
import random

import numpy as np
import pytest

from ember_b200.cache import CacheManager
from ember_b200.engine.batch import BatchError, StepEntry, attention_tiles, build_batch, pad_tables
from ember_b200.parts.base import CacheNeed
from ember_b200.runtime import pack_step

FULL = CacheNeed(kind="full", num_kv_heads=2, head_dim=16)
WIN = CacheNeed(kind="window", num_kv_heads=2, head_dim=16, window=40)
STATE = CacheNeed(kind="state", state_shape=(4,), state_dtype="float32")


def test_packer_equals_numpy_layout_on_random_steps():
    rng = random.Random(5)
    cache = CacheManager({0: FULL, 1: WIN, 2: STATE}, 16, 4096, 8)
    live = {}
    keys = [(32, "multi"), (1, "single"), (7, "all")]
    for step in range(300):
        if len(live) < 5 and rng.random() < 0.4:
            rid = f"r{step}"
            cache.admit(rid)
            live[rid] = 0
        if not live:
            continue
        chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
        entries = []
        for rid in chosen:
            n = rng.choice([1, 1, 1, 2, 5, 33, 64])
            assert cache.ensure(rid, live[rid] + n)
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))
            entries.append(StepEntry(rid, [rng.randrange(500) for _ in range(n)], want))
        b = build_batch(entries, cache, 500)
        widths = [t.shape[1] + rng.choice([0, 3]) for t in b.block_tables]
        p = pack_step(entries, cache, 500, tile_keys=keys, widths=widths)
        bp = pad_tables(b, widths)
        assert (p.T, p.S, p.R, p.max_context) == (b.T, b.S, b.R, int(b.context_len.max()))
        for name in ("tokens", "positions", "seq_of", "query_start", "context_len", "state_slots", "logit_rows"):
            assert np.array_equal(getattr(p, name), getattr(b, name)), name
        for g in range(len(widths)):
            assert np.array_equal(p.block_table(g), bp.block_tables[g])
        for i, (tq, kind) in enumerate(keys):
            assert np.array_equal(p.tiles(i), attention_tiles(b, tq, kind))
        for e in entries:
            live[e.request] += len(e.tokens)
            cache.advance(e.request, live[e.request])
        if rng.random() < 0.2:
            rid = rng.choice(sorted(live))
            cache.release(rid)
            del live[rid]
    assert cache.check() == ""


def test_packer_rejects_what_the_numpy_path_rejects():
    cache = CacheManager({0: FULL}, 16, 256, 4)
    cache.admit("a")
    cache.ensure("a", 8)
    for bad in ([StepEntry("a", [1, 2], [2])], [StepEntry("a", [999], [])], [StepEntry("a", [], [])],
                [StepEntry("a", [1], []), StepEntry("a", [2], [])], [StepEntry("a", [1] * 40, [])], []):
        with pytest.raises(BatchError):
            pack_step(bad, cache, 500)
        with pytest.raises(BatchError):
            build_batch(bad, cache, 500)
