"""The cache manager: no page lost, held twice or freed twice, under random orders (no GPU)."""
import random

import pytest

from ember_b200.cache import CacheError, CacheManager, PagePool
from ember_b200.parts.base import CacheNeed

FULL = CacheNeed(kind="full", num_kv_heads=2, head_dim=16)
WIN = CacheNeed(kind="window", num_kv_heads=2, head_dim=16, window=40)
STATE = CacheNeed(kind="state", state_shape=(4,), state_dtype="float32")


def test_pool_order_and_double_free():
    p = PagePool(4)
    assert [p.allocate() for _ in range(4)] == [0, 1, 2, 3] and p.allocate() == -1
    p.release(2)
    p.release(0)
    assert p.allocate() == 0 and p.allocate() == 2          # most recently freed first
    p.release(1)
    with pytest.raises(CacheError, match="twice"):
        p.release(1)
    with pytest.raises(CacheError, match="outside"):
        p.release(9)
    assert p.check() == ""


def test_groups_by_need():
    m = CacheManager({0: FULL, 1: WIN, 2: FULL, 3: STATE, 4: WIN}, 16, 256, 4)
    assert [(g.need.kind, g.layers) for g in m.groups] == [("full", [0, 2]), ("window", [1, 4]), ("state", [3])]
    assert m.layer_group == {0: 0, 2: 0, 1: 1, 4: 1, 3: 2}
    assert m.groups[2].pool is None


def test_ensure_is_all_or_nothing_and_release_returns_everything():
    m = CacheManager({0: FULL, 1: WIN}, 16, 64, 2)           # 4 pages per group
    assert m.admit("a") is not None and m.admit("b") is not None and m.admit("c") is None
    assert m.ensure("a", 33)                                  # 3 pages in each group
    assert m.used_pages() == [3, 3]
    assert not m.ensure("b", 17)                              # needs 2, only 1 left: nothing is taken
    assert m.used_pages() == [3, 3] and m.get("b").tables == [[], []]
    assert m.ensure("b", 16)
    m.release("a")
    assert m.used_pages() == [1, 1] and m.free_slots() == 1
    with pytest.raises(CacheError):
        m.release("a")
    assert m.check() == ""


def test_window_pages_are_given_back_and_used_again():
    m = CacheManager({0: FULL, 1: WIN}, 16, 1024, 2, pages_per_group=[64, 5])
    m.admit("a")
    held = set()
    for upto in range(8, 400, 8):
        assert m.ensure("a", upto), upto                      # 5 window pages suffice for any length
        m.advance("a", upto)
        t = m.get("a").tables[1]
        live = [p for p in t if p >= 0]
        assert len(live) <= 5
        first_needed = max(0, upto - 40 + 1) // 16
        assert all(p == -1 for p in t[:first_needed]) and all(p >= 0 for p in t[first_needed:])
        held |= set(live)
        assert m.check() == ""
    assert held <= set(range(5))                              # 25 logical pages went through at most 5 physical ones
    assert len(m.get("a").tables[0]) == 25                    # the full group kept everything
    m.release("a")
    assert m.used_pages() == [0, 0]


def test_random_orders_never_lose_or_share_a_page():
    rng = random.Random(7)
    m = CacheManager({0: FULL, 1: WIN, 2: STATE}, 16, 640, 6)
    live = {}
    next_id = 0
    for step in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            assert m.admit(next_id) is not None
            live[next_id] = 0
            next_id += 1
        elif op < 0.75 and live:
            r = rng.choice(list(live))
            n = live[r] + rng.randint(1, 70)
            if m.ensure(r, n):
                live[r] = n
                m.advance(r, n)
        elif op < 0.9 and live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        elif live:
            r = rng.choice(list(live))
            m.reset(r)
            live[r] = 0
        assert m.check() == "", f"step {step}: {m.check()}"
        slots = [m.get(r).slot for r in live]
        assert len(set(slots)) == len(slots)
    for r in list(live):
        m.release(r)
    assert m.used_pages() == [0, 0, 0] and m.free_slots() == 6 and m.check() == ""
