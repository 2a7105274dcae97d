"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of requests;
groups with windows give pages back early; state slots."""
import random

import pytest

from serve_b200.cache import CacheManager, NoFreeSlot, OutOfPages, PagePool
from serve_b200.parts import CacheNeed


def _mgr(num_pages=16, page=4, slots=4, needs=None, ctx=256):
    needs = needs if needs is not None else [CacheNeed(2, 16), CacheNeed(2, 16)]
    return CacheManager(needs, [None] * len(needs), page, num_pages, slots, ctx)


def test_pool_refuses_double_free_and_strangers():
    pool = PagePool(4)
    a = pool.take(2, "a")
    with pytest.raises(OutOfPages):
        pool.take(3, "b")
    assert pool.available == 2
    with pytest.raises(RuntimeError, match="held by"):
        pool.give_back(a, "b")
    pool.give_back(a, "a")
    with pytest.raises(RuntimeError, match="free"):
        pool.give_back(a, "a")
    pool.check()


def test_grow_free_reuse():
    m = _mgr()
    assert len(m.groups) == 1     # equal geometry: one group, one table, for both layers
    m.open("a")
    m.reserve([("a", 9)])
    m.commit("a", 9)
    assert m.groups[0].pool.in_use == 3
    m.reserve([("a", 12)])        # still three pages
    assert m.groups[0].pool.in_use == 3
    m.reserve([("a", 13)])
    assert m.groups[0].pool.in_use == 4
    first = [int(p) for p in m.table_rows(0, ["a"])[0]]
    m.close("a")
    m.check()
    m.open("b")
    m.reserve([("b", 16)])
    again = [int(p) for p in m.table_rows(0, ["b"])[0]]
    assert sorted(again) == sorted(first)       # the pages come back
    assert again[0] == first[-1]                # the page freed last is used first
    m.check()


def test_reserve_is_all_or_nothing():
    m = _mgr(num_pages=5)
    m.open("a"); m.open("b")
    m.reserve([("a", 8)])
    with pytest.raises(OutOfPages):
        m.reserve([("a", 12), ("b", 12)])       # 1 + 3 wanted, 3 free
    assert m.groups[0].pool.in_use == 2 and m.pages_wanted("b", 12) == [3]
    m.check()
    with pytest.raises(ValueError, match="context limit"):
        m.reserve([("a", 10_000)])


def test_slots():
    m = _mgr(slots=2)
    m.open("a"); m.open("b")
    with pytest.raises(NoFreeSlot):
        m.open("c")
    with pytest.raises(KeyError):
        m.open("a")
    s = m.slot("a")
    m.close("a")
    assert m.open("c") == s
    m.check()


def test_groups_with_other_needs_have_pages_of_their_own():
    needs = [CacheNeed(2, 16), CacheNeed(2, 16, window=6), CacheNeed(1, 32), None, CacheNeed(2, 16)]
    m = CacheManager(needs, [None, None, None, None, None], 4, 12, 2, 256)
    assert len(m.groups) == 3
    views = m.views()
    assert views[3] is None and views[0].group == views[4].group != views[1].group
    m.open("a")
    m.reserve([("a", 20)])
    m.commit("a", 20)
    full, win, other = (g.pool.in_use for g in m.groups)
    # window 6 at length 20: next query (position 20) reads keys 15..20 -> blocks 3.. ; blocks 0,1,2 went back
    assert (full, win, other) == (5, 2, 5)
    row = m.table_rows(1, ["a"])[0]
    assert list(row[:3]) == [-1, -1, -1] and all(p >= 0 for p in row[3:5])
    m.reserve([("a", 30)])
    m.commit("a", 30)
    assert m.groups[1].pool.in_use == 2 and m.groups[0].pool.in_use == 8
    m.check()
    m.close("a")
    assert all(g.pool.in_use == 0 for g in m.groups)
    m.check()


def test_cache_of_shares_the_owner_view():
    needs = [CacheNeed(2, 16), None]
    m = CacheManager(needs, [None, 0], 4, 8, 2, 64)
    v = m.views()
    assert v[0].writes and not v[1].writes and v[1].group == v[0].group


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    needs = [CacheNeed(2, 16), CacheNeed(2, 16, window=rng.choice([3, 9, 17]))]
    m = CacheManager(needs, [None, None], rng.choice([2, 4, 8]), rng.choice([6, 11, 24]), 4, 512)
    live = {}
    n_open = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{n_open}"; n_open += 1
            m.open(rid); live[rid] = 0
        elif op < 0.8 and live:
            batch = [(rid, live[rid] + rng.choice([1, 1, 2, 5, 13])) for rid in rng.sample(sorted(live), rng.randint(1, len(live)))]
            try:
                m.reserve(batch)
            except OutOfPages:
                m.check()
                continue
            for rid, n in batch:
                m.commit(rid, n); live[rid] = n
        elif live:
            rid = rng.choice(sorted(live))
            m.close(rid); del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
            for gi, g in enumerate(m.groups):
                row = m.table_rows(gi, [rid], m.max_blocks)[0]
                lo = 0 if g.window is None else max(0, n - g.window + 1) // m.page_size
                assert all(row[b] >= 0 for b in range(lo, m.blocks_for(n))), "a block a later query reads is missing"
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(g.pool.in_use == 0 for g in m.groups) and m.free_slots == 4
