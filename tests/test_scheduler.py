"""The scheduler's decisions, with a stand-in for the step (no model): admission, portions under a
token budget, mixing, finishing, and what happens when pages run out."""
import pytest

from serve_b200.cache import CacheManager
from serve_b200.engine.scheduler import SchedRequest, Scheduler
from serve_b200.parts import CacheNeed


def _cache(num_pages, page=4, slots=8, ctx=512):
    return CacheManager([CacheNeed(1, 16)], [None], page, num_pages, slots, ctx)


def run(sched, cache, max_steps=10_000, token_of=lambda r: 7):
    """Play the step function's part: reserve, commit, hand back a token per sampling entry."""
    log = []
    for _ in range(max_steps):
        if not sched.has_work():
            return log
        planned = sched.plan()
        for v in sched.evicted:
            cache.close(v.rid)
        assert planned, "nothing planned although there is work"
        batch = []
        for p in planned:
            if not cache.is_open(p.request.rid):
                cache.open(p.request.rid)
            assert cache.length(p.request.rid) == p.request.fed
            batch.append((p.request.rid, p.request.fed + len(p.tokens)))
        cache.reserve(batch)          # must never raise: the scheduler counted the pages
        for rid, n in batch:
            cache.commit(rid, n)
        cache.check()
        log.append([(p.request.rid, len(p.tokens), p.samples) for p in planned])
        done = sched.update(planned, [token_of(p.request) for p in planned if p.samples])
        for r in done:
            cache.close(r.rid)
    raise AssertionError("the scheduler did not finish")


def test_portions_under_a_token_budget_and_mixing():
    cache = _cache(64)
    s = Scheduler(cache, max_tokens_per_step=16, prefill_chunk=10)
    s.add(SchedRequest(0, list(range(25)), 3))
    s.add(SchedRequest(1, list(range(7)), 2))
    log = run(s, cache)
    assert log[0] == [(0, 10, False), (1, 6, False)]          # budget 16: 10 + 6
    assert log[1] == [(1, 1, True), (0, 10, False)]            # single tokens first, then the next portion
    flat = [e for step in log for e in step]
    assert sum(n for rid, n, _ in flat if rid == 0) == 25 + 2  # prompt + fed-back tokens (the last is never fed)
    assert all(sum(n for _, n, _ in step) <= 16 for step in log)
    assert [len(r.generated) for r in sorted(s.finished, key=lambda r: r.rid)] == [3, 2]
    # decode tokens come first in a step, beside portions of others
    mixed = [step for step in log if any(n == 1 and smp for _, n, smp in step) and any(n > 1 for _, n, _ in step)]
    assert mixed and all(step[0][1] == 1 for step in mixed)


def test_first_come_first_served_and_slots():
    cache = _cache(64, slots=2)
    s = Scheduler(cache, max_tokens_per_step=64)
    for i in range(4):
        s.add(SchedRequest(i, [1] * 5, 2))
    log = run(s, cache)
    assert [rid for rid, _, _ in log[0]] == [0, 1]            # two slots
    assert s.stats.max_running == 2
    assert [r.rid for r in s.finished] == [0, 1, 2, 3]


def test_finish_by_length_and_by_stop_id():
    cache = _cache(64)
    s = Scheduler(cache, 64)
    s.add(SchedRequest(0, [1, 2, 3], 1))
    s.add(SchedRequest(1, [1, 2, 3], 50, stop_ids=(9,)))
    run(s, cache, token_of=lambda r: 9 if len(r.generated) == 4 else 5)
    a, b = sorted(s.finished, key=lambda r: r.rid)
    assert a.generated == [5] and a.finish_reason == "length"     # one token, from the prompt's last place, then freed
    assert b.generated == [5, 5, 5, 5, 9] and b.finish_reason == "stop"
    assert cache.live == 0


def test_pages_run_out_evicts_the_last_admitted_and_recomputes():
    cache = _cache(num_pages=6, page=4)                       # 24 tokens of cache
    s = Scheduler(cache, max_tokens_per_step=32)
    s.add(SchedRequest(0, [1] * 8, 12))                        # grows to 19 tokens: 5 pages
    s.add(SchedRequest(1, [2] * 8, 12))
    log = run(s, cache)
    assert s.stats.preemptions >= 1
    r0, r1 = sorted(s.finished, key=lambda r: r.rid)
    assert len(r0.generated) == 12 and len(r1.generated) == 12
    assert r0.preemptions == 0 and r1.preemptions >= 1        # the one admitted last gives way
    # after eviction request 1 is recomputed from its prompt plus what it had generated
    refeeds = [n for step in log for rid, n, _ in step if rid == 1 and n > 8]
    assert refeeds, "the evicted request must come back with prompt + generated tokens"
    assert cache.live == 0 and cache.groups[0].pool.in_use == 0


def test_reserve_full_never_evicts():
    cache = _cache(num_pages=10, page=4)
    s = Scheduler(cache, max_tokens_per_step=32, reserve_full=True, admission_fraction=1.0)
    for i in range(3):
        s.add(SchedRequest(i, [1] * 8, 9))                    # 16 tokens -> 4 pages promised each
    log = run(s, cache)
    assert s.stats.preemptions == 0
    assert [rid for rid, _, _ in log[0]] == [0, 1]            # the third would break the promise
    assert s.promised == [0]


def test_a_request_that_can_never_fit_is_refused():
    cache = _cache(num_pages=3, page=4, ctx=64)
    s = Scheduler(cache, 32)
    with pytest.raises(ValueError, match="cache pages"):
        s.add(SchedRequest(0, [1] * 10, 8))
    with pytest.raises(ValueError, match="context limit"):
        s.add(SchedRequest(1, [1] * 60, 8))
    with pytest.raises(ValueError, match="empty prompt"):
        s.add(SchedRequest(2, [], 8))
    s.add(SchedRequest(3, [1] * 10, 3))                        # 12 tokens: exactly the pool
    run(s, cache)
    assert len(s.finished) == 1


@pytest.mark.parametrize("seed", range(24))
def test_random_loads_keep_every_promise(seed):
    """Random requests, budgets, chunk sizes, pools and slot counts (pools small enough to force evictions): every
    step stays under the token budget and the slot count, the pages it needs are there, nobody is fed a token twice
    or out of order, requests are admitted in arrival order, and everybody ends with the tokens it asked for.
    Every other seed has a second cache group with a window and a smaller pool of its own, whose pages go back
    while a request runs: the scheduler's counts must still be the cache manager's."""
    import random

    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    n_req = rng.randint(3, 14)
    reqs = [SchedRequest(i, [rng.randrange(100) for _ in range(rng.randint(1, 40))], rng.randint(1, 12)) for i in range(n_req)]
    biggest = max(-(-(len(r.prompt) + r.max_new_tokens - 1) // page) for r in reqs)
    num_pages = biggest + rng.randint(0, 2 * biggest)
    slots = rng.randint(1, 6)
    budget = rng.randint(2, 48)
    chunk = rng.choice([None, rng.randint(1, 16)])
    reserve_full = rng.random() < 0.3
    if seed % 2:
        window = rng.randint(1, 20)
        portion = min(chunk or budget, budget)
        longest = max(len(r.prompt) + r.max_new_tokens - 1 for r in reqs)
        small = CacheManager.most_pages_of_a_request(window, page, longest, portion)
        cache = CacheManager([CacheNeed(1, 16), CacheNeed(2, 8, window=window), CacheNeed(1, 16)], [None] * 3, page,
                             [num_pages, small + rng.randint(0, small)], slots, 64)
        assert len(cache.groups) == 2
    else:
        cache = _cache(num_pages, page=page, slots=slots, ctx=64)
    s = Scheduler(cache, max_tokens_per_step=budget, prefill_chunk=chunk, reserve_full=reserve_full)
    for r in reqs:
        s.add(r)
    fed = {r.rid: [] for r in reqs}          # what the cache of each request holds, in order
    first_seen = []
    for _ in range(20_000):
        if not s.has_work():
            break
        planned = s.plan()
        for v in s.evicted:
            cache.close(v.rid)
            fed[v.rid] = []                  # recomputed from its prompt and what it had generated
        assert planned
        assert sum(len(p.tokens) for p in planned) <= budget
        assert len({p.request.rid for p in planned}) == len(planned) <= slots
        batch = []
        for p in planned:
            r = p.request
            if r.rid not in first_seen:
                first_seen.append(r.rid)
            if not cache.is_open(r.rid):
                cache.open(r.rid)
            whole = r.prompt + [t for t in r.generated]
            assert p.tokens == whole[len(fed[r.rid]): len(fed[r.rid]) + len(p.tokens)], "a token was skipped or fed twice"
            assert p.samples == (len(fed[r.rid]) + len(p.tokens) == len(whole))
            fed[r.rid] += p.tokens
            batch.append((r.rid, len(fed[r.rid])))
        cache.reserve(batch)                 # never raises: the scheduler counted the pages
        for rid, n in batch:
            cache.commit(rid, n)
        cache.check()
        done = s.update(planned, [rng.randrange(100) for p in planned if p.samples])
        for r in done:
            cache.close(r.rid)
    assert not s.has_work(), "the scheduler did not finish"
    assert first_seen == sorted(first_seen), "admission is in arrival order"
    assert sorted(r.rid for r in s.finished) == list(range(n_req))
    assert all(len(r.generated) == r.max_new_tokens for r in s.finished)
    assert cache.live == 0 and all(g.pool.in_use == 0 for g in cache.groups)
    if reserve_full:
        assert s.stats.preemptions == 0
