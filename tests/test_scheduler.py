"""The scheduler's decisions, against the cache manager alone (no GPU): a stand-in for the step
function reserves and commits the pages and hands back made-up tokens."""
import random
import sys

import pytest

from quench6k_b200.cache import CacheManager, GroupSpec, NativeCacheManager, PyCacheManager
from quench6k_b200.engine.scheduler import (FINISH_CANCELLED, FINISH_LENGTH, FINISH_STOP, NativeScheduler, PyScheduler,
                                            Request, Scheduler)
from quench6k_b200.sampling import SamplingParams


@pytest.fixture(params=["native", "python"], autouse=True)
def backend(request, monkeypatch):
    """Every test of this file runs against the C++ cache manager and against its Python twin."""
    monkeypatch.setattr(sys.modules[__name__], "CacheManager", NativeCacheManager if request.param == "native" else PyCacheManager)
    return request.param


def make(pages=16, page_size=4, budget=16, max_requests=4, sliding=None):
    groups = [GroupSpec("full")] + ([GroupSpec("sliding", sliding)] if sliding else [])
    m = CacheManager(groups, page_size, [pages] * len(groups), max_requests)
    return m, Scheduler(m, max_batch_tokens=budget)


def run_step(m, s, token_of=lambda req: 7):
    plan = s.schedule()
    for e in plan.step_entries():
        m.reserve(e.rid, len(e.tokens))
    for e in plan.step_entries():
        m.commit(e.rid)
    sampled = [token_of(e.request) for e in plan.entries if e.samples]
    done = s.update(plan, sampled)
    m.check()
    return plan, done


def req(rid, n, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(temperature=0.0, **kw))


def test_prompt_is_cut_under_the_budget_and_then_decodes():
    m, s = make(pages=32, budget=8)
    s.add(req("a", 19, max_tokens=3))
    plan, _ = run_step(m, s)
    assert [(e.start, e.count, e.samples) for e in plan.entries] == [(0, 8, False)]
    plan, _ = run_step(m, s)
    assert [(e.start, e.count, e.samples) for e in plan.entries] == [(8, 8, False)]
    plan, _ = run_step(m, s)
    assert [(e.start, e.count, e.samples) for e in plan.entries] == [(16, 3, True)]
    plan, _ = run_step(m, s)
    assert [(e.start, e.count, e.samples) for e in plan.entries] == [(19, 1, True)]
    plan, done = run_step(m, s)
    assert [r.rid for r in done] == ["a"] and done[0].finish_reason == FINISH_LENGTH and len(done[0].output) == 3
    assert not s.has_work() and m.pools[0].num_free == 32 and m.slots.num_free == 4


def test_decode_tokens_come_first_and_portions_fill_the_rest():
    m, s = make(pages=64, budget=10)
    s.add(req("a", 4, max_tokens=50))
    run_step(m, s)                                    # a prefilled, first token sampled
    s.add(req("b", 30, max_tokens=5))
    plan, _ = run_step(m, s)
    assert [(e.request.rid, e.count, e.samples) for e in plan.entries] == [("a", 1, True), ("b", 9, False)]
    assert plan.num_tokens == 10
    plan, _ = run_step(m, s)
    assert [(e.request.rid, e.start, e.count) for e in plan.entries] == [("a", 5, 1), ("b", 9, 9)]


def test_stop_token_and_max_tokens_and_abort():
    m, s = make(pages=32)
    s.add(req("a", 3, max_tokens=10, stop_tokens=[42]))
    s.add(req("b", 3, max_tokens=2))
    s.add(req("c", 3, max_tokens=10))
    toks = iter([5, 5, 5, 42, 6, 9])
    plan, done = run_step(m, s, lambda r: next(toks))          # a:5 b:5 c:5
    assert not done
    s.abort("c")
    assert m.slots.num_free == 2                               # c's slot is back at once
    plan, done = run_step(m, s, lambda r: next(toks))          # a:42 -> stop, b:6 -> length
    reasons = {r.rid: r.finish_reason for r in done}
    assert reasons == {"a": FINISH_STOP, "b": FINISH_LENGTH}
    assert done[0].output[-1] == 42                            # the stop token is emitted
    assert not s.has_work() and m.pools[0].num_free == 32 and m.slots.num_free == 4


def test_waiting_prompt_waits_for_pages_fifo():
    m, s = make(pages=6, page_size=4, budget=64)               # 24 token places
    s.add(req("a", 14, max_tokens=4))
    s.add(req("b", 12, max_tokens=2))
    s.add(req("c", 2, max_tokens=2))
    plan, _ = run_step(m, s)
    # a takes 4 pages; b gets the 8 places that are left as a portion; c must not overtake b
    assert [(e.request.rid, e.count) for e in plan.entries] == [("a", 14), ("b", 8)]
    assert [r.rid for r in s.waiting] == ["c"]


def test_preemption_when_decode_runs_out_of_pages():
    m, s = make(pages=4, page_size=4, budget=64)               # 16 token places
    s.add(req("a", 7, max_tokens=20))
    s.add(req("b", 7, max_tokens=20))
    plan, _ = run_step(m, s)                                   # both prefilled: 2 pages each, pool empty
    assert m.pools[0].num_free == 0
    plan, _ = run_step(m, s)                                   # position 7 still fits in page 2
    assert not plan.preempted and len(plan.entries) == 2
    plan, _ = run_step(m, s)                                   # position 8 needs a new page: b (admitted last) is preempted
    assert [r.rid for r in plan.preempted] == ["b"]
    assert [e.request.rid for e in plan.entries][0] == "a"
    b = s.by_id["b"]
    assert b.preemptions == 1 and len(b.output) == 2
    # b comes back when a page frees up, recomputed from prompt + its output so far
    for _ in range(40):
        if not s.has_work():
            break
        run_step(m, s)
    assert not s.has_work()
    assert m.pools[0].num_free == 4 and m.slots.num_free == 4


def test_request_alone_that_fills_the_cache_ends_with_length():
    m, s = make(pages=3, page_size=4, budget=64)               # 12 token places
    with pytest.raises(ValueError, match="exceeds the cache capacity"):
        s.add(req("big", 12, max_tokens=5))
    s.add(req("a", 9, max_tokens=50))
    ended = []
    for _ in range(10):
        _, done = run_step(m, s)
        ended += done
        if not s.has_work():
            break
    assert [r.finish_reason for r in ended] == [FINISH_LENGTH]
    assert len(ended[0].prompt) + len(ended[0].output) <= 12
    assert m.pools[0].num_free == 3


@pytest.mark.parametrize("seed", range(4))
def test_random_traffic_finishes_everything(seed):
    rng = random.Random(seed)
    m, s = make(pages=24, page_size=4, budget=rng.choice([5, 16, 40]), max_requests=4, sliding=rng.choice([None, 6]))
    total, finished = 0, []
    for step in range(3000):
        if total < 25 and rng.random() < 0.3:
            n = rng.randint(1, 40)
            s.add(req(f"r{total}", n, max_tokens=rng.randint(1, 30), stop_tokens=[3]))
            total += 1
        if rng.random() < 0.02 and s.running:
            s.abort(rng.choice(s.running).rid)
        if s.has_work():
            plan, done = run_step(m, s, lambda r: rng.randint(0, 9))
            assert plan.num_tokens <= s.max_batch_tokens
            assert len({e.request.rid for e in plan.entries}) == len(plan.entries)
            finished += done + plan.finished
        elif total >= 25:
            break
    assert not s.has_work()
    assert all(p.num_free == 24 for p in m.pools) and m.slots.num_free == 4
    for r in finished:
        assert r.finish_reason in (FINISH_STOP, FINISH_LENGTH)
        assert 1 <= len(r.output) <= r.params.max_tokens


@pytest.mark.parametrize("seed", range(6))
def test_both_schedulers_decide_alike(seed):
    """The same random traffic (arrivals, sampled tokens, aborts) through the C++ scheduler and the
    Python one: the same entries, preemptions and endings in every step."""
    rng = random.Random(500 + seed)
    pages, ps = rng.choice([6, 12, 24]), rng.choice([2, 4])
    budget, sliding = rng.choice([3, 7, 16, 40]), rng.choice([None, 5])
    groups = [GroupSpec("full")] + ([GroupSpec("sliding", sliding)] if sliding else [])
    pair = []
    for cm, sc in ((NativeCacheManager, NativeScheduler), (PyCacheManager, PyScheduler)):
        m = cm(groups, ps, [pages] * len(groups), 4)
        admitted = []
        pair.append((m, sc(m, max_batch_tokens=budget, on_admit=admitted.append), admitted))
    total = 0
    for step in range(1500):
        if total < 30 and rng.random() < 0.35:
            n, mt = rng.randint(1, pages * ps - 1), rng.randint(1, 25)
            for m, s, _ in pair:
                s.add(req(("r", total), n, max_tokens=mt, stop_tokens=[3]))
            total += 1
        if rng.random() < 0.03 and pair[1][1].running:
            k = rng.randrange(len(pair[1][1].running))
            assert [r.rid for r in pair[0][1].running] == [r.rid for r in pair[1][1].running]
            for m, s, _ in pair:
                s.abort(s.running[k].rid)
        if rng.random() < 0.02 and pair[1][1].waiting:
            for m, s, _ in pair:
                s.abort(s.waiting[-1].rid)
        assert pair[0][1].has_work() == pair[1][1].has_work()
        if not pair[1][1].has_work():
            if total >= 30:
                break
            continue
        toks = [rng.randint(0, 9) for _ in range(8)]
        seen = []
        for m, s, admitted in pair:
            del admitted[:]
            it = iter(toks)
            plan, done = run_step(m, s, lambda r: next(it))
            seen.append(([(e.request.rid, e.start, e.count, e.samples) for e in plan.entries],
                         [r.rid for r in plan.preempted], [r.rid for r in plan.finished],
                         [(r.rid, r.finish_reason, list(r.output), r.preemptions) for r in done],
                         sorted(admitted), [p.num_free for p in m.pools], m.slots.num_free,
                         [(r.rid, r.num_computed, list(r.output)) for r in s.running], [r.rid for r in s.waiting]))
        assert seen[0] == seen[1], f"step {step}"
    assert total == 30 and not pair[0][1].has_work()


def test_placeholder_tokens_are_patched_and_a_late_stop_ends_the_request():
    """What the engine's look-ahead needs: a step is planned while the token before it is still a
    placeholder (-1); the value arrives later; a stop token found then ends the request at that
    token, whatever was planned or produced after it."""
    m, s = make(pages=32, budget=8)
    a, b = req("a", 5, max_tokens=10, stop_tokens=[3]), req("b", 6, max_tokens=2, stop_tokens=[3])
    s.add(a), s.add(b)
    run_step(m, s, lambda q: -1)                             # a's prompt and first token; three tokens of b's prompt
    plan, done = run_step(m, s, lambda q: -1)                # a decodes from a placeholder; b's prompt ends
    assert a.output == [-1, -1] and b.output == [-1] and not done
    assert [t for e in plan.step_entries() if e.rid == "a" for t in e.tokens] == [-1]
    s.set_output_token(a, 0, 7)
    s.set_output_token(b, 0, 3)                              # b's first token was a stop token: it ends there
    s.stop_at(b, 1)
    assert b.finish_reason == FINISH_STOP and b.output == [3] and m.slots.num_free == 3
    plan, done = run_step(m, s, lambda q: -1)
    assert [e.request.rid for e in plan.entries] == ["a"] and a.output == [7, -1, -1]
    s.set_output_token(a, 1, 3)                              # found a step late: the token after it is dropped
    s.stop_at(a, 2)
    assert a.finish_reason == FINISH_STOP and a.output == [7, 3]
    assert not s.has_work() and m.pools[0].num_free == 32 and m.slots.num_free == 4
    m.check()
    # a request that had already ended by length at the very token that turns out to be a stop token
    c = req("c", 3, max_tokens=1, stop_tokens=[3])
    s.add(c)
    plan, done = run_step(m, s, lambda q: -1)
    assert done == [c] and c.finish_reason == FINISH_LENGTH
    s.set_output_token(c, 0, 3)
    s.stop_at(c, 1)
    assert c.finish_reason == FINISH_STOP and c.output == [3] and not s.has_work()


def test_a_small_sliding_pool_bounds_nothing():
    """The capacity of a request is what the groups that keep every key can hold; a sliding group
    with a pool of a window's worth of pages neither refuses a long prompt nor ends a request early."""
    groups = [GroupSpec("full"), GroupSpec("sliding", 9)]
    m = CacheManager(groups, 4, [40, 8], 2)                  # 160 token places in the full group, 32 in the sliding one
    s = Scheduler(m, max_batch_tokens=6)
    assert s.capacity_tokens() == 160
    s.add(req("long", 100, max_tokens=20))                   # far beyond the sliding pool's 32 places
    with pytest.raises(ValueError):
        s.add(req("too long", 160))
    done = []
    for _ in range(200):
        if not s.has_work():
            break
        _, d = run_step(m, s)
        done += d
    assert [r.rid for r in done] == ["long"] and done[0].finish_reason == FINISH_LENGTH and len(done[0].output) == 20
    assert m.pools[0].num_free == 40 and m.pools[1].num_free == 8
    # a sliding pool that cannot hold its window and one more token is refused when the scheduler is made
    with pytest.raises(ValueError, match="window of 9 keys"):
        Scheduler(CacheManager(groups, 4, [40, 3], 2), max_batch_tokens=6)
