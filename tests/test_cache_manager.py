import random
import sys

import numpy as np
import pytest

from quench6k_b200.cache import (CacheManager, GroupSpec, NativeCacheManager, OutOfPages, OutOfSlots, PagePool,
                                 PyCacheManager)


@pytest.fixture(params=["native", "python"], autouse=True)
def backend(request, monkeypatch):
    """Every test of this file runs against the C++ cache manager and against its Python twin."""
    monkeypatch.setattr(sys.modules[__name__], "CacheManager", NativeCacheManager if request.param == "native" else PyCacheManager)
    return request.param


def test_pool_lifo_and_double_free():
    pool = PagePool(4)
    a, b = pool.take("x"), pool.take("y")
    assert (a, b) == (0, 1)
    pool.give_back(a, "x")
    assert pool.take("z") == a                      # the page just freed is used again
    with pytest.raises(RuntimeError, match="belongs to"):
        pool.give_back(b, "x")
    pool.give_back(b, "y")
    with pytest.raises(RuntimeError, match="freed twice"):
        pool.give_back(b, "y")
    pool.take("q"), pool.take("q"), pool.take("q")
    with pytest.raises(OutOfPages):
        pool.take("q")


def test_full_group_pages_follow_length():
    m = CacheManager([GroupSpec("full")], page_size=4, num_pages=[8], max_requests=2)
    m.add("a")
    assert m.pages_needed("a", 9) == [3]
    m.reserve("a", 9)
    m.commit("a")
    assert m.length("a") == 9 and m.table("a", 0) == [0, 1, 2]
    assert m.pages_needed("a", 3) == [0] and m.pages_needed("a", 4) == [1]
    m.reserve("a", 4)
    m.commit("a")
    assert len(m.table("a", 0)) == 4
    m.check()
    m.remove("a")
    assert m.pools[0].num_free == 8
    m.check()


def test_sliding_group_returns_pages_the_window_has_passed():
    W, ps = 6, 4
    m = CacheManager([GroupSpec("full"), GroupSpec("sliding", W)], page_size=ps, num_pages=[16, 16], max_requests=2)
    m.add("a")
    m.reserve("a", 10)
    m.commit("a")
    # next query at position 10 sees keys 5..10: block 0 (positions 0..3) is dead, block 1 (4..7) is not
    assert m.table("a", 1)[0] == -1 and m.table("a", 1)[1] >= 0 and m.table("a", 1)[2] >= 0
    assert all(p >= 0 for p in m.table("a", 0))
    for _ in range(30):
        m.reserve("a", 1)
        m.commit("a")
        m.check()
    held = [p for p in m.table("a", 1) if p >= 0]
    assert len(held) <= (W + ps - 1) // ps + 1
    n = m.length("a")
    lo = n - W + 1                                   # oldest key the next query sees
    tab = m.table("a", 1)
    for pos in range(lo, n):
        assert tab[pos // ps] >= 0
    m.remove("a")
    assert m.pools[0].num_free == 16 and m.pools[1].num_free == 16


def test_reserve_is_all_or_nothing():
    m = CacheManager([GroupSpec("full"), GroupSpec("sliding", 5)], page_size=4, num_pages=[8, 2], max_requests=2)
    m.add("a")
    assert not m.can_reserve([("a", 12)])            # the sliding pool has 2 pages, 12 tokens need 3
    with pytest.raises(OutOfPages):
        m.reserve("a", 12)
    assert m.pools[0].num_free == 8 and m.pools[1].num_free == 2 and m.length("a") == 0
    m.reserve("a", 8)
    m.commit("a")
    m.check()


def test_slots():
    m = CacheManager([GroupSpec("full")], page_size=4, num_pages=[4], max_requests=2)
    s0, s1 = m.add("a"), m.add("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(OutOfSlots):
        m.add("c")
    with pytest.raises(KeyError):
        m.add("a")
    m.remove("a")
    assert m.add("c") == s0
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    ps = rng.choice([2, 4, 16])
    groups = [GroupSpec("full"), GroupSpec("sliding", rng.choice([3, 9, 33]))]
    m = CacheManager(groups, page_size=ps, num_pages=[40, 24], max_requests=4)
    live, n = [], 0
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 4:
            rid = f"r{n}"
            n += 1
            m.add(rid)
            live.append(rid)
        elif op < 0.25 and live:
            rid = live.pop(rng.randrange(len(live)))
            m.remove(rid)
        elif live:
            rid = rng.choice(live)
            k = rng.choice([1, 1, 1, 2, 5, 13])
            if m.can_reserve([(rid, k)]):
                m.reserve(rid, k)
                if rng.random() < 0.1:
                    m.cancel(rid)
                else:
                    m.commit(rid)
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, k)
        m.check()
    for rid in live:
        m.remove(rid)
    m.check()
    assert m.pools[0].num_free == 40 and m.pools[1].num_free == 24 and m.slots.num_free == 4


@pytest.mark.parametrize("seed", range(4))
def test_both_managers_agree_on_tables_and_packed_steps(seed):
    """The same random traffic through the C++ manager and the Python one: the same pages in the
    same blocks, the same free counts, and the same packed step description."""
    rng = random.Random(100 + seed)
    ps = rng.choice([2, 4, 16])
    groups = [GroupSpec("full"), GroupSpec("sliding", rng.choice([3, 9, 33]))]
    pair = [cls(groups, page_size=ps, num_pages=[40, 24], max_requests=4) for cls in (NativeCacheManager, PyCacheManager)]
    live, n = [], 0
    for _ in range(400):
        op = rng.random()
        if op < 0.15 and len(live) < 4:
            rid = ("r", n)
            n += 1
            assert len({m.add(rid) for m in pair}) == 1
            live.append(rid)
        elif op < 0.25 and live:
            rid = live.pop(rng.randrange(len(live)))
            for m in pair:
                m.remove(rid)
        elif live:
            rid = rng.choice(live)
            k = rng.choice([1, 1, 2, 5, 13])
            assert pair[0].pages_needed(rid, k) == pair[1].pages_needed(rid, k)
            ok = {m.can_reserve([(rid, k)]) for m in pair}
            assert len(ok) == 1
            if ok.pop():
                # the packed description of a step over every live request that can run one token more
                for m in pair:
                    m.reserve(rid, k)
                others = [r for r in live if r != rid and pair[1].pages_needed(r, 1) == [0, 0]][:2]
                rids = [rid] + others
                toks = [[rng.randrange(50) for _ in range(k)]] + [[rng.randrange(50)] for _ in others]
                want = [[k - 1]] + [[0] for _ in others]
                widths = [max(1, max(pair[1].table_len(r, g) for r in rids)) + g for g in range(2)]
                blocks = []
                pad = rng.choice([0, 0, 1, 3])
                for m in pair:
                    out = np.full(4096, -7, dtype=np.int32)
                    meta = m.pack_step(rids, toks, want, widths, 50, out, 0, pad, [31, 32], 9)
                    blocks.append((meta, out[:meta[0]].tolist()))
                assert blocks[0] == blocks[1]
                for m in pair:
                    m.commit(rid)
        for rid in live:
            assert [pair[0].table(rid, g) for g in range(2)] == [pair[1].table(rid, g) for g in range(2)]
            assert pair[0].length(rid) == pair[1].length(rid) and pair[0].slot(rid) == pair[1].slot(rid)
        assert [p.num_free for p in pair[0].pools] == [p.num_free for p in pair[1].pools]
        for m in pair:
            m.check()


def test_pack_step_refuses_bad_tokens_and_places():
    m = CacheManager([GroupSpec("full")], page_size=4, num_pages=[8], max_requests=2)
    m.add("a")
    m.reserve("a", 3)
    out = np.zeros(256, dtype=np.int32)
    with pytest.raises(ValueError, match="token id outside"):
        m.pack_step(["a"], [[1, 99, 2]], [[2]], [1], 50, out)
    with pytest.raises(ValueError, match="wanted place 3"):
        m.pack_step(["a"], [[1, 2, 3]], [[3]], [1], 50, out)
    with pytest.raises(ValueError):
        m.pack_step(["a"], [[1, 2, 3]], [[2]], [1], 50, out[:5])
    total, T, W, ctx, q = m.pack_step(["a"], [[1, 2, 3]], [[0, 2]], [2], 50, out)
    assert (T, W, ctx, q) == (3, 2, 3, 3)
    assert out[:total].tolist() == [1, 2, 3, 0, 1, 2, 0, 0, 0, 0, 3, 0, m.slot("a"), 0, 2, 0, -1]


@pytest.mark.parametrize("backend", ["python", "native"])
def test_pack_step_appends_filler_entries(backend):
    """Filler entries after the real ones: one token 0 at position 0 each, its logits wanted, the
    given slot, and one page per group that the manager never hands out."""
    from quench6k_b200.cache import NativeCacheManager, PyCacheManager
    cls = PyCacheManager if backend == "python" else NativeCacheManager
    m = cls([GroupSpec("full"), GroupSpec("sliding", 8)], page_size=4, num_pages=[8, 6], max_requests=2)
    m.add("a")
    m.reserve("a", 3)
    out = np.full(256, -7, dtype=np.int32)
    total, T, W, ctx, q = m.pack_step(["a"], [[4, 5, 6]], [[2]], [2, 3], 50, out, 0, 2, [8, 6], 2)
    assert (T, W, ctx, q) == (5, 3, 3, 3)
    a0, a1 = m.table("a", 0)[0], m.table("a", 1)[0]
    assert out[:total].tolist() == ([4, 5, 6, 0, 0] + [0, 1, 2, 0, 0] + [0, 0, 0, 1, 2] + [0, 3, 4, 5] + [0, 0, 0] + [m.slot("a"), 2, 2]
                                    + [2, 3, 4] + [a0, -1, 8, -1, 8, -1] + [a1, -1, -1, 6, -1, -1, 6, -1, -1])
    with pytest.raises(ValueError):
        m.pack_step(["a"], [[4, 5, 6]], [[2]], [2, 3], 50, out, 0, 1, [8], 2)

