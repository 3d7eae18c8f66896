import random

import pytest

from quench6k_b200.cache import CacheManager, GroupSpec, OutOfPages, OutOfSlots, PagePool


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
