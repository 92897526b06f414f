"""The cache manager: pages, block tables, window release, state slots.  After every
operation under random orders of requests no page is lost, held twice or freed
twice."""
import random

import pytest

from inferx_b200.cache import CacheError, CacheGroup, CacheManager, PagePool, groups_for
from inferx_b200.parts import PagedKvNeed, StateNeed


def test_pool_hands_out_page_zero_first_and_refuses_double_free():
    pool = PagePool(3)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    assert pool.allocate() is None
    pool.release(1)
    assert pool.allocate() == 1            # LIFO: the page just freed comes back first
    pool.release(0)
    with pytest.raises(CacheError, match="freed twice"):
        pool.release(0)
    with pytest.raises(CacheError):
        pool.release(9)


def test_groups_are_formed_by_window():
    needs = [[PagedKvNeed(2, 16, 0)], [PagedKvNeed(2, 16, 8)], [PagedKvNeed(1, 32, 8)], [],
             [StateNeed("s", (4,))]]
    groups = groups_for(needs)
    assert [(g.window, g.layers) for g in groups] == [(0, (0,)), (8, (1, 2))]


def _mgr(pages=10, page=4, slots=3, windows=(0,)):
    return CacheManager([CacheGroup(window=w) for w in windows], pages, page, slots)


def test_reserve_is_all_or_nothing_over_groups():
    m = CacheManager([CacheGroup(0), CacheGroup(8)], [6, 2], 4, 2)
    assert m.open("a") == 0
    assert m.reserve("a", 8)                       # 2 pages in each group
    assert not m.reserve("a", 12)                  # group 1 has none left
    assert m.free_pages(0) == 4 and m.free_pages(1) == 0    # group 0's page was given back
    assert m.capacity("a") == 8
    m.check_invariants()


def test_window_group_gives_back_pages_behind_the_window():
    m = CacheManager([CacheGroup(0), CacheGroup(8)], 10, 4, 2)
    m.open("a")
    assert m.reserve("a", 20)
    m.advance("a", 20)
    # next query at position 20 sees keys from 13: pages 0,1,2 (positions 0..11) are dead
    assert list(m.table("a", 1)[:3]) == [-1, -1, -1] and m.table("a", 1)[3] >= 0
    assert all(p >= 0 for p in m.table("a", 0))
    assert m.pages_held("a", 1) == 2 and m.free_pages(1) == 8
    m.check_invariants()
    assert m.reserve("a", 24)
    m.advance("a", 4)
    assert m.table("a", 1)[3] == -1 and m.pages_held("a", 1) == 2
    m.close("a")
    assert m.free_pages(0) == 10 and m.free_pages(1) == 10 and m.free_slots() == 2
    m.check_invariants()


def test_slots_are_reported_fresh_once():
    m = _mgr(slots=2)
    assert m.open("a") == 0 and m.open("b") == 1
    assert m.open("c") is None
    assert sorted(m.take_fresh_slots()) == [0, 1] and m.take_fresh_slots() == []
    m.close("a")
    assert m.open("c") == 0 and m.take_fresh_slots() == [0]
    with pytest.raises(CacheError):
        m.open("c")
    with pytest.raises(CacheError):
        m.length("zzz")


def test_advance_beyond_capacity_is_an_error():
    m = _mgr()
    m.open("a")
    m.reserve("a", 4)
    with pytest.raises(CacheError, match="exceed"):
        m.advance("a", 5)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    windows = rng.choice([(0,), (0, 6), (5, 0, 11)])
    page = rng.choice([1, 2, 4, 8])
    pages = rng.randint(6, 24)
    m = CacheManager([CacheGroup(w) for w in sorted(set(windows))], pages, page,
                     rng.randint(1, 5))
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 or not live:
            rid = f"r{next_id}"
            next_id += 1
            if m.open(rid) is not None:
                live[rid] = 0
        elif op < 0.8:
            rid = rng.choice(list(live))
            n = rng.randint(1, 3 * page)
            if m.reserve(rid, live[rid] + n):
                m.advance(rid, n)
                live[rid] += n
                assert m.length(rid) == live[rid]
                for g, grp in enumerate(m.groups):
                    table = m.table(rid, g)
                    # every position the next query may see still has its page
                    lo = max(0, live[rid] - grp.window + 1) if grp.window else 0
                    for pos in range(lo, live[rid]):
                        assert table[pos // page] >= 0
            else:
                # a failed reserve changes nothing
                assert m.length(rid) == live[rid]
        else:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.close(rid)
    m.check_invariants()
    assert all(p.free_count == p.num_pages for p in m.pools)
    assert m.free_slots() == m.max_slots
