"""The cache manager's bookkeeping (CPU): no page lost, held twice or freed twice."""
import random

import pytest

from velox_b200.cache import CacheAccountingError, CacheManager, PageAllocator, SlotAllocator
from velox_b200.parts.base import FixedState, PagedKV


def test_allocator_round_trip_and_order():
    a = PageAllocator(6)
    assert a.alloc(3) == [0, 1, 2]  # page 0 first (src/paged/pages.rs:113)
    assert a.alloc(4) is None and a.num_free == 3  # all or nothing
    a.free([1])
    assert a.alloc(1) == [1]  # the page just freed is the next one out
    a.free([0, 1, 2])
    assert a.num_free == 6


def test_double_free_and_bad_ids_raise():
    a = PageAllocator(4)
    p = a.alloc(2)
    a.free(p)
    with pytest.raises(CacheAccountingError):
        a.free([p[0]])
    with pytest.raises(CacheAccountingError):
        a.free([99])
    with pytest.raises(CacheAccountingError):
        a.incref([3])  # free page cannot be shared


def test_refcounts_share_pages():
    a = PageAllocator(4)
    p = a.alloc(2)
    a.incref(p)
    a.free(p)
    assert a.num_free == 2 and a.refcount(p[0]) == 1
    a.free(p)
    assert a.num_free == 4


def test_slots():
    s = SlotAllocator(2)
    assert (s.alloc(), s.alloc(), s.alloc()) == (0, 1, None)
    s.free(0)
    with pytest.raises(CacheAccountingError):
        s.free(0)
    assert s.alloc() == 0


def manager(num_pages=16, page=4, window=0, max_requests=4, max_blocks=64, mixed=False):
    specs = [PagedKV(2, 16, 0), PagedKV(2, 16, window), PagedKV(2, 16, window)] if mixed else [PagedKV(2, 16, window)] * 2
    return CacheManager(specs, [None] * len(specs), page, num_pages, max_requests, max_blocks)


def test_groups_by_need():
    m = manager(mixed=True, window=6)
    assert len(m.groups) == 2 and m.groups[0].layers == [0] and m.groups[1].layers == [1, 2]
    assert m.layer(0).group == 0 and m.layer(2).group == 1
    fixed = CacheManager([PagedKV(2, 16), FixedState((3, 5)), None], [None, None, 0], 4, 8, 2, 8)
    assert len(fixed.groups) == 1
    assert fixed.layer(2).group == 0 and not fixed.layer(2).writes  # reads layer 0's cache
    assert fixed.layer(1).group == -1


def test_reserve_commit_release():
    m = manager(num_pages=8, page=4)
    assert m.add_request("a") == 0
    assert m.pages_needed("a", 5) == [2]
    assert m.reserve("a", 5)
    m.commit("a", 5)
    assert m.length("a") == 5 and m.free_pages() == [6]
    assert m.pages_needed("a", 3) == [0] and m.pages_needed("a", 4) == [1]
    assert m.reserve("a", 1) and m.free_pages() == [6]
    m.commit("a", 1)
    assert not m.reserve("a", 100) and m.free_pages() == [6]  # nothing taken on failure
    m.check()
    m.release("a")
    assert m.free_pages() == [8] and m.slots.num_free == 4
    m.check()


def test_window_pages_come_back_while_the_request_lives():
    m = manager(num_pages=32, page=4, window=6, mixed=True)
    m.add_request("r")
    for _ in range(30):
        assert m.reserve("r", 1)
        m.commit("r", 1)
        m.check()
    full, windowed = m.requests["r"].tables
    assert all(p >= 0 for p in full) and len(full) == 8
    # next query is position 30: it sees keys 25..30, so pages 0..5 (positions < 24) are back
    assert [p >= 0 for p in windowed] == [False] * 6 + [True, True]
    assert m.free_pages() == [32 - 8, 32 - 2]
    m.release("r")
    assert m.free_pages() == [32, 32]
    m.check()


def test_random_orders_lose_nothing():
    rng = random.Random(7)
    for trial in range(20):
        m = manager(num_pages=rng.randint(6, 24), page=rng.choice([2, 4, 8]), window=rng.choice([0, 5, 9]),
                    mixed=rng.random() < 0.5)
        total = [g.allocator.num_pages for g in m.groups]
        live, next_id = [], 0
        for _ in range(300):
            op = rng.random()
            if op < 0.25 and len(live) < 4:
                assert m.add_request(next_id) is not None
                live.append(next_id)
                next_id += 1
            elif op < 0.85 and live:
                r = rng.choice(live)
                k = rng.choice([1, 1, 1, 2, 3, 7, 13])
                if m.length(r) + k <= m.max_blocks * m.page_size and m.reserve(r, k):
                    m.commit(r, k)
            elif live:
                r = live.pop(rng.randrange(len(live)))
                m.release(r)
            m.check()
        for r in live:
            m.release(r)
        m.check()
        assert m.free_pages() == total and m.slots.num_free == 4


def test_no_fifth_request_without_a_slot():
    m = manager(max_requests=2)
    assert m.add_request(0) == 0 and m.add_request(1) == 1 and m.add_request(2) is None
    with pytest.raises(CacheAccountingError):
        m.add_request(0)


def test_a_cache_need_of_unknown_kind_is_refused():
    from dataclasses import dataclass
    from velox_b200.cache import CacheManager

    @dataclass(frozen=True)
    class Unheard:
        size: int

    with pytest.raises(TypeError, match="unknown kind"):
        CacheManager([Unheard(3)], [None], 8, 4, 2, 4)
