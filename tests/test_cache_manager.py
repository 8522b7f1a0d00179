"""The paged cache's bookkeeping: no page lost, held twice or freed twice (no GPU)."""

import random

import pytest

from matricxon_b200.cache.manager import (
    CacheError,
    CacheManager,
    GroupRule,
    OutOfPages,
    PagePool,
    SlotPool,
)


def make(window=None, pages=16, page_size=4, slots=4, groups=1):
    rules = [GroupRule(window=window)] * groups
    return CacheManager(rules, pages, page_size, slots)


def test_pool_allocate_release_and_double_free():
    pool = PagePool(4)
    pages = pool.allocate(3)
    assert pages == [0, 1, 2] and pool.free_count == 1
    pool.release([1])
    assert pool.allocate(1) == [1]                 # the page freed last is used again first
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    pool.release([0])
    with pytest.raises(CacheError):
        pool.release([0])
    with pytest.raises(CacheError):
        pool.release([9])


def test_slot_pool():
    slots = SlotPool(2)
    a, b = slots.allocate(), slots.allocate()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        slots.allocate()
    slots.release(a)
    with pytest.raises(CacheError):
        slots.release(a)


def test_reserve_commit_free():
    cache = make()
    cache.add_request("a")
    assert cache.pages_needed("a", 5) == [2]
    cache.reserve("a", 5)
    assert cache.record("a").reserved == 5 and cache.free_pages() == [14]
    assert cache.slot_ids("a", 0, 0, 5).tolist() == [0, 1, 2, 3, 4]
    cache.commit("a", 5)
    assert cache.record("a").length == 5
    assert cache.pages_needed("a", 3) == [0]       # room left in the second page
    assert cache.pages_needed("a", 4) == [1]
    cache.reserve("a", 4)
    cache.commit("a", 4)
    assert cache.held_pages("a", 0) == [0, 1, 2]
    cache.check_invariants()
    cache.free_request("a")
    assert cache.free_pages() == [16]
    with pytest.raises(CacheError):
        cache.free_request("a")
    cache.check_invariants()


def test_out_of_pages_takes_nothing():
    cache = make(pages=3, groups=2)
    cache.add_request("a")
    cache.add_request("b")
    cache.reserve("a", 8)
    before = cache.free_pages()
    with pytest.raises(OutOfPages):
        cache.reserve("b", 8)
    assert cache.free_pages() == before and cache.record("b").reserved == 0
    assert not cache.can_reserve("b", 8) and cache.can_reserve("b", 4)
    cache.check_invariants()


def test_commit_more_than_reserved_is_an_error():
    cache = make()
    cache.add_request("a")
    cache.reserve("a", 2)
    with pytest.raises(CacheError):
        cache.commit("a", 3)


def test_cancel_reservation_returns_only_uncommitted_pages():
    cache = make()
    cache.add_request("a")
    cache.reserve("a", 6)
    cache.commit("a", 6)                            # pages 0, 1 (second half full)
    cache.reserve("a", 7)                           # needs pages for positions 6..12
    assert len(cache.held_pages("a", 0)) == 4
    cache.cancel_reservation("a")
    assert len(cache.held_pages("a", 0)) == 2 and cache.record("a").reserved == 0
    cache.check_invariants()


def test_window_releases_pages_the_next_query_cannot_see():
    cache = make(window=6, page_size=4)
    cache.add_request("a")
    cache.reserve("a", 9)
    cache.commit("a", 9)
    # length 9: the next query (p >= 9) sees j > 3, so page 0 (positions 0..3) is gone
    assert cache.record("a").tables[0] == [-1, 1, 2]
    cache.reserve("a", 1)
    cache.commit("a", 1)                            # length 10: j > 4, page 1 holds 4..7: stays
    assert cache.record("a").tables[0] == [-1, 1, 2]
    cache.reserve("a", 4)
    cache.commit("a", 4)                            # length 14: j > 8 -> page 1 goes; page 0 reused
    assert cache.record("a").tables[0][:2] == [-1, -1]
    assert cache.pages_reused >= 1
    with pytest.raises(CacheError):
        cache.slot_ids("a", 0, 2, 1)                # a released position has no slot
    cache.check_invariants()


def test_window_boundary_is_exact():
    # window 4, page 4: after length 7 the next query p=7 sees j in 4..7 -> page 0 released
    cache = make(window=4, page_size=4)
    cache.add_request("a")
    cache.reserve("a", 6)
    cache.commit("a", 6)                            # p=6 sees 3..6: page 0 still needed
    assert cache.record("a").tables[0][0] >= 0
    cache.reserve("a", 1)
    cache.commit("a", 1)
    assert cache.record("a").tables[0][0] == -1


def test_groups_have_tables_of_their_own():
    cache = CacheManager([GroupRule(None), GroupRule(4)], [8, 8], 4, 2)
    cache.add_request("a")
    cache.reserve("a", 12)
    cache.commit("a", 12)
    full, sliding = cache.record("a").tables
    assert all(page >= 0 for page in full) and sliding[:2] == [-1, -1]
    assert cache.free_pages() == [5, 7]
    cache.check_invariants()


def test_requests_and_slots():
    cache = make(slots=2)
    a, b = cache.add_request("a"), cache.add_request("b")
    assert a.state_slot != b.state_slot
    with pytest.raises(CacheError):
        cache.add_request("a")
    with pytest.raises(OutOfPages):
        cache.add_request("c")
    cache.free_request("a")
    assert cache.add_request("c").state_slot == a.state_slot


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 5, 16, 33])
    cache = CacheManager([GroupRule(window), GroupRule(None)], [24, 40], rng.choice([2, 4, 16]), 4)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and len(live) < 4:
            name = f"r{counter}"
            counter += 1
            cache.add_request(name)
            live[name] = 0
        elif action < 0.85 and live:
            name = rng.choice(list(live))
            count = rng.choice([1, 1, 1, 2, 7, 19])
            try:
                cache.reserve(name, count)
            except OutOfPages:
                victim = max(live, key=live.get)
                cache.free_request(victim)
                del live[victim]
                cache.check_invariants()
                continue
            if rng.random() < 0.1:
                cache.cancel_reservation(name)
            else:
                cache.commit(name, count)
                live[name] += count
        elif live:
            name = rng.choice(list(live))
            cache.free_request(name)
            del live[name]
        cache.check_invariants()
        for name, length in live.items():
            assert cache.record(name).length == length
    for name in list(live):
        cache.free_request(name)
    assert cache.free_pages() == [24, 40] and cache.slots.free_count == 4
