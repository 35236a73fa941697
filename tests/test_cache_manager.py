"""The cache manager: demand, allocation order, give-back, windows, slots; and
that under random orders of requests no page is lost, held twice or freed twice."""

import random

import pytest

from shrike_b200.cache import CacheError, CacheManager, IdPool, KVGroupSpec, group_caches
from shrike_b200.parts.base import KVNeed

FULL = KVGroupSpec((0, 1), 2, 16, None)
WINDOW = KVGroupSpec((2,), 2, 16, 10)


def test_delta_allocation_and_free():
    # 10 tokens at page size 4 -> 3 pages; the 13th token needs a 4th
    # (shrike tests/test_block_manager.py:11-58).
    manager = CacheManager([FULL], 4, 8, 4)
    cache = manager.open()
    assert manager.pages_needed(cache, 0, 10) == [3]
    manager.append(cache, 0, 10)
    assert cache.tables[0].tolist() == [0, 1, 2] and manager.num_free == [5]
    assert manager.pages_needed(cache, 10, 2) == [0]
    assert manager.pages_needed(cache, 12, 1) == [1]
    manager.append(cache, 12, 1)
    assert cache.tables[0].tolist() == [0, 1, 2, 3]
    manager.free(cache)
    assert manager.whole() and manager.num_free == [8]


def test_exact_fill_boundary():
    # 2 pages of 4: 8 tokens fit, 9 do not (shrike tests/test_block_manager_edges.py:15-67).
    manager = CacheManager([FULL], 4, 2, 4)
    assert manager.can_append(None, 0, 8) and not manager.can_append(None, 0, 9)
    cache = manager.open()
    manager.append(cache, 0, 8)
    assert not manager.can_append(cache, 8, 1)
    with pytest.raises(CacheError, match="without room"):
        manager.append(cache, 8, 1)


def test_freed_pages_are_reused_in_fifo_order():
    manager = CacheManager([FULL], 4, 4, 4)
    a, b = manager.open(), manager.open()
    manager.append(a, 0, 8)   # pages 0, 1
    manager.append(b, 0, 4)   # page 2
    manager.free(a)           # free list: 3, 0, 1
    c = manager.open()
    manager.append(c, 0, 12)
    assert c.tables[0].tolist() == [3, 0, 1]


def test_double_free_and_use_after_free_raise():
    manager = CacheManager([FULL], 4, 4, 2)
    cache = manager.open()
    manager.append(cache, 0, 5)
    manager.free(cache)
    with pytest.raises(CacheError, match="twice"):
        manager.free(cache)
    with pytest.raises(CacheError, match="freed"):
        manager.append(cache, 0, 1)
    pool = IdPool(2)
    ident = pool.take()
    pool.give_back(ident)
    with pytest.raises(CacheError, match="not held"):
        pool.give_back(ident)


def test_slots_are_taken_and_returned():
    manager = CacheManager([FULL], 4, 16, 2)
    a, b = manager.open(), manager.open()
    assert {a.slot, b.slot} == {0, 1} and not manager.can_open()
    assert not manager.can_append(None, 0, 1)
    manager.free(a)
    assert manager.can_open() and manager.open().slot == 0


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    manager = CacheManager([FULL, WINDOW], 4, [16, 6], 4)
    cache = manager.open()
    manager.append(cache, 0, 9)
    assert cache.tables[0].tolist() == [0, 1, 2] and cache.tables[1].tolist() == [0, 1, 2]
    assert manager.num_free == [13, 3]
    assert manager.advance(cache, 9) == 0          # next query at 9 sees keys 0..9: nothing passed
    manager.append(cache, 9, 8)
    assert manager.advance(cache, 17) == 2         # next query at 17 sees 8..17: pages 0, 1 passed
    assert cache.tables[1].tolist() == [-1, -1, 2, 3, 4] and manager.num_free == [11, 3]
    assert cache.tables[0].tolist() == [0, 1, 2, 3, 4]   # the group that keeps all keys gave nothing back
    manager.append(cache, 17, 4)
    assert cache.tables[1].tolist()[-1] == 5         # the FIFO order of the group's own pool
    manager.free(cache)
    assert manager.whole()


def test_group_caches_merges_equal_needs():
    needs = {0: KVNeed(2, 16, None), 1: KVNeed(2, 16, 24), 2: KVNeed(2, 16, None), 3: KVNeed(2, 16, 24), 4: KVNeed(1, 16, None)}
    groups = group_caches(needs)
    assert [g.cache_ids for g in groups] == [(0, 2), (1, 3), (4,)]
    assert [g.window for g in groups] == [None, 24, None]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    page_size = rng.choice([1, 4, 16])
    counts = [rng.randrange(6, 30), rng.randrange(6, 30)]
    manager = CacheManager([FULL, KVGroupSpec((2,), 1, 32, rng.choice([3, 10, 50]))], page_size, counts, 5)
    live = []  # (cache, computed)
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and manager.can_open() and len(live) < 5:
            n = rng.randrange(1, 40)
            if manager.can_append(None, 0, n):
                cache = manager.open()
                manager.append(cache, 0, n)
                live.append([cache, n])
                manager.advance(cache, n)
        elif action < 0.8 and live:
            entry = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 7, 19])
            if manager.can_append(entry[0], entry[1], n):
                manager.append(entry[0], entry[1], n)
                entry[1] += n
                manager.advance(entry[0], entry[1])
        elif live:
            entry = live.pop(rng.randrange(len(live)))
            manager.free(entry[0])
        # invariants: every page is free or held exactly once; counts add up
        for group, pool in enumerate(manager.pools):
            held = [p for cache, _ in live for p in cache.tables[group].tolist() if p >= 0]
            assert len(held) == len(set(held)), "a page is held twice"
            assert not set(held) & set(pool.free_queue), "a held page is on the free list"
            assert len(held) + pool.num_free == pool.count, "a page was lost"
            assert len(set(pool.free_queue)) == pool.num_free, "a page is on the free list twice"
        for cache, computed in live:
            need = manager.blocks_for(computed)
            assert all(table.length >= need for table in cache.tables)
            window = manager.groups[1].window
            first_block = max(0, computed - window + 1) // page_size
            assert all(p >= 0 for p in cache.tables[1].tolist()[first_block:]), "a page inside the window is gone"
            assert all(p >= 0 for p in cache.tables[0].tolist())
        slots = [cache.slot for cache, _ in live]
        assert len(slots) == len(set(slots))
    for cache, _ in live:
        manager.free(cache)
    assert manager.whole()


def test_pools_are_sized_by_need():
    """Groups that keep every key share the budget in equal page counts; a group with a window
    gets no more than its requests can hold at once; per-request state comes off the budget first
    (that is the caller's part: the budget given here is what is left for pages)."""
    from shrike_b200.cache.manager import pages_in_flight, pages_per_group

    page = 16
    full, window = KVGroupSpec((0,), 2, 16, None), KVGroupSpec((1,), 2, 16, 100)
    # a window of 100 and portions of 64: from key p - 99 to key p + 63 -> at most 12 pages of 16
    assert pages_in_flight(1000, 100, 64, page) == (100 + 64 - 2) // 16 + 2 == 12
    assert pages_in_flight(5, 100, 64, page) == 5 and pages_in_flight(1000, None, 64, page) == 1000
    bytes_per_page = [1000, 1000]
    counts = pages_per_group([full, window], page, 1_000_000, bytes_per_page, 4, 64)
    assert counts == [1_000_000 // 1000 - 48, 48]          # 4 requests x 12 pages, the rest to the full group
    assert pages_per_group([full, window], page, 50_000, bytes_per_page, 4, 64) == [25, 25]   # too little to reach the cap
    assert pages_per_group([window], page, 1_000_000, [1000], 4, 64) == [48]
    assert pages_per_group([], page, 1_000_000, [], 4, 64) == []
    manager = CacheManager([full, window], page, counts, 4)
    assert manager.total_pages == counts[0] and manager.portion_limit() == (48 - 2) * 16 - 100 + 2
    assert manager.worst_case_pages(5000, 64) == [313, 12] and manager.worst_case_pages(5000) == [313, 313]
    assert CacheManager([full], page, 8, 4).portion_limit() is None


def test_opened_slots_are_remembered_until_taken():
    manager = CacheManager([FULL], 4, 8, 3)
    a, b = manager.open(), manager.open()
    assert manager.take_opened() == [a.slot, b.slot] and manager.take_opened() == []
    manager.free(a)
    c = manager.open()
    assert manager.take_opened() == [c.slot]


def test_a_manager_without_page_groups_keeps_slots_only():
    manager = CacheManager([], 16, [], 2)
    assert manager.can_append(None, 0, 1000) and manager.total_pages == 0 and manager.free_pages == 0
    a, b = manager.open(), manager.open()
    manager.append(a, 0, 500)
    assert not manager.can_append(None, 0, 1) and manager.has_room(a, 10_000)
    manager.free(a)
    manager.free(b)
    assert manager.whole()
