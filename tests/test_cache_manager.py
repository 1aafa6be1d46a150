"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; groups have pages of their own."""

import random

import pytest

from lalamo_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool, SlotPool, plan_cache_layout
from lalamo_b200.parts.base import PagedKVNeed, SlotStateNeed

FULL = PagedKVNeed(num_groups=2, head_dim=16)
WINDOWED = PagedKVNeed(num_groups=1, head_dim=32, window=20)
STATE = SlotStateNeed(shape=(2, 64))


def manager(needs, cache_from=None, page_size=4, num_pages=12, num_slots=3):
    return CacheManager(needs, cache_from or [None] * len(needs), None, page_size=page_size, num_pages=num_pages, num_slots=num_slots)


def test_page_pool_basics():
    pool = PagePool(4)
    pages = pool.allocate(3)
    assert sorted(pages) == [0, 1, 2] and pool.free_count == 1
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    assert pool.free_count == 1  # nothing was taken
    pool.release([pages[1]])
    with pytest.raises(ValueError, match="freed twice"):
        pool.release([pages[1]])
    with pytest.raises(ValueError, match="outside"):
        pool.release([9])
    assert pool.allocate(1) == [pages[1]]  # last freed, first reused
    pool.check()


def test_slot_pool():
    slots = SlotPool(2)
    a, b = slots.allocate(), slots.allocate()
    with pytest.raises(OutOfSlots):
        slots.allocate()
    slots.release(a)
    with pytest.raises(ValueError):
        slots.release(a)
    assert slots.allocate() == a and b != a


def test_layout_groups_by_retention_rule():
    layout = plan_cache_layout([STATE, FULL, WINDOWED, FULL, None, FULL], [None, None, None, None, None, 1])
    assert layout.group_windows == [None, 20]
    assert layout.group_entries == [[1, 3], [2]]
    assert layout.entry_group == [None, 0, 1, 0, None, 0]
    assert layout.entry_owner == [0, 1, 2, 3, None, 1]  # entry 5 reads entry 1's cache
    assert layout.slot_entries == [0]
    with pytest.raises(ValueError):
        plan_cache_layout([STATE, None], [None, 0][::-1])


def test_reserve_is_all_or_nothing_and_release_returns_everything():
    cache = manager([STATE, FULL], num_pages=5)
    cache.admit("a")
    cache.reserve("a", 9)  # 3 pages of 4
    assert cache.free_pages() == 2 and cache.pages_needed("a", 12) == 0 and cache.pages_needed("a", 13) == 1
    cache.admit("b")
    with pytest.raises(OutOfPages):
        cache.reserve("b", 12)
    assert cache.free_pages() == 2 and cache.requests["b"].blocks[0] == []
    cache.commit("a", 9)
    cache.check()
    cache.release("a")
    cache.release("b")
    assert cache.free_pages() == 5 and cache.slots.free_count == 3
    with pytest.raises(KeyError):
        cache.release("a")
    cache.admit("c")
    with pytest.raises(ValueError, match="already live"):
        cache.admit("c")


def test_window_gives_pages_back_and_groups_are_separate():
    cache = manager([FULL, WINDOWED], page_size=4, num_pages=12)
    cache.admit("r")
    cache.reserve("r", 30)
    cache.commit("r", 30)
    full, windowed = cache.requests["r"].blocks[0], cache.requests["r"].blocks[1]
    assert len(full) == 8 and all(page >= 0 for page in full)
    # later queries (position >= 30) see keys j > 30 - 20 = 10, i.e. from 11 on: blocks 0 and 1 (keys 0..7) are dead
    assert [page >= 0 for page in windowed] == [False, False, True, True, True, True, True, True]
    assert cache.groups[0].pool.free_count == 4 and cache.groups[1].pool.free_count == 6
    cache.check()
    cache.reserve("r", 41)
    cache.commit("r", 41)
    assert sum(page >= 0 for page in cache.requests["r"].blocks[1]) == 6  # keys from 22 on: blocks 5..10
    cache.release("r")
    cache.check()
    assert cache.free_pages() == 12


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    generator = random.Random(seed)
    cache = manager([STATE, FULL, WINDOWED, FULL], page_size=4, num_pages=24, num_slots=4)
    live: dict[int, int] = {}
    next_id = 0
    reused = False
    ever_freed: set[int] = set()
    for _ in range(600):
        action = generator.random()
        if action < 0.25 and len(live) < 4:
            cache.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            request = generator.choice(list(live))
            grow = generator.choice([1, 1, 1, 2, 5, 9, 17])
            try:
                cache.reserve(request, live[request] + grow)
            except OutOfPages:
                before = {g: list(blocks) for g, blocks in cache.requests[request].blocks.items()}
                assert before == cache.requests[request].blocks
            else:
                new_pages = set(cache.requests[request].blocks[0])
                reused |= bool(new_pages & ever_freed)
                live[request] += grow
                cache.commit(request, live[request])
        elif live:
            request = generator.choice(list(live))
            ever_freed |= {page for page in cache.requests[request].blocks[0] if page >= 0}
            cache.release(request)
            del live[request]
        cache.check()
    for request in list(live):
        cache.release(request)
    cache.check()
    assert cache.free_pages() == 24 and cache.slots.free_count == 4
    assert reused  # pages did go round


def test_block_table_rows_are_padded():
    cache = manager([FULL], num_pages=8)
    cache.admit("a")
    cache.admit("b")
    cache.reserve("a", 9)
    cache.reserve("b", 2)
    (rows,) = cache.block_table_rows(["b", "a"])
    assert len(rows) == 2 and len(rows[0]) == len(rows[1]) == 3
    assert rows[0][1:] == [-1, -1] and all(page >= 0 for page in rows[1])
