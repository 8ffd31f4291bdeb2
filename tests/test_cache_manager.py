"""The cache manager on the CPU: allocator, block tables and slots, step transactions, windows,
prefix reuse, state slots; no page lost, held twice or freed twice under random orders."""

from __future__ import annotations

import random

import pytest

import miniserve_b200  # noqa: F401
from miniserve_b200.cache import (RELEASED, CacheManager, OutOfPagesError, OutOfSlotsError, PageAllocator, StateSlots)
from miniserve_b200.parts import CacheGroup, PagedKVNeed, StateNeed

FULL = CacheGroup(PagedKVNeed(2, 16, None), 3)


def window_group(window):
    return CacheGroup(PagedKVNeed(2, 16, window), 2)


def test_allocator_lowest_first_refcounts_and_atomic_failure():
    allocator = PageAllocator(4)
    assert allocator.allocate(2) == [0, 1]
    allocator.retain(1)
    assert allocator.release(1) is False and allocator.release(1) is True
    assert allocator.allocate(1) == [1]
    with pytest.raises(OutOfPagesError, match="requested=3, free=2"):
        allocator.allocate(3)
    assert allocator.free_count == 2
    with pytest.raises(RuntimeError, match="freed twice"):
        allocator.release(3)
    with pytest.raises(RuntimeError, match="retained"):
        allocator.retain(3)
    allocator.check_invariants()


def test_state_slots_lifecycle():
    slots = StateSlots(2)
    a, b = slots.allocate("a"), slots.allocate("b")
    assert (a, b) == (0, 1) and slots.owner(1) == "b"
    with pytest.raises(OutOfSlotsError):
        slots.allocate("c")
    slots.release(a)
    with pytest.raises(RuntimeError, match="freed twice"):
        slots.release(a)
    assert slots.allocate("c") == 0
    slots.check_invariants()


def test_slots_follow_non_contiguous_tables():
    manager = CacheManager([FULL], page_size=16, num_pages=8, max_seqs=4)
    manager.admit("a"), manager.admit("b")
    r = manager.prepare([("a", 17), ("b", 3)])
    assert r.items[0].tables == [[0, 1]] and r.items[1].tables == [[2]]
    manager.commit(r)
    r = manager.prepare([("a", 16), ("b", 30)])          # a: page 3; b: pages 4, 5
    a, b = r.items
    assert a.tables == [[0, 1, 3]] and b.tables == [[2, 4, 5]]
    for position, slot in zip(range(17, 33), a.slots[0]):
        assert slot == a.tables[0][position // 16] * 16 + position % 16
    assert list(b.slots[0][12:15]) == [2 * 16 + 15, 4 * 16 + 0, 4 * 16 + 1]       # positions 15, 16, 17
    manager.commit(r)
    assert manager.length("a") == 33 and manager.length("b") == 33
    manager.check_invariants()


def test_abort_returns_pages_and_keeps_lengths():
    manager = CacheManager([FULL], page_size=4, num_pages=4, max_seqs=2)
    manager.admit("a")
    manager.commit(manager.prepare([("a", 5)]))
    before = manager.capacity()
    r = manager.prepare([("a", 6)])
    assert manager.capacity().free_pages == (1,)
    with pytest.raises(RuntimeError, match="neither committed nor aborted"):
        manager.prepare([("a", 1)])
    with pytest.raises(RuntimeError, match="open step"):
        manager.release("a")
    manager.abort(r)
    assert manager.capacity() == before and manager.length("a") == 5
    with pytest.raises(RuntimeError):
        manager.commit(r)
    manager.check_invariants()


def test_prepare_is_all_or_nothing():
    manager = CacheManager([FULL], page_size=4, num_pages=3, max_seqs=3)
    manager.admit("a"), manager.admit("b")
    with pytest.raises(OutOfPagesError):
        manager.prepare([("a", 8), ("b", 5)])
    assert manager.capacity().free_pages == (3,)
    manager.commit(manager.prepare([("a", 8), ("b", 4)]))
    with pytest.raises(ValueError, match="twice"):
        manager.prepare([("a", 1), ("a", 1)])
    manager.release("a"), manager.release("b")
    assert manager.capacity().free_pages == (3,) and manager.capacity().free_slots == 3
    with pytest.raises(KeyError):
        manager.release("a")


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    manager = CacheManager([FULL, window_group(6)], page_size=4, num_pages=10, max_seqs=2)
    manager.admit("a")
    manager.commit(manager.prepare([("a", 9)]))           # pages 0..2 in both groups
    entry = manager.requests["a"]
    # next query at position 9 sees keys 4..9 in the window group: page 0 (positions 0..3) is given back
    assert entry.tables[0] == [0, 1, 2] and entry.tables[1] == [RELEASED, 1, 2]
    assert manager.capacity().free_pages == (7, 8)
    manager.commit(manager.prepare([("a", 8)]))           # length 17: window keys 12..17 -> pages 0,1,2 gone
    assert entry.tables[1][:3] == [RELEASED] * 3 and entry.tables[1][3] == 0     # the freed page 0 is used again
    assert all(p != RELEASED for p in entry.tables[0])
    manager.check_invariants()
    manager.release("a")
    assert manager.capacity().free_pages == (10, 10)


def test_state_groups_disable_prefix_reuse_and_count_slots():
    manager = CacheManager([FULL, CacheGroup(StateNeed((4,)), 1)], page_size=4, num_pages=4, max_seqs=2,
                           enable_prefix_cache=True)
    assert manager.prefix is None and len(manager.allocators) == 1
    assert manager.group_index == [("paged", 0), ("state", 0)]
    assert CacheManager([window_group(8)], 4, 4, 2, enable_prefix_cache=True).prefix is None


def test_prefix_pages_are_shared_and_evicted_when_needed():
    manager = CacheManager([FULL], page_size=4, num_pages=6, max_seqs=3, enable_prefix_cache=True)
    prompt = list(range(100, 110))                        # 2 full pages + 2 tokens
    manager.admit("a")
    assert manager.attach_prefix("a", prompt) == 0
    manager.commit(manager.prepare([("a", 10)]))
    assert manager.cache_prefix("a", prompt) == 2
    manager.admit("b")
    assert manager.attach_prefix("b", prompt[:8] + [7, 7, 7]) == 8
    assert manager.requests["b"].tables == [[0, 1]] and manager.allocators[0].refcount(0) == 3
    manager.admit("c")
    assert manager.attach_prefix("c", prompt[:8]) == 4    # a full hit leaves the last page to compute
    manager.check_invariants()
    manager.release("a"), manager.release("b"), manager.release("c")
    snapshot = manager.capacity()
    assert snapshot.free_pages == (4,) and snapshot.reclaimable_pages == (2,)
    manager.admit("d")
    manager.commit(manager.prepare([("d", 21)]))          # needs all 6 pages: both cached pages are evicted
    assert manager.capacity().free_pages == (0,) and not manager.prefix.entries
    manager.check_invariants()


def test_prefix_in_use_is_not_evicted():
    manager = CacheManager([FULL], page_size=4, num_pages=4, max_seqs=3, enable_prefix_cache=True)
    prompt = list(range(9))
    manager.admit("a")
    manager.commit(manager.prepare([("a", 9)]))
    manager.cache_prefix("a", prompt)
    manager.admit("b")
    manager.attach_prefix("b", prompt)
    manager.release("a")                                  # page 2 free; pages 0, 1 held by b and the cache
    with pytest.raises(OutOfPagesError):
        manager.prepare([("b", 9)])                       # needs 3 pages, 2 are free, nothing reclaimable
    manager.check_invariants()


@pytest.mark.parametrize("seed", range(10))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    groups = [FULL, window_group(rng.choice((5, 9, 16)))] if seed % 2 else [FULL]
    manager = CacheManager(groups, page_size=rng.choice((1, 4, 16)), num_pages=24, max_seqs=5,
                           enable_prefix_cache=True, prefix_cache_max_entries=rng.choice((3, 8, 64)))
    live: dict[str, list[int]] = {}
    shared = [rng.randrange(50) for _ in range(40)]
    counter = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and manager.slots.free_count:
            rid = f"r{counter}"
            counter += 1
            manager.admit(rid)
            live[rid] = shared[:rng.randrange(0, 40)] + [rng.randrange(50) for _ in range(rng.randrange(1, 30))]
            manager.attach_prefix(rid, live[rid])
        elif action < 0.8 and live:
            chosen = rng.sample(sorted(live), rng.randrange(1, len(live) + 1))
            items = [(rid, rng.randrange(1, 12)) for rid in chosen]
            try:
                reservation = manager.prepare(items)
            except OutOfPagesError:
                manager.check_invariants()
                continue
            manager.check_invariants()
            if rng.random() < 0.2:
                manager.abort(reservation)
            else:
                manager.commit(reservation)
                for rid, _ in items:
                    if manager.length(rid) >= len(live[rid]):
                        manager.cache_prefix(rid, live[rid])
        elif live:
            rid = rng.choice(sorted(live))
            manager.release(rid)
            del live[rid]
        manager.check_invariants()
    for rid in list(live):
        manager.release(rid)
    manager.check_invariants()
    snapshot = manager.capacity()
    assert all(f + r == t for f, r, t in zip(snapshot.free_pages, snapshot.reclaimable_pages, snapshot.total_pages))
    assert snapshot.free_slots == 5


def _cache_prompt(manager, rid, prompt):
    manager.admit(rid)
    matched = manager.attach_prefix(rid, prompt)
    manager.commit(manager.prepare([(rid, len(prompt) - matched)]))
    added = manager.cache_prefix(rid, prompt)
    manager.check_invariants()
    return matched, added


def test_prefix_cache_at_its_limit_replaces_the_least_recently_used():
    """With ``prefix_cache_max_entries`` reached, a new prompt's pages take the place of the oldest ones that
    nobody holds (miniserve/kv/prefix_cache.py:122-125), and are then hit."""
    manager = CacheManager([FULL], page_size=4, num_pages=16, max_seqs=4, enable_prefix_cache=True,
                           prefix_cache_max_entries=3)
    first = list(range(100, 112)) + [1]                   # three full pages
    assert _cache_prompt(manager, "a", first) == (0, 3)
    manager.release("a")
    second = list(range(200, 208)) + [2]                  # two full pages: the first prompt's last two make room
    assert _cache_prompt(manager, "b", second) == (0, 2)
    manager.release("b")
    assert len(manager.prefix.entries) == 3
    manager.admit("c")
    assert manager.attach_prefix("c", second + [5]) == 8   # the new prompt is hit in full
    manager.admit("d")
    assert manager.attach_prefix("d", first) == 4          # of the old one the first page is left
    manager.check_invariants()
    manager.release("c"), manager.release("d")
    assert manager.capacity().free_pages == (13,) and manager.capacity().reclaimable_pages == (3,)


def test_prefix_cache_at_its_limit_never_replaces_an_entry_in_use():
    manager = CacheManager([FULL], page_size=4, num_pages=16, max_seqs=4, enable_prefix_cache=True,
                           prefix_cache_max_entries=2)
    first = list(range(100, 108)) + [1]
    assert _cache_prompt(manager, "a", first) == (0, 2)    # "a" stays live: both entries are in use
    held = [manager.prefix.entries[d].pages for d in manager.prefix.entries]
    second = list(range(200, 208)) + [2]
    assert _cache_prompt(manager, "b", second) == (0, 0)   # nothing can be replaced: the prompt stays uncached
    assert [manager.prefix.entries[d].pages for d in manager.prefix.entries] == held
    manager.release("a")
    third = list(range(300, 312)) + [3]                    # three pages into a cache of two: two are cached, and
    assert _cache_prompt(manager, "c", third) == (0, 2)    # the chain being inserted never replaces itself
    manager.admit("e")
    assert manager.attach_prefix("e", third) == 8
    manager.check_invariants()


def test_reclaimable_counts_only_what_eviction_can_free():
    """An entry that only the cache holds, standing before one that a request holds, is not reclaimable:
    eviction takes leaves first and the leaf is in use."""
    manager = CacheManager([FULL], page_size=4, num_pages=12, max_seqs=4, enable_prefix_cache=True)
    head = list(range(50, 54))
    manager.admit("b")                                     # admitted before anything is cached: no hit,
    assert manager.attach_prefix("b", head + [9, 9, 9, 9, 1]) == 0
    assert _cache_prompt(manager, "a", head + [3]) == (0, 1)
    manager.release("a")                                   # the cache alone holds the page of `head`
    manager.commit(manager.prepare([("b", 9)]))            # "b" computes its own copy of `head`
    assert manager.cache_prefix("b", head + [9, 9, 9, 9, 1]) == 1   # and caches its second page behind a's entry
    snapshot = manager.capacity()
    assert snapshot.reclaimable_pages == (0,) and manager.evictable_now() == 0
    with pytest.raises(OutOfPagesError):
        manager.prepare([("b", 4 * snapshot.free_pages[0] + 4)])
    manager.check_invariants()
    manager.release("b")
    assert manager.capacity().reclaimable_pages == (2,) and manager.evictable_now() == 2


def test_truncate_gives_back_the_pages_behind_the_new_end():
    manager = CacheManager([FULL], page_size=4, num_pages=8, max_seqs=2, enable_prefix_cache=True)
    prompt = list(range(13))
    manager.admit("a")
    manager.commit(manager.prepare([("a", 13)]))            # 4 pages
    manager.cache_prefix("a", prompt)                       # the cache holds the first 3 too
    with pytest.raises(RuntimeError, match="shares the page"):
        manager.truncate("a", 6)                            # page 1 is the cache's too: new tokens must not land in it
    manager.prefix.remove(next(e for e in manager.prefix.entries.values() if e.pages == (2,)))
    manager.allocators[0].release(2)                        # (the cache gives up its last two pages, leaves first)
    manager.prefix.remove(next(e for e in manager.prefix.entries.values() if e.pages == (1,)))
    manager.allocators[0].release(1)
    manager.truncate("a", 6)
    assert manager.length("a") == 6 and manager.requests["a"].tables == [[0, 1]]
    assert manager.capacity().free_pages == (6,)            # pages 2 and 3 are free
    manager.check_invariants()
    reservation = manager.prepare([("a", 3)])               # goes on from token 6, in page 1 and a new page
    assert list(reservation.items[0].slots[0]) == [6, 7, 8] and reservation.items[0].start == 6
    manager.commit(reservation)
    with pytest.raises(ValueError):
        manager.truncate("a", 10)
    reservation = manager.prepare([("a", 1)])
    with pytest.raises(RuntimeError):
        manager.truncate("a", 2)
    manager.abort(reservation)
    manager.truncate("a", 0)
    assert manager.requests["a"].tables == [[]]
    manager.check_invariants()
    windowed = CacheManager([window_group(8)], 4, 4, 2)
    windowed.admit("w")
    windowed.commit(windowed.prepare([("w", 3)]))
    with pytest.raises(RuntimeError):
        windowed.truncate("w", 1)
