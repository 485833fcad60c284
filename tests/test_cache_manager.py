"""The cache manager on the host: no page lost, held twice or freed twice, under random orders
of requests; windows give pages back; slots are cleared and reused."""
from __future__ import annotations

import random

import pytest

from celeg_b200.cache import (NO_PAGE, CacheManager, OutOfPages, PageError, PagedNeed, PagePool, StateLayout)


def make(pages=(8,), windows=(None,), page_tokens=4, slots=3, cleared=None):
    groups = [(("g", i, w), PagedNeed(kv_heads=1, head_dim=8, window=w)) for i, w in enumerate(windows)]
    layout = StateLayout()
    layout.add(0, 10)
    layout.add(3, 7)
    return CacheManager(page_tokens, list(pages), groups, layout, slots,
                        clear_slot=(cleared.append if cleared is not None else None))


def test_pool_allocation_is_all_or_nothing_and_lifo():
    pool = PagePool(4, 16)
    assert pool.allocate(5) is None and pool.free_pages == 4
    first = pool.allocate(3)
    assert first == [0, 1, 2]
    pool.release([1])
    assert pool.allocate(1) == [1]                      # the page just given back is used again first
    assert pool.allocate_tokens(17) is None             # needs 2, one free
    assert pool.pages_for(16) == 1 and pool.pages_for(17) == 2


def test_pool_refuses_double_free_and_bad_ids():
    pool = PagePool(3, 4)
    pages = pool.allocate(2)
    pool.release(pages)
    with pytest.raises(PageError):
        pool.release(pages)
    with pytest.raises(PageError):
        pool.release([7])
    with pytest.raises(PageError):
        pool.retain([0])
    held = pool.allocate(1)
    pool.retain(held)
    assert pool.ref_count(held[0]) == 2
    with pytest.raises(PageError):
        pool.release([held[0]] * 3)                     # validated before anything changes
    assert pool.ref_count(held[0]) == 2
    pool.release(held)
    pool.release(held)
    assert pool.free_pages == 3


def test_state_layout_is_aligned():
    layout = StateLayout()
    assert layout.add(0, 10) == 0 and layout.add(1, 7) == 12 and layout.slot_elements == 20


def test_open_reserve_advance_close():
    cleared = []
    manager = make(cleared=cleared)
    a = manager.open("a")
    assert cleared == [a.slot]
    manager.reserve(a, 9)                               # 3 pages of 4 tokens
    assert len(a.tables[0]) == 3 and manager.groups[0].pool.free_pages == 5
    manager.reserve(a, 9)                               # nothing more needed
    assert len(a.tables[0]) == 3
    with pytest.raises(PageError):
        manager.advance(a, 13)                          # beyond what was reserved
    manager.advance(a, 9)
    with pytest.raises(ValueError):
        manager.advance(a, 8)
    manager.check_invariants()
    manager.close("a")
    assert manager.groups[0].pool.free_pages == 8 and manager.free_slots == 3
    with pytest.raises(PageError):
        manager.close("a")
    with pytest.raises(PageError):
        manager.reserve(a, 4)


def test_reserve_across_groups_is_all_or_nothing():
    manager = make(pages=(8, 2), windows=(None, None))
    a = manager.open("a")
    with pytest.raises(OutOfPages):
        manager.reserve(a, 12)                          # 3 pages: group 1 has only 2
    assert manager.groups[0].pool.free_pages == 8 and a.tables == [[], []]
    manager.reserve(a, 8)
    assert [len(t) for t in a.tables] == [2, 2]


def test_no_slot_no_request():
    manager = make(slots=1)
    manager.open("a")
    assert not manager.can_hold(1)
    with pytest.raises(OutOfPages):
        manager.open("b")
    with pytest.raises(ValueError):
        manager.open("a")


def test_window_gives_pages_back_as_it_passes():
    manager = make(pages=(8, 8), windows=(None, 6))
    a = manager.open("a")
    total = 0
    for step in (5, 4, 3, 7, 1, 1, 1):
        manager.reserve(a, total + step)
        total += step
        released = manager.advance(a, total)
        manager.check_invariants()
        # the next query sits at `total` and reads positions > total - 6
        first_needed = max(0, total - 6 + 1)
        table = a.tables[1]
        for logical, page in enumerate(table):
            if (logical + 1) * 4 <= first_needed:
                assert page == NO_PAGE
            else:
                assert page != NO_PAGE
        assert all(group == 1 for group, _ in released)
        assert NO_PAGE not in a.tables[0]
    assert manager.groups[1].pool.used_pages <= 3       # ceil((6-1)/4)+1 pages in steady state
    manager.close("a")
    assert manager.groups[1].pool.free_pages == 8


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_keeps_the_books(seed):
    rng = random.Random(seed)
    cleared = []
    manager = make(pages=(12, 9), windows=(None, 10), page_tokens=4, slots=4, cleared=cleared)
    live, lengths, serial = {}, {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and manager.free_slots:
            name = f"r{serial}"
            serial += 1
            live[name] = manager.open(name)
            lengths[name] = 0
        elif action < 0.85 and live:
            name = rng.choice(sorted(live))
            grow = rng.randint(1, 9)
            before = [list(t) for t in live[name].tables]
            try:
                manager.reserve(live[name], lengths[name] + grow)
            except OutOfPages:
                assert [list(t) for t in live[name].tables] == before
            else:
                lengths[name] += grow
                manager.advance(live[name], lengths[name])
        elif live:
            name = rng.choice(sorted(live))
            manager.close(name)
            del live[name], lengths[name]
        manager.check_invariants()
        for name, cache in live.items():
            assert cache.tokens == lengths[name]
    for name in list(live):
        manager.close(name)
    manager.check_invariants()
    assert all(group.pool.free_pages == group.pool.total_pages for group in manager.groups)
    assert manager.free_slots == 4 and len(cleared) == serial


@pytest.mark.parametrize("seed,windows", [(0, (None,)), (1, (None, 10)), (2, (None,)), (3, (None, 6))])
def test_batched_calls_and_table_mirrors_agree_with_the_single_ones(seed, windows):
    """Steps of many requests: pages_needed_each / reserve_each / advance_each against the calls for one request
    on a twin manager, under random traffic; and the table mirrors (one int32 row per slot and group) hold
    every live request's table, with NO_PAGE everywhere else, whatever was opened, grown and closed."""
    import numpy as np
    rng = random.Random(seed)
    pages = tuple(80 for _ in windows)
    groups = [(("g", i, w), PagedNeed(kv_heads=1, head_dim=8, window=w)) for i, w in enumerate(windows)]
    batched = CacheManager(4, list(pages), groups, StateLayout(), 5, table_capacity=16)
    single = CacheManager(4, list(pages), groups, StateLayout(), 5)
    live, serial = [], 0
    for _ in range(300):
        action = rng.random()
        if action < 0.2 and batched.free_slots:
            name = f"r{serial}"
            serial += 1
            batched.open(name)
            single.open(name)
            live.append(name)
        elif action < 0.9 and live:
            chosen = rng.sample(live, rng.randint(1, len(live)))
            counts = [rng.choice((1, 1, 1, 2, 5, 9)) for _ in chosen]
            kept = [(n, c) for n, c in zip(chosen, counts) if batched.get(n).tokens + c <= 60]
            chosen, counts = [n for n, _ in kept], [c for _, c in kept]
            caches = [batched.get(n) for n in chosen]
            need = batched.pages_needed_each(caches, counts)
            want = [0] * len(windows)
            for n, c in zip(chosen, counts):
                twin = single.get(n)
                for g, pages_g in enumerate(single.pages_needed(twin, twin.tokens + c)):
                    want[g] += pages_g
            assert need == want
            batched.reserve_each(caches, counts)
            batched.advance_each(caches, counts)
            for n, c in zip(chosen, counts):
                twin = single.get(n)
                single.reserve(twin, twin.tokens + c)
                single.advance(twin, twin.tokens + c)
        elif live:
            name = live.pop(rng.randrange(len(live)))
            batched.close(name)
            single.close(name)
        batched.check_invariants()
        assert [g.pool.free_pages for g in batched.groups] == [g.pool.free_pages for g in single.groups]
        for name in live:
            a, b = batched.get(name), single.get(name)
            # (the page numbers may differ: the twin gives pages back between two requests of a step, the
            # batched calls after all of them; which places of a table hold a page must not)
            assert a.tokens == b.tokens and a.first_live_page == b.first_live_page
            assert [[p == NO_PAGE for p in t] for t in a.tables] == [[p == NO_PAGE for p in t] for t in b.tables]
            assert a.capacity == min(len(t) for t in a.tables) * 4
        for g, mirror in enumerate(batched.table_mirrors):
            expect = np.full_like(mirror, NO_PAGE)
            for name in live:
                cache = batched.get(name)
                expect[cache.slot, :len(cache.tables[g])] = cache.tables[g]
            assert np.array_equal(mirror, expect)
    for name in live:
        batched.close(name)
    assert all(np.all(mirror == NO_PAGE) for mirror in batched.table_mirrors)
    assert all(group.pool.free_pages == group.pool.total_pages for group in batched.groups)


def test_values_may_be_narrower_than_keys_or_absent():
    """A paged need states the width of what is kept beside the keys on its own: equal (attention), narrower,
    or nothing (one latent vector per position). Needs that differ in it form groups of their own."""
    import torch
    from celeg_b200.cache.storage import CacheStorage
    needs = [PagedNeed(2, 16), PagedNeed(2, 16, value_head_dim=8), PagedNeed(1, 48, value_head_dim=0)]
    assert len({need.group_key() for need in needs}) == 3
    assert [need.value_dim for need in needs] == [16, 8, 0]
    storage = CacheStorage([(need, 2) for need in needs], [5, 5, 5], 4, StateLayout(), 3, torch.float32,
                           torch.device("cpu"))
    assert [tuple(k.shape) for k in storage.k] == [(2, 37, 2, 4, 16), (2, 37, 2, 4, 16), (2, 37, 1, 4, 48)]
    assert [tuple(v.shape) for v in storage.v] == [(2, 37, 2, 4, 16), (2, 37, 2, 4, 8), (2, 37, 1, 4, 0)]
    assert storage.scratch_pages == [5, 5, 5] and storage.scratch_page_count == 32
    assert storage.scratch_slot == 3 and storage.state.shape[0] == 4
