"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""
import random

import pytest

from roost_b200.cache.block_pool import NULL_PAGE, BlockPool, PoolError
from roost_b200.cache.manager import CacheGroup, CacheManager, OutOfPages, build_groups, leading_releasable_pages
from roost_b200.parts.base import CacheNeed


def groups(page=4, window=10):
    return [CacheGroup("full", "paged", runs=(0, 2), page_size=page, kv_heads=1, head_dim=16),
            CacheGroup("win", "paged", runs=(1,), page_size=page, window=window, kv_heads=1, head_dim=16),
            CacheGroup("state", "state", runs=(3,), state_shape=(8,))]


def test_pool_hands_out_zero_first_and_reuses_the_last_freed():
    p = BlockPool(4)
    assert p.try_allocate(2) == [0, 1]
    assert p.try_allocate(3) is None and p.free_count == 2      # all or none
    p.release(0)
    assert p.try_allocate(1) == [0]                              # the page just given back is the next one taken
    with pytest.raises(PoolError, match="double release"):
        p.release(3)
    with pytest.raises(PoolError):
        p.release(7)
    p.check_invariants()
    p._refs[2] = 1                                               # a page that is neither free nor held by a table
    p._free.remove(2)
    p._refs[2] = 0
    with pytest.raises(PoolError, match="lost"):
        p.check_invariants()


def test_pages_are_taken_for_the_step_only_and_given_back_at_the_end():
    cm = CacheManager(groups(), [10, 10, 2])
    assert cm.pages_needed("a", 9) == [3, 3, 1]
    rc = cm.extend("a", 9)
    assert rc.tables[0] == [0, 1, 2] and rc.tables[1] == [0, 1, 2] and rc.slots[2] == 0
    cm.commit("a", 9)
    assert cm.pages_needed("a", 12) == [0, 0, 0] and cm.pages_needed("a", 13) == [1, 1, 0]
    with pytest.raises(ValueError):
        cm.extend("a", 5)
    cm.extend("b", 4)
    with pytest.raises(OutOfPages):
        cm.extend("c", 1)                                        # no state slot left
    assert "c" not in cm
    cm.check_invariants()
    cm.free("a")
    assert cm.extend("c", 8).tables[0] == [0, 1]                 # a's first pages, used again
    cm.free("a")                                                 # freeing twice is a no-op, not a double release
    cm.free_all()
    cm.check_invariants()
    assert [p.free_count for p in cm.pools] == [10, 10, 2]


def test_all_or_none_across_groups():
    cm = CacheManager(groups(), [10, 2, 2])
    with pytest.raises(OutOfPages):
        cm.extend("a", 12)                                       # the window group has 2 pages, 3 are needed
    assert "a" not in cm and cm.pools[0].free_count == 10 and cm.pools[2].free_count == 2


def test_window_pages_are_given_back_when_the_window_has_passed_them():
    assert [leading_releasable_pages(t, 10, 4) for t in (0, 10, 13, 14, 17, 18, 30)] == [0, 0, 0, 1, 1, 2, 5]
    cm = CacheManager(groups(page=4, window=10), [20, 5, 1])
    total = 0
    for step in (7, 5, 1, 1, 1, 9, 1, 1, 1, 1, 6, 1):
        total += step
        cm.extend("a", total)
        cm.commit("a", total)
        rc = cm.get("a")
        cut = leading_releasable_pages(total, 10, 4)
        assert all(p == NULL_PAGE for p in rc.tables[1][:cut]) and all(p != NULL_PAGE for p in rc.tables[1][cut:])
        assert NULL_PAGE not in rc.tables[0]
        # every key a later query can see is still held: positions >= total - window + 1
        first_needed = max(0, total - 10 + 1) // 4
        assert all(p != NULL_PAGE for p in rc.tables[1][first_needed:])
        cm.check_invariants()
    assert cm.held("a")[1] <= 10 // 4 + 2                        # the window group never holds much more than a window
    assert cm.pools[1].used_count == cm.held("a")[1]
    cm.free("a")
    assert cm.pools[1].free_count == 5


def test_random_orders_of_requests():
    rng = random.Random(0)
    cm = CacheManager(groups(page=4, window=10), [40, 16, 5])
    live = {}
    for it in range(3000):
        op = rng.random()
        if op < 0.5 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.choice([1, 1, 1, 2, 5, 17])
            try:
                cm.extend(rid, new)
                cm.commit(rid, new)
                live[rid] = new
            except OutOfPages:
                before = cm.held(rid)
                assert cm.get(rid).tokens == live[rid] and cm.held(rid) == before
        elif op < 0.75:
            rid = f"r{it}"
            n = rng.choice([1, 3, 8, 30])
            try:
                cm.extend(rid, n)
                cm.commit(rid, n)
                live[rid] = n
            except OutOfPages:
                assert rid not in cm
        elif live:
            rid = rng.choice(list(live))
            cm.free(rid)
            del live[rid]
        cm.check_invariants()
        assert set(cm.live_requests) == set(live)
    cm.free_all()
    assert all(p.free_count == p.capacity for p in cm.pools)


def test_groups_are_built_from_what_the_runs_need():
    full = CacheNeed("paged", kv_heads=2, head_dim=16)
    win = CacheNeed("paged", kv_heads=2, head_dim=16, window=24)
    other = CacheNeed("paged", kv_heads=1, head_dim=32)
    state = CacheNeed("state", state_shape=(4, 8))
    g = build_groups([full, win, None, full, other, state, win], page_size=8)
    assert [(x.kind, x.runs, x.window) for x in g] == [("paged", (0, 3), None), ("paged", (1, 6), 24), ("paged", (4,), None),
                                                        ("state", (5,), None)]
    g = build_groups([full, full], page_size=16)
    # the fixed-size state group is always there, empty for a model without such state, so slots are handed out on every path
    assert [(x.kind, x.runs, x.state_shape) for x in g] == [("paged", (0, 1), ()), ("state", (), (0,))]
    assert g[0].bytes_per_page(2) == 2 * 2 * 16 * 2 * 16 * 2
    # a run that keeps one tensor a token (a latent) gets a group of its own, half the bytes a page
    latent = CacheNeed("paged", kv_heads=2, head_dim=16, planes=1)
    g = build_groups([full, latent, latent], page_size=16)
    assert [(x.kind, x.runs, x.planes) for x in g[:2]] == [("paged", (0,), 2), ("paged", (1, 2), 1)]
    assert g[1].bytes_per_page(2) == 1 * 2 * 16 * 2 * 16 * 2
    with pytest.raises(ValueError):
        build_groups([CacheNeed("paged", kv_heads=2, head_dim=16, planes=3)], page_size=16)
