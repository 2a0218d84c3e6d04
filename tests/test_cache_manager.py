"""The host side of the cache: no page lost, held twice or freed twice, under random orders."""

import random

import numpy as np
import pytest

from cloud_inference_from_scratch_b200.cache import (
    NO_PAGE,
    CacheCapacityFull,
    CacheManager,
    DoubleFreeError,
    GroupSpec,
    PageAllocator,
)


def test_allocator_rounding_exhaustion_and_lifo_reuse():
    alloc = PageAllocator(4, 16)
    assert [alloc.pages_for(n) for n in (0, 1, 16, 17, 64)] == [0, 1, 1, 2, 4]
    first = alloc.allocate("a", 3)
    assert first == [0, 1, 2]
    with pytest.raises(CacheCapacityFull):
        alloc.allocate("b", 2)
    assert alloc.free_count == 1  # the failed call took nothing
    alloc.free([first[1]], "a")
    assert alloc.allocate("b", 1) == [first[1]]  # most recently freed page comes first
    alloc.assert_invariants()


def test_allocator_double_foreign_and_duplicate_free_change_nothing():
    alloc = PageAllocator(4, 4)
    pages = alloc.allocate("a", 2)
    other = alloc.allocate("b", 1)
    for bad, owner in ((pages + other, "a"), ([pages[0], pages[0]], "a"), ([3], "a")):
        with pytest.raises(DoubleFreeError):
            alloc.free(bad, owner)
        assert alloc.used_count == 3
        alloc.assert_invariants()
    alloc.free(pages, "a")
    with pytest.raises(DoubleFreeError):
        alloc.free(pages, "a")
    alloc.assert_invariants()


def make(pages=8, page=4, requests=4, tokens=64, groups=(GroupSpec("full"),)):
    return CacheManager(groups, page, pages, requests, tokens)


def test_growth_is_transactional_across_requests():
    cache = make(pages=5)
    cache.admit("a"), cache.admit("b")
    cache.ensure_capacity_batch({"a": 9, "b": 4})  # 3 + 1 pages
    assert cache.free_pages() == 1
    before = (cache.block_table("a"), cache.block_table("b"))
    with pytest.raises(CacheCapacityFull):
        cache.ensure_capacity_batch({"a": 12, "b": 9})  # needs 0 + 2 > 1
    assert (cache.block_table("a"), cache.block_table("b")) == before
    assert cache.free_pages() == 1
    cache.assert_invariants()
    cache.ensure_capacity_batch({"b": 8})
    assert cache.free_pages() == 0
    cache.commit_lengths({"a": 9, "b": 8})
    with pytest.raises(RuntimeError):
        cache.commit_lengths({"a": 13})
    assert cache.allocated_tokens("a") == 12
    cache.release("a")
    cache.release("a")  # idempotent
    assert cache.free_pages() == 3
    cache.assert_invariants()


def test_slots_host_tables_and_dirty_marks():
    cache = make(requests=2)
    slot_a = cache.admit("a")
    slot_b = cache.admit("b")
    assert {slot_a, slot_b} == {0, 1} and cache.take_dirty_slots() == [slot_a, slot_b]
    with pytest.raises(CacheCapacityFull):
        cache.admit("c")
    with pytest.raises(ValueError):
        cache.admit("a")
    cache.ensure_capacity_batch({"a": 6})
    rows = cache.table_rows(0, np.array([slot_a, slot_b]), 3)
    assert rows.shape == (2, 3) and list(rows[0][:2]) == cache.block_table("a")
    assert rows[0][2] == NO_PAGE and (rows[1] == NO_PAGE).all()
    cache.release("a")
    assert cache.admit("c") == slot_a and cache.take_dirty_slots() == [slot_a]
    assert (cache.table_rows(0, np.array([slot_a]), 3) == NO_PAGE).all()
    with pytest.raises(KeyError):
        cache.ensure_capacity_batch({"zz": 1})
    with pytest.raises(ValueError):
        cache.ensure_capacity_batch({"c": 65})
    cache.assert_invariants()


def test_window_group_gives_pages_back_as_the_window_passes():
    groups = (GroupSpec("full"), GroupSpec("window", window=6))
    cache = CacheManager(groups, 4, [16, 4], 2, 64)
    cache.admit("a")
    position = 0
    for step in (5, 3, 1, 1, 1, 7, 1, 1, 2):
        cache.ensure_capacity_batch({"a": (position, position + step)})
        position += step
        cache.commit_lengths({"a": position})
        cache.assert_invariants()
        table = cache.block_table("a", 1)
        # next query at `position` reads keys >= position - 5: every such page is present
        first_key = max(0, position - 6 + 1)
        for page_index in range(first_key // 4, -(-position // 4)):
            assert table[page_index] != NO_PAGE
        for page_index in range(first_key // 4):
            assert table[page_index] == NO_PAGE
        assert NO_PAGE not in cache.block_table("a", 0)
    assert cache.free_pages(1) >= 1  # 22 tokens passed through a pool of 4 pages
    cache.release("a")
    assert cache.free_pages(0) == 16 and cache.free_pages(1) == 4


def test_window_group_capacity_counts_only_live_pages():
    cache = CacheManager((GroupSpec("w", window=4),), 4, 3, 1, 400)
    cache.admit("a")
    position = 0
    for _ in range(90):  # 360 tokens through 3 pages, up to 4 at a time
        cache.ensure_capacity_batch({"a": (position, position + 4)})
        position += 4
        cache.commit_lengths({"a": position})
    cache.assert_invariants()
    with pytest.raises(CacheCapacityFull):
        cache.ensure_capacity_batch({"a": (position, position + 12)})


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = (GroupSpec("full"), GroupSpec("window", window=rng.choice([3, 8, 13])))
    cache = CacheManager(groups, rng.choice([2, 4, 8]), [rng.randint(6, 20), rng.randint(6, 12)], 4, 96)
    length: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and len(length) < 4:
            counter += 1
            name = f"r{counter}"
            cache.admit(name)
            length[name] = 0
        elif action < 0.35 and length:
            name = rng.choice(sorted(length))
            cache.release(name)
            del length[name]
        elif length:
            chosen = rng.sample(sorted(length), rng.randint(1, len(length)))
            spans = {}
            for name in chosen:
                grow = rng.choice([1, 1, 1, 2, 5, 9])
                if length[name] + grow <= 96:
                    spans[name] = (length[name], length[name] + grow)
            if not spans:
                continue
            free_before = [cache.free_pages(0), cache.free_pages(1)]
            try:
                cache.ensure_capacity_batch(spans)
            except CacheCapacityFull:
                assert [cache.free_pages(0), cache.free_pages(1)] == free_before
                victim = max(spans, key=lambda name: cache.allocated_tokens(name))
                cache.release(victim)
                del length[victim]
            else:
                for name, (_, end) in spans.items():
                    length[name] = end
                cache.commit_lengths({name: end for name, (_, end) in spans.items()})
        cache.assert_invariants()
    for name in list(length):
        cache.release(name)
    cache.assert_invariants()
    assert cache.free_pages(0) == cache.total_pages(0) and cache.free_pages(1) == cache.total_pages(1)
    assert cache.stats()["requests"] == 0


def test_page_counts_follow_what_a_group_can_use():
    """A windowed group never needs more than requests x (window + step tokens) of pages; under a byte
    budget what it does not need goes to the groups that keep everything."""
    from cloud_inference_from_scratch_b200.cache.manager import GroupSpec
    from cloud_inference_from_scratch_b200.cache.pools import plan_page_counts

    full = GroupSpec(name="full", window=0, bytes_per_token=1024)
    window = GroupSpec(name="window64", window=64, bytes_per_token=2048)
    # page count given: the windowed group is capped, the full one is not
    assert plan_page_counts([full, window], 16, max_requests=4, step_tokens=32, num_pages=1000) == [1000, 4 * 7]
    assert plan_page_counts([full, window], 16, max_requests=4, step_tokens=0, num_pages=1000) == [1000, 1000]
    assert plan_page_counts([full], 16, 4, 32, num_pages=77) == [77]
    assert plan_page_counts([], 16, 4, 32, num_pages=5) == [1]
    # bytes given: equal pages while both grow, then everything to the full group
    budget = 10 * 16 * (1024 + 2048)
    assert plan_page_counts([full, window], 16, 4, 32, kv_cache_bytes=budget) == [10, 10]
    budget = 28 * 16 * 2048 + 500 * 16 * 1024
    counts = plan_page_counts([full, window], 16, 4, 32, kv_cache_bytes=budget)
    assert counts == [500, 28]
    spent = sum(g.bytes_per_token * 16 * n for g, n in zip((full, window), counts))
    assert spent <= budget < spent + 16 * 1024
    only_windows = plan_page_counts([window], 16, 4, 32, kv_cache_bytes=1 << 40)
    assert only_windows == [28]
    with pytest.raises(ValueError):
        plan_page_counts([full], 16, 4, 32, kv_cache_bytes=100)
    with pytest.raises(ValueError):
        plan_page_counts([full], 16, 4, 32)
