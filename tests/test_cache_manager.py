"""The cache manager's books: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; prefixes are shared."""

from __future__ import annotations

import random

import pytest

from vllm_from_scratch_b200.cache import RELEASED, CacheError, CacheManager, PagePool, PagePoolError


def test_pool_take_share_give_back():
    pool = PagePool(4)
    pages = pool.take(3)
    assert sorted(pages) == [0, 1, 2] and pool.num_free == 1
    with pytest.raises(PagePoolError):
        pool.take(2)
    pool.give_back([pages[0]])
    with pytest.raises(PagePoolError, match="more often"):
        pool.give_back([pages[0]])
    pool.publish(pages[1], b"h1")
    pool.give_back([pages[1]])
    assert pool.lookup(b"h1") == pages[1]           # still hittable while free
    pool.share(pages[1])
    assert pool.ref_count[pages[1]] == 1 and pages[1] not in pool._free
    pool.give_back([pages[1]])
    # un-hashed pages are handed out before hashed ones
    first = pool.take(2)
    assert pages[1] not in first
    pool.take(1)
    assert pool.lookup(b"h1") is None               # handed out again: the hash is gone


def test_allocation_is_all_or_nothing_across_groups():
    manager = CacheManager([None, 8], page_size=4, num_pages=6, max_requests=2)
    manager.admit("a")
    assert manager.allocate("a", 16)                # 4 pages in both groups
    manager.admit("b")
    assert not manager.allocate("b", 12)            # 3 pages: only 2 free
    assert manager.block_table("b", 0) == [] and manager.block_table("b", 1) == []
    assert manager.num_free_pages(0) == 2 and manager.num_free_pages(1) == 2
    manager.check_invariants()
    with pytest.raises(CacheError):
        manager.admit("a")
    with pytest.raises(CacheError, match="slots"):
        manager.admit("c")
    manager.release("a")
    with pytest.raises(CacheError, match="released twice"):
        manager.release("a")
    assert manager.allocate("b", 12)
    manager.check_invariants()


def test_window_gives_pages_back_and_never_reads_them_again():
    manager = CacheManager([None, 10], page_size=4, num_pages=32, max_requests=1)
    manager.admit("w")
    computed = 0
    for portion in (7, 2, 30, 1, 1, 1, 9):
        assert manager.allocate("w", computed + portion)
        computed += portion
        manager.commit("w", computed)
        full, windowed = manager.block_table("w", 0), manager.block_table("w", 1)
        assert RELEASED not in full
        first_needed = max(0, computed - 10 + 1)
        for index, page in enumerate(windowed):
            wholly_before = (index + 1) * 4 <= first_needed
            assert (page == RELEASED) == wholly_before, (computed, index)
        manager.check_invariants()
    live = sum(page != RELEASED for page in manager.block_table("w", 1))
    assert live <= 10 // 4 + 2
    manager.release("w")
    assert manager.num_free_pages(0) == manager.num_free_pages(1) == 32


def test_prefix_sharing_cap_and_eviction():
    manager = CacheManager([None], page_size=4, num_pages=8, max_requests=3, enable_prefix_caching=True)
    tokens = list(range(100, 118))                  # 18 tokens: 4 full pages + 2
    manager.admit("a")
    assert manager.match_prefix("a", tokens) == 0
    assert manager.allocate("a", 18)
    manager.commit("a", 18, tokens)
    first = list(manager.block_table("a", 0))
    manager.admit("b")
    assert manager.match_prefix("b", tokens[:16]) == 12     # capped: one token must be computed
    assert manager.block_table("b", 0) == first[:3]
    manager.admit("c")
    assert manager.match_prefix("c", tokens[:9] + [7, 7, 7, 7]) == 8
    manager.check_invariants()
    manager.release("a")
    manager.release("b")
    manager.release("c")
    manager.check_invariants()
    # released pages keep their hashes until handed out again
    manager.admit("d")
    assert manager.match_prefix("d", tokens) == 16
    manager.release("d")
    manager.admit("e")
    assert manager.allocate("e", 32)                # takes every page: hashes are dropped
    manager.release("e")
    manager.admit("f")
    assert manager.match_prefix("f", tokens) == 0
    # windows or state switch sharing off
    assert not CacheManager([None, 4], 4, 8, 2, enable_prefix_caching=True).prefix_caching
    assert not CacheManager([None], 4, 8, 2, enable_prefix_caching=True, has_state=True).prefix_caching


def test_fresh_slots_are_reported_once():
    manager = CacheManager([None], page_size=4, num_pages=8, max_requests=2, has_state=True)
    slot = manager.admit("a")
    assert manager.take_fresh_slots() == [slot] and manager.take_fresh_slots() == []
    manager.allocate("a", 5)
    manager.drop_pages("a")                          # preempted: state starts again
    assert manager.take_fresh_slots() == [slot]
    manager.release("a")
    assert manager.admit("b") == slot


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books_straight(seed):
    rng = random.Random(seed)
    windows = [None, rng.choice([5, 9, 16])] if seed % 2 else [None]
    manager = CacheManager(windows, page_size=4, num_pages=24, max_requests=5,
                           enable_prefix_caching=seed % 2 == 0)
    live: dict[str, dict] = {}
    shared_prefix = [rng.randrange(50) for _ in range(12)]
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and manager.num_free_slots:
            counter += 1
            name = f"r{counter}"
            manager.admit(name)
            tokens = (shared_prefix if rng.random() < 0.5 else []) + [rng.randrange(50) for _ in range(rng.randrange(1, 30))]
            hit = manager.match_prefix(name, tokens)
            assert hit <= len(tokens) - 1 and hit % 4 == 0
            live[name] = {"tokens": tokens, "computed": hit}
        elif action < 0.75 and live:
            name = rng.choice(sorted(live))
            state = live[name]
            portion = rng.randrange(1, 12)
            while len(state["tokens"]) < state["computed"] + portion:
                state["tokens"].append(rng.randrange(50))
            before = [list(manager.block_table(name, g)) for g in range(len(windows))]
            if manager.allocate(name, state["computed"] + portion):
                state["computed"] += portion
                manager.commit(name, state["computed"], state["tokens"])
            else:
                assert before == [manager.block_table(name, g) for g in range(len(windows))]
        elif action < 0.85 and live:
            name = rng.choice(sorted(live))
            manager.drop_pages(name)
            live[name]["computed"] = 0
        elif live:
            name = rng.choice(sorted(live))
            manager.release(name)
            del live[name]
        manager.check_invariants()
    for name in list(live):
        manager.release(name)
    manager.check_invariants()
    assert all(pool.num_free == pool.num_pages for pool in manager.pools)
    assert manager.num_free_slots == 5
