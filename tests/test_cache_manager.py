"""Page pool and cache manager: no page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from einf_b200.cache import CacheManager, GroupSpec, PagePool


def test_pool_is_all_or_nothing_and_reuses_pages():
    pool = PagePool(4)
    assert pool.allocate(3) == [0, 1, 2]
    assert pool.allocate(2) is None and pool.free_count == 1  # no partial effect
    pool.release([1])
    assert pool.allocate(2) == [1, 3]  # the page freed last comes back first
    pool.release([0, 1, 2])
    assert pool.allocate(3) == [0, 1, 2]  # pages freed together come back in the order they were held
    assert pool.high_water == 4
    with pytest.raises(RuntimeError, match="named twice"):
        pool.release([0, 0])
    assert pool.is_held(0)  # the faulty call released nothing
    pool.release([0])
    with pytest.raises(RuntimeError, match="freed twice"):
        pool.release([0])
    with pytest.raises(RuntimeError, match="outside"):
        pool.release([9])
    with pytest.raises(ValueError):
        PagePool(0)


def test_reserve_grows_a_table_page_by_page():
    manager = CacheManager([GroupSpec(3, 4)])
    assert manager.reserve("a", 0, 4) and manager.block_table("a") == [0]
    assert manager.reserve("a", 4, 5) and manager.block_table("a") == [0, 1]  # growth at the page edge
    assert manager.reserve("a", 5, 8) and manager.block_table("a") == [0, 1]
    assert manager.pages_needed("a", 8, 13) == [2]
    assert not manager.reserve("a", 8, 13)  # 2 more pages, 1 free
    assert manager.block_table("a") == [0, 1] and manager.free_pages() == 1  # unchanged on failure
    assert manager.reserve("b", 0, 1) and manager.block_table("b") == [2]
    manager.release("a")
    assert manager.free_pages() == 2 and not manager.holds("a")
    # a's pages are used again, in the order a held them: a context reserved in one go is a run of pages
    assert manager.reserve("b", 1, 9) and manager.block_table("b") == [2, 0, 1]
    manager.check_invariants()
    manager.release("missing")  # unknown ids are ignored
    assert manager.capacity_tokens() == 12


def test_all_groups_or_none():
    manager = CacheManager([GroupSpec(8, 4), GroupSpec(2, 4)])
    assert manager.reserve("a", 0, 8)
    assert not manager.reserve("b", 0, 4)  # group 1 is full
    assert manager.free_pages(0) == 6 and not manager.holds("b")
    manager.check_invariants()


def test_window_gives_pages_back_as_it_passes():
    manager = CacheManager([GroupSpec(16, 4), GroupSpec(5, 4, window=6)])
    assert manager.reserve("a", 0, 10)
    assert manager.block_table("a", 1) == [0, 1, 2]
    assert manager.advance("a", 10) == 1  # next query at 10 sees keys 5..10: page 0 (keys 0..3) has passed
    assert manager.block_table("a", 1) == [-1, 1, 2] and manager.block_table("a", 0) == [0, 1, 2]
    assert manager.reserve("a", 10, 11) and manager.advance("a", 11) == 0
    assert manager.reserve("a", 11, 14) and manager.block_table("a", 1) == [-1, 1, 2, 0]  # page 0 again
    assert manager.advance("a", 14) == 1 and manager.block_table("a", 1) == [-1, -1, 2, 0]
    # a long decode never holds more than ceil(window / page) + 1 pages of the windowed group
    for length in range(14, 60):
        assert manager.reserve("a", length, length + 1)
        manager.advance("a", length + 1)
        assert manager.held_pages(1) <= 3
        manager.check_invariants()
    manager.release("a")
    assert manager.free_pages(1) == 5 and manager.free_pages(0) == 16


def test_window_needs_only_what_the_portion_sees():
    manager = CacheManager([GroupSpec(4, 4, window=4)])
    assert manager.reserve("a", 0, 12) is False or True  # 3 pages for 12 tokens of one portion
    manager.release("a")
    assert manager.reserve("a", 0, 8) and manager.advance("a", 8) == 1
    assert manager.pages_needed("a", 8, 16) == [2]
    assert manager.reserve("a", 8, 16)
    manager.check_invariants()


def test_state_slots_go_with_the_request():
    manager = CacheManager([GroupSpec(8, 4)], num_state_slots=2)
    assert manager.reserve("a", 0, 1) and manager.reserve("b", 0, 1)
    assert {manager.state_slot("a"), manager.state_slot("b")} == {0, 1}
    assert not manager.reserve("c", 0, 1) and manager.free_pages() == 6  # no slot: nothing is taken
    slot = manager.state_slot("a")
    manager.release("a")
    assert manager.reserve("c", 0, 1) and manager.state_slot("c") == slot
    assert manager.state_slot("nobody") == -1
    manager.check_invariants()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(24, 4), GroupSpec(12, 4, window=9)]
    manager = CacheManager(groups, num_state_slots=5)
    lengths: dict[str, int] = {}
    names = [f"r{i}" for i in range(8)]
    reused = False
    seen_pages: set[int] = set()
    for _ in range(600):
        name = rng.choice(names)
        action = rng.random()
        if name in lengths and action < 0.15:
            manager.release(name)
            del lengths[name]
        else:
            start = lengths.get(name, 0)
            portion = rng.choice([1, 1, 1, 2, 3, 7, 13])
            before = [manager.free_pages(g) for g in range(2)]
            held_before = manager.holds(name)
            if manager.reserve(name, start, start + portion):
                lengths[name] = start + portion
                table = manager.block_table(name, 0)
                assert len(table) == -(-lengths[name] // 4) and min(table) >= 0
                windowed = manager.block_table(name, 1)
                first_key = max(0, start - 9 + 1)
                assert min(windowed[first_key // 4:]) >= 0
                manager.advance(name, lengths[name])
                for page in table:
                    if page in seen_pages:
                        reused = True
                seen_pages.update(table)
            else:
                assert [manager.free_pages(g) for g in range(2)] == before
                assert manager.holds(name) == held_before
                victim = rng.choice(sorted(lengths)) if lengths else None
                if victim:
                    manager.release(victim)
                    del lengths[victim]
        manager.check_invariants()
        assert sorted(manager.holders()) == sorted(lengths)
    for name in list(lengths):
        manager.release(name)
    assert manager.free_pages(0) == 24 and manager.free_pages(1) == 12 and manager.free_state_slots == 5
    assert reused


def test_room_for_a_window_never_asks_for_more_pages_than_the_context_has():
    """A windowed group holds the window plus one portion, and a page more when the window straddles
    a page edge; but a context that fits one page needs one page, whatever the window."""
    manager = CacheManager([GroupSpec(1, 32), GroupSpec(1, 32, 11)], 0)
    assert manager.room_for(19, 5)                     # 19 tokens: one page of 32 in both groups
    assert not manager.room_for(33, 5)                 # two pages in the group that keeps all keys
    wide = CacheManager([GroupSpec(8, 32), GroupSpec(2, 4, 11)], 0)
    assert not wide.room_for(100, 5)                   # window 11 + portion 5 = 16 tokens: 4 pages of 4, + 1
    assert CacheManager([GroupSpec(8, 32), GroupSpec(5, 4, 11)], 0).room_for(100, 5)
