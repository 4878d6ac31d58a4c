"""The cache manager: pages, block tables, windows, state slots (no GPU)."""
import random

import pytest

from vllm_oxide_b200.csrc.build import runtime_module

rt = runtime_module()


def full(pages, page=4, slots=4):
    return rt.CacheManager(page, [rt.GroupSpec(rt.FULL, 0, pages)], slots)


def test_slot_addressing_matches_the_reference_rule():
    # slot = table[pos / bs] * bs + pos % bs   (crates/engine/src/backend/paged.rs:48-52,221-228)
    c = full(16)
    c.admit(1)
    assert c.reserve(1, 10)
    table = c.block_table(1, 0)
    assert len(table) == 3 and len(set(table)) == 3
    for pos in range(10):
        assert c.slot_of(1, 0, pos) == table[pos // 4] * 4 + pos % 4
    with pytest.raises(rt.RuntimeFault, match="does not cover position 12"):     # paged.rs:57-80
        c.slot_of(1, 0, 12)


def test_pages_are_taken_at_page_edges_only():
    c = full(8)
    c.admit(7)
    assert c.reserve(7, 4) and len(c.block_table(7, 0)) == 1
    c.commit(7, 4)
    assert c.reserve(7, 1) and len(c.block_table(7, 0)) == 2      # position 4 opens a page
    c.commit(7, 1)
    for _ in range(3):
        assert c.reserve(7, 1)
        c.commit(7, 1)
    assert len(c.block_table(7, 0)) == 2 and c.length(7) == 8
    assert c.tokens_that_fit(7) == 6 * 4


def test_reserve_is_all_or_nothing_and_release_gives_everything_back():
    c = full(4)
    c.admit(1), c.admit(2)
    assert c.reserve(1, 9)             # 3 pages
    assert not c.reserve(2, 8)         # needs 2, one left: nothing is taken
    assert c.num_free_pages(0) == 1 and c.block_table(2, 0) == []
    assert c.reserve(2, 4)
    assert c.num_free_pages(0) == 0
    c.release(1)
    assert c.num_free_pages(0) == 3 and c.num_free_slots() == 3
    assert c.check_invariants() == ""
    with pytest.raises(rt.RuntimeFault):
        c.release(1)                   # freed twice
    with pytest.raises(rt.RuntimeFault):
        c.commit(2, 5)                 # more than was reserved


def test_freed_pages_are_used_again_at_once():
    c = full(6)
    c.admit(1)
    c.reserve(1, 8)
    mine = c.block_table(1, 0)
    c.release(1)
    c.admit(2)
    c.reserve(2, 8)
    assert set(c.block_table(2, 0)) == set(mine)      # last freed, first reused


def test_state_slots():
    c = full(8, slots=2)
    s1, s2 = c.admit(10), c.admit(11)
    assert {s1, s2} == {0, 1} and c.admit(12) == -1
    with pytest.raises(rt.RuntimeFault, match="already admitted"):
        c.admit(10)
    c.release(10)
    assert c.admit(12) == s1 and c.state_slot(12) == s1


def test_window_group_gives_back_passed_pages():
    page, window = 4, 6
    c = rt.CacheManager(page, [rt.GroupSpec(rt.FULL, 0, 32), rt.GroupSpec(rt.WINDOW, window, 32)], 2)
    c.admit(1)
    live_max = 0
    for step in range(40):
        n = [1, 3, 5, 2][step % 4]
        assert c.reserve(1, n)
        released = c.commit(1, n)
        L = c.length(1)
        t_full, t_win = c.block_table(1, 0), c.block_table(1, 1)
        assert all(p >= 0 for p in t_full) and len(t_full) == -(-L // page)
        first = max(0, L + 1 - window)            # first key the next query (position L) reads
        for i, p in enumerate(t_win):
            dead = (i + 1) * page <= first
            assert (p < 0) == dead, (L, i, t_win)
        assert all(g == 1 for g, _ in released)
        live_max = max(live_max, sum(p >= 0 for p in t_win))
        assert c.check_invariants() == ""
    assert live_max <= -(-(window + 5) // page) + 1     # bounded by the window plus the portion, not by the length
    c.release(1)
    assert c.num_free_pages(1) == 32 and c.num_free_pages(0) == 32


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    groups = [rt.GroupSpec(rt.FULL, 0, 24)]
    if seed % 2:
        groups.append(rt.GroupSpec(rt.WINDOW, 10, 12))
    c = rt.CacheManager(8, groups, 5)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and c.num_free_slots() > 0:
            assert c.admit(next_id) >= 0
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 20])
            fits = c.tokens_that_fit(rid) >= n
            before = [c.num_free_pages(g) for g in range(c.num_groups)]
            ok = c.reserve(rid, n)
            if len(groups) == 1:
                assert ok == fits
            if ok:
                c.commit(rid, n)
                live[rid] += n
                assert c.length(rid) == live[rid]
            else:
                assert before == [c.num_free_pages(g) for g in range(c.num_groups)]
        elif live:
            rid = rng.choice(list(live))
            c.release(rid)
            del live[rid]
        assert c.check_invariants() == "", c.check_invariants()
        held = sum(sum(p >= 0 for p in c.block_table(r, 0)) for r in live)
        assert held + c.num_free_pages(0) == 24
    for rid in list(live):
        c.release(rid)
    assert all(c.num_free_pages(g) == c.num_pages(g) for g in range(c.num_groups)) and c.num_free_slots() == 5


def test_bad_construction():
    with pytest.raises(rt.RuntimeFault):
        rt.CacheManager(0, [rt.GroupSpec(rt.FULL, 0, 4)], 1)
    with pytest.raises(rt.RuntimeFault):
        rt.CacheManager(4, [rt.GroupSpec(rt.WINDOW, 0, 4)], 1)
    with pytest.raises(rt.RuntimeFault):
        rt.CacheManager(4, [rt.GroupSpec(rt.FULL, 0, 0)], 1)
