"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; slots; rollback."""

import random

import pytest

from quantinfer_b200.cache import CacheManager, PageAllocator, PagedKVNeed, StateNeed
from quantinfer_b200.errors import CacheError, OutOfPages


def _mgr(num_pages=16, page_size=4, window=None, max_requests=4, max_seq_len=64):
    needs = [PagedKVNeed(2, 8), PagedKVNeed(2, 8)]
    if window:
        needs.append(PagedKVNeed(2, 8, window))
    needs.append(StateNeed((3,)))
    return CacheManager(needs, page_size, num_pages, max_requests, max_seq_len, device=None)


def test_allocator_rejects_double_free():
    a = PageAllocator(3)
    p = a.alloc()
    a.free(p)
    with pytest.raises(CacheError):
        a.free(p)
    with pytest.raises(CacheError):
        a.free(99)
    got = [a.alloc() for _ in range(3)]
    assert sorted(got) == [0, 1, 2]
    with pytest.raises(OutOfPages):
        a.alloc()


def test_groups_share_by_need():
    m = _mgr(window=6)
    assert len(m.groups) == 2                       # two full-attention entries share a group
    assert m.groups[0].entries == [0, 1] and m.groups[1].entries == [2]
    assert m.view(1).group == 0 and m.view(2).group == 1 and m.view(3).group == -1


def test_pages_follow_length_and_are_reused():
    m = _mgr()
    m.open("a")
    m.prepare("a", 5)
    assert len(m.table_row("a", 0)) == 2 and m.free_pages() == 14
    m.commit("a")
    m.prepare("a", 3)            # 8 positions: still 2 pages
    m.commit("a")
    assert len(m.table_row("a", 0)) == 2
    m.prepare("a", 1)
    m.commit("a")
    assert len(m.table_row("a", 0)) == 3
    pages = list(m.table_row("a", 0))
    m.close("a")
    assert m.free_pages() == 16
    m.open("b")
    m.prepare("b", 12)
    assert set(m.table_row("b", 0)) == set(pages)   # last freed, first reused
    m.check_invariants()


def test_prepare_is_all_or_nothing():
    m = _mgr(num_pages=4, window=6)
    m.open("a")
    m.prepare("a", 12)          # 3 pages in both groups
    m.commit("a")
    m.open("b")
    free = [m.free_pages(g) for g in range(2)]
    with pytest.raises(OutOfPages):
        m.prepare("b", 8)       # needs 2 pages, group 0 has 1
    assert [m.free_pages(g) for g in range(2)] == free and m.get("b").pending == 0
    m.check_invariants()


def test_rollback_gives_back_what_the_step_took():
    m = _mgr()
    m.open("a")
    m.prepare("a", 6)
    m.commit("a")
    before = m.free_pages()
    m.prepare("a", 9)
    assert m.free_pages() < before
    m.rollback("a")
    assert m.free_pages() == before and m.get("a").length == 6
    m.check_invariants()


def test_window_pages_go_back_once_passed():
    m = _mgr(num_pages=32, page_size=4, window=6)
    m.open("a")
    m.prepare("a", 20)
    m.commit("a")
    full, win = m.table_row("a", 0), m.table_row("a", 1)
    assert all(p >= 0 for p in full) and len(full) == 5
    # next query at position 20 reads keys 15..20: blocks 0..2 (positions 0..11) are passed
    assert [p >= 0 for p in win] == [False, False, False, True, True]
    assert m.free_pages(1) == 32 - 2
    m.prepare("a", 1)
    m.commit("a")          # position 21 -> keys 16..: block 3 (12..15) is passed too
    assert [p >= 0 for p in m.table_row("a", 1)] == [False, False, False, False, True, True]
    m.check_invariants()
    m.close("a")
    assert m.free_pages(1) == 32


def test_slots_and_limits():
    m = _mgr(max_requests=2)
    a, b = m.open("a"), m.open("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(CacheError, match="slots"):
        m.open("c")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    m.close("a")
    assert m.open("c").slot == a.slot
    with pytest.raises(CacheError, match="not open"):
        m.prepare("zzz", 1)
    with pytest.raises(CacheError, match="limit"):
        m.prepare("b", 65)
    m.prepare("b", 2)
    with pytest.raises(CacheError, match="uncommitted"):
        m.prepare("b", 2)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books_straight(seed):
    rng = random.Random(seed)
    m = _mgr(num_pages=24, page_size=4, window=10 if seed % 2 else None, max_requests=5, max_seq_len=60)
    live, next_id = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            m.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.randint(1, 9)
            if live[rid] + n > 60:
                continue
            try:
                m.prepare(rid, n)
            except OutOfPages:
                m.check_invariants()
                continue
            if rng.random() < 0.15:
                m.rollback(rid)
            else:
                m.commit(rid)
                live[rid] += n
            assert m.get(rid).length == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.close(rid)
    m.check_invariants()
    assert all(m.free_pages(g) == 24 for g in range(len(m.groups)))
