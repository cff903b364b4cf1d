"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed
twice, under random orders of requests; windows give pages back; slots."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from easy_gpt.cpp_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool
from easy_gpt.cpp_b200.parts.base import PagedKVNeed, StateNeed

FULL = PagedKVNeed(2, 16, None)
WIN = PagedKVNeed(2, 16, 10)


def manager(num_pages=16, page_size=4, slots=4, needs=None, per_request=64):
    needs = needs if needs is not None else {0: FULL, 1: FULL, 2: WIN, 3: StateNeed((3,)), 4: None}
    return CacheManager(needs, page_size, num_pages, slots, per_request)


def test_pool_is_lifo_and_catches_double_free():
    p = PagePool(4)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.free_count == 1
    p.free([1])
    assert p.alloc(1) == [1]                         # a page given back is the next one handed out
    with pytest.raises(OutOfPages):
        p.alloc(2)
    assert p.free_count == 1                         # nothing changed
    p.free([0, 2])
    with pytest.raises(ValueError, match="freed twice"):
        p.free([2])
    with pytest.raises(ValueError, match="not of this pool"):
        p.free([9])
    p.check()


def test_groups_are_formed_by_need():
    m = manager()
    assert len(m.groups) == 2
    assert m.groups[0].cache_ids == [0, 1] and m.groups[0].window is None
    assert m.groups[1].cache_ids == [2] and m.groups[1].window == 10
    assert m.view(1).group == 0 and m.view(2).group == 1 and m.view(4).group == -1


def test_reserve_commit_end():
    m = manager()
    slot = m.begin_request("a")
    assert slot == 0 and m.slot_of("a") == 0
    m.reserve("a", 9)                                # 3 pages in each group
    assert m.free_pages(0) == 13 and m.free_pages(1) == 13
    m.reserve("a", 9)                                # idempotent while nothing is committed
    assert m.free_pages(0) == 13
    assert m.slot_positions(0, "a", 0, 9).tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 8]
    m.commit("a", 9)
    with pytest.raises(ValueError, match="exceeds what was reserved"):
        m.commit("a", 4)
    m.begin_request("b")
    m.reserve("b", 4)
    assert m.slot_positions(0, "b", 0, 4).tolist() == [12, 13, 14, 15]     # page 3
    m.check()
    m.end_request("a")
    assert m.free_pages(0) == 15
    m.begin_request("c")
    m.reserve("c", 1)
    assert m.table_rows(0, ["c"], 1).tolist() == [[0]]                   # a's first page is used again
    assert m.slot_of("c") == 0                                          # and its slot
    m.check()


def test_out_of_pages_changes_nothing():
    m = manager(num_pages=4)
    m.begin_request("a")
    m.reserve("a", 12)
    m.commit("a", 12)
    m.begin_request("b")
    before = (m.free_pages(0), m.free_pages(1))
    assert not m.can_reserve("b", 8)
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert (m.free_pages(0), m.free_pages(1)) == before
    m.check()
    mm = manager(num_pages=64, per_request=16)
    mm.begin_request("x")
    with pytest.raises(OutOfPages, match="at most"):
        mm.reserve("x", 17)


def test_window_gives_pages_back_exactly_when_they_are_out_of_sight():
    m = manager(num_pages=32)
    m.begin_request("a")
    held = []
    for pos in range(40):
        m.reserve("a", 1)
        m.commit("a", 1)
        row = m.groups[1].tables[m.slot_of("a")]
        live = [i for i in range(len(row)) if row[i] >= 0]
        held.append(len(live))
        # the next token sits at position pos+1 and sees keys pos+1-9 .. pos+1
        first_key = max(0, pos + 1 - 10 + 1)
        assert live[0] == first_key // 4, (pos, live)
        assert m.groups[0].tables[m.slot_of("a")][0] >= 0              # the full group keeps everything
    assert max(held) <= 4                                              # ceil(10/4) + 1
    m.check()
    m.end_request("a")
    assert m.free_pages(0) == 32 and m.free_pages(1) == 32


def test_slots_and_state():
    m = manager(slots=2)
    m.begin_request("a")
    m.begin_request("b")
    with pytest.raises(OutOfSlots):
        m.begin_request("c")
    with pytest.raises(KeyError):
        m.begin_request("a")
    m.end_request("a")
    assert m.begin_request("c") == 0
    assert m.free_slot_count() == 0


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 5), st.integers(1, 23), st.booleans()), min_size=1, max_size=120),
       st.integers(2, 7), st.integers(6, 40))
def test_random_orders_keep_the_books_straight(ops, page_size, num_pages):
    m = manager(num_pages=num_pages, page_size=page_size, slots=4, per_request=10_000)
    lengths = {}
    for rid, n, end in ops:
        if rid not in lengths:
            if m.free_slot_count() == 0:
                continue
            m.begin_request(rid)
            lengths[rid] = 0
        if m.can_reserve(rid, n):
            m.reserve(rid, n)
            phys = m.slot_positions(0, rid, lengths[rid], n)
            assert len(set(phys.tolist())) == n
            m.commit(rid, n)
            lengths[rid] += n
            assert m.length_of(rid) == lengths[rid]
        else:
            free = (m.free_pages(0), m.free_pages(1))
            with pytest.raises(OutOfPages):
                m.reserve(rid, n)
            assert free == (m.free_pages(0), m.free_pages(1))
        if end:
            m.end_request(rid)
            del lengths[rid]
        m.check()
        # the full group holds exactly ceil(len / page) pages per request
        for r, length in lengths.items():
            row = m.groups[0].tables[m.slot_of(r)]
            assert (row >= 0).sum() == -(-length // page_size)
    m.reset()
    m.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in m.groups)


def test_pool_free_is_all_or_nothing():
    p = PagePool(6)
    p.alloc(4)
    with pytest.raises(ValueError, match="freed twice"):
        p.free([0, 1, 1])                            # a page named twice in one call
    with pytest.raises(ValueError, match="freed twice"):
        p.free([2, 5])                               # page 5 is not held
    assert p.free_count == 2 and p.used_count == 4   # neither call gave anything back
    p.check()
    p.free([3, 0])
    assert p.alloc(2) == [3, 0] and p.total_allocated == 6 and p.high_water == 4      # the first of a batch comes out first


def test_requests_are_known_by_any_hashable_name():
    m = manager(slots=3)
    m.begin_request("a")
    m.begin_request(7)
    m.begin_request(("t", 1))
    assert sorted(map(str, m.live_requests())) == ["('t', 1)", "7", "a"]
    assert not m.has_request("b") and not m.has_request(8)
    with pytest.raises(KeyError):
        m.length_of("b")
    m.end_request(("t", 1))
    with pytest.raises(KeyError):
        m.end_request(("t", 1))
    assert set(m.live_requests()) == {7, "a"}
    m.check()
