"""The native cache manager: no page is lost, held twice or freed twice, under random
orders of requests; pages come back and are used again; windows give pages back
early; state slots are booked the same way."""

import random

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from kv_cache_optimization_for_llm_b200.cache import host_runtime

H = host_runtime()


def make(pages=8, page_size=4, slots=3, window=0):
    return H.CacheManager([H.GroupSpec(page_size, window)], [pages], slots)


def test_pages_are_taken_and_returned_lifo():
    m = make()
    assert m.admit(10) == 0 and m.admit(11) == 1
    assert m.extend(10, 9)                      # 3 pages of 4 tokens
    assert m.block_table(10, 0) == [7, 6, 5]    # the list is popped from the back, as upstream's
    assert m.free_pages(0) == 5 and m.check() == ""
    assert m.extend(10, 9) and m.free_pages(0) == 5      # idempotent
    assert m.extend(11, 4) and m.block_table(11, 0) == [4]
    m.advance(10, 9)
    m.release(10)
    assert m.free_pages(0) == 7 and not m.has(10) and m.check() == ""
    # the pages just returned are the next ones handed out: immediate reuse
    assert m.admit(12) == 0
    assert m.extend(12, 8) and set(m.block_table(12, 0)) <= {7, 6, 5}


def test_extend_is_all_or_nothing():
    m = make(pages=4)
    m.admit(1)
    assert m.pages_needed(1, 17) == [5]
    assert not m.extend(1, 17)
    assert m.free_pages(0) == 4 and m.block_table(1, 0) == [] and m.check() == ""
    assert m.extend(1, 16) and m.free_pages(0) == 0


def test_slots_run_out_and_come_back():
    m = make(slots=2)
    assert m.admit(1) == 0 and m.admit(2) == 1 and m.admit(3) == -1
    assert not m.has(3) and m.free_slots() == 0
    m.release(1)
    assert m.admit(3) == 0 and m.check() == ""
    with pytest.raises(ValueError):
        m.admit(3)
    with pytest.raises(IndexError):
        m.extend(99, 4)


def test_double_release_is_an_error_not_a_double_free():
    m = make()
    m.admit(1)
    m.extend(1, 5)
    m.release(1)
    with pytest.raises(IndexError):
        m.release(1)
    assert m.free_pages(0) == 8 and m.check() == ""


def test_window_group_gives_pages_back_once_passed():
    m = make(pages=6, page_size=4, window=6)
    m.admit(1)
    assert m.extend(1, 10)                     # pages 0..2
    m.advance(1, 10)                           # next query at 10 reads keys > 4: page 0 (tokens 0-3) is passed
    assert m.block_table(1, 0)[0] == -1 and m.block_table(1, 0)[1] >= 0
    assert m.free_pages(0) == 4 and m.check() == ""
    # a long life in a small pool: a request far longer than the pool
    for n in range(11, 200):
        assert m.extend(1, n), n
        m.advance(1, n)
        assert m.check() == ""
    assert m.free_pages(0) >= 3
    # a portion of 12 tokens needs the window before it and all its own pages at once
    assert m.pages_needed(1, 211) == [3]
    m.release(1)
    assert m.free_pages(0) == 6


def test_two_groups_have_pools_of_their_own():
    m = H.CacheManager([H.GroupSpec(4, 0), H.GroupSpec(4, 4)], [8, 3], 2)
    m.admit(1)
    assert m.extend(1, 8)
    m.advance(1, 8)
    assert m.free_pages(0) == 6 and m.free_pages(1) == 2      # the window group kept one page
    assert not m.extend(1, 8 + 16)                             # group 1 cannot hold a 16-token portion
    assert m.free_pages(0) == 6 and m.free_pages(1) == 2 and m.check() == ""
    assert m.extend(1, 8 + 8)
    m.release(1)
    assert m.free_pages(0) == 8 and m.free_pages(1) == 3


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2**31), st.integers(4, 24), st.sampled_from([1, 4, 16]), st.integers(1, 5),
       st.sampled_from([0, 0, 5, 16]))
def test_random_orders_keep_the_books(seed, pages, page_size, slots, window):
    rng = random.Random(seed)
    m = make(pages, page_size, slots, window)
    live = {}
    next_id = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.25:
            slot = m.admit(next_id)
            assert (slot >= 0) == (len(live) < slots)
            if slot >= 0:
                live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.randint(1, 3 * page_size)
            free_before = m.free_pages(0)
            need = m.pages_needed(rid, new_len)[0]
            ok = m.extend(rid, new_len)
            assert ok == (need <= free_before)
            assert m.free_pages(0) == free_before - (need if ok else 0)
            if ok:
                m.advance(rid, new_len)
                live[rid] = new_len
                table = m.block_table(rid, 0)
                lo = max(0, new_len - window + 1) // page_size if window else 0
                assert all(p >= 0 for p in table[lo:]) and all(p < 0 for p in table[:lo])
        elif live:
            rid = rng.choice(list(live))
            (m.drop_pages if rng.random() < 0.3 else m.release)(rid)
            if m.has(rid):
                live[rid] = 0
            else:
                del live[rid]
        assert m.check() == ""
        held = sum(sum(p >= 0 for p in m.block_table(r, 0)) for r in live)
        assert held + m.free_pages(0) == pages
        assert m.free_slots() + len(live) == slots
    for rid in list(live):
        m.release(rid)
    assert m.free_pages(0) == pages and m.free_slots() == slots and m.check() == ""
