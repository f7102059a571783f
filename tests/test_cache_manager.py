"""The host cache manager: no page is lost, held twice or freed twice, under random orders of requests;
allocation is all-or-nothing; freed pages are the next ones handed out; windows give pages back."""
import random

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from vllm_cpp_b200.runtime import runtime


def manager(groups, slots=4):
    rt = runtime()
    return rt, rt.CacheManager([rt.GroupSpec(ps, n, w) for ps, n, w in groups], slots)


def test_id_pool_rejects_double_and_foreign_frees():
    rt = runtime()
    p = rt.IdPool(3)
    assert p.alloc(2) == [0, 1] and p.alloc(2) is None and p.free_count() == 1       # all or nothing
    p.free(0)
    with pytest.raises(RuntimeError, match="twice"):
        p.free(0)
    with pytest.raises(RuntimeError, match="outside"):
        p.free(7)
    assert p.alloc(1) == [0]                                                        # last freed, first reused


def test_reserve_is_all_or_nothing_across_groups():
    rt, m = manager([(4, 10, 0), (4, 3, 0)])
    assert m.open(1) == 0
    assert m.reserve(1, 12)                      # 3 pages in each group
    assert m.open(2) == 1
    assert not m.reserve(2, 4)                   # group 1 is empty: nothing may be taken from group 0 either
    assert m.free_pages(0) == 7 and m.block_table(2, 0) == [] and m.reserved_tokens(2) == 0
    m.check_invariants()
    m.close(1)
    assert m.reserve(2, 4) and m.free_pages(0) == 9 and m.free_pages(1) == 2
    m.check_invariants()


def test_freed_pages_are_reused_first():
    rt, m = manager([(4, 8, 0)])
    m.open(1); m.reserve(1, 16)
    first = list(m.block_table(1, 0))
    m.close(1)
    m.open(2); m.reserve(2, 8)
    assert set(m.block_table(2, 0)) <= set(first) and m.block_table(2, 0)[0] == first[-1]


def test_window_group_gives_pages_back_as_the_window_passes():
    rt, m = manager([(4, 100, 0), (4, 100, 10)])          # group 1: position p reads keys (p - 10, p]
    m.open(1)
    assert m.reserve(1, 30)
    m.commit(1, 30)                                       # next query at 30 reads keys >= 21: blocks 0..4 are dead
    assert m.block_table(1, 1)[:6] == [-1, -1, -1, -1, -1, m.block_table(1, 1)[5]]
    assert m.block_table(1, 0).count(-1) == 0 and m.free_pages(1) == 100 - 3
    assert m.reserve(1, 31); m.commit(1, 31)
    assert m.reserve(1, 33); m.commit(1, 33)              # keys >= 24: block 5 (20..23) is dead now
    assert m.block_table(1, 1)[5] == -1 and len(m.block_table(1, 1)) == 9
    m.check_invariants()
    assert m.peak_pages(1, 1000, 16) == (10 + 16 + 3) // 4 + 1 and m.peak_pages(0, 1000, 16) == 250
    m.close(1)
    assert m.free_pages(0) == 100 and m.free_pages(1) == 100 and m.free_slots() == 4


def test_slots_and_misuse():
    rt, m = manager([(4, 8, 0)], slots=2)
    assert m.open(10) == 0 and m.open(11) == 1 and m.open(12) == -1
    with pytest.raises(RuntimeError, match="already open"):
        m.open(10)
    with pytest.raises(RuntimeError, match="not open"):
        m.reserve(99, 4)
    m.reserve(10, 8)
    with pytest.raises(RuntimeError, match="beyond the reserved"):
        m.commit(10, 9)
    m.commit(10, 8)
    with pytest.raises(RuntimeError, match="below the committed"):
        m.commit(10, 4)
    m.close(10)
    with pytest.raises(RuntimeError, match="not open"):
        m.close(10)
    assert m.open(13) == 0                                  # the slot is handed out again


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(seed=st.integers(0, 10 ** 6), page=st.sampled_from([1, 4, 16]), window=st.sampled_from([0, 5, 24]),
       pages=st.integers(4, 40))
def test_random_orders_keep_the_books(seed, page, window, pages):
    """Random opens, growths, commits and closes against a model kept in Python."""
    rt, m = manager([(page, pages, 0), (page, pages, window)], slots=5)
    rng = random.Random(seed)
    live = {}            # id -> (reserved, committed)
    next_id = 0
    for _ in range(200):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            assert m.open(next_id) >= 0
            live[next_id] = (0, 0)
            next_id += 1
        elif op < 0.7 and live:
            rid = rng.choice(list(live))
            res, com = live[rid]
            want = res + rng.randint(1, 3 * page)
            free_before = [m.free_pages(0), m.free_pages(1)]
            need = [m.pages_missing(rid, g, want) for g in range(2)]
            ok = m.reserve(rid, want)
            assert ok == all(n <= f for n, f in zip(need, free_before))
            if ok:
                assert [m.free_pages(g) for g in range(2)] == [f - n for f, n in zip(free_before, need)]
                live[rid] = (want, com)
            else:
                assert [m.free_pages(0), m.free_pages(1)] == free_before
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            res, com = live[rid]
            if res > com:
                new = rng.randint(com, res)
                m.commit(rid, new)
                live[rid] = (res, new)
                tab = m.block_table(rid, 1)
                first_needed = max(0, new - window + 1) if window else 0
                for b, pg in enumerate(tab):               # a page is gone exactly when no later query can read it
                    dead = window > 0 and (b + 1) * page <= first_needed
                    assert (pg == -1) == dead or (pg == -1 and dead is False and False), (b, pg, new)
                assert all(p >= 0 for p in m.block_table(rid, 0))
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
        held = [sum(1 for r in live for p in m.block_table(r, g) if p >= 0) for g in range(2)]
        assert [m.free_pages(g) + held[g] for g in range(2)] == [pages, pages]
        assert m.free_slots() == 5 - len(live)
    for rid in list(live):
        m.close(rid)
    assert m.free_pages(0) == pages and m.free_pages(1) == pages and m.free_slots() == 5
