"""The cache manager's accounting, without a GPU: no page lost, held twice or freed twice,
under random orders of requests; window groups give pages back; slots."""

import random

import pytest
import torch

from scratch_llm_b200.cache import CacheManager, PageAccountingError, PagePool
from scratch_llm_b200.parts import KVSpec, StateSpec

FULL = KVSpec(2, 16, None)
WIN = KVSpec(2, 16, 20)


def test_pool_alloc_free_reuse():
    pool = PagePool(4)
    a = pool.alloc(3, "a")
    assert a == [0, 1, 2] and pool.n_free == 1
    assert pool.alloc(2, "b") is None and pool.n_free == 1  # nothing taken
    pool.free([1], "a")
    assert pool.alloc(1, "b") == [1]  # the page just freed is handed out again
    with pytest.raises(PageAccountingError, match="held by"):
        pool.free([0], "b")
    pool.free([0, 2], "a")
    with pytest.raises(PageAccountingError, match="double free"):
        pool.free([0], "a")
    pool.check()


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([FULL, KVSpec(1, 32, None)], [None, None], page_size=8, n_pages=4,
                     max_requests=2)
    assert len(m.groups) == 2
    m.admit("a")
    assert m.reserve("a", 17)  # 3 pages in each group
    m.commit("a", 17)
    m.admit("b")
    assert m.pages_needed("b", 9) == [2, 2]
    assert not m.reserve("b", 9)
    assert m.free_pages() == [1, 1] and m.table_of("b", 0) == []
    assert m.reserve("b", 8)
    m.check()
    m.release("a")
    assert m.free_pages() == [3, 3]
    assert m.reserve("b", 9)  # now it fits, with a's pages
    m.check()


def test_entries_with_equal_needs_share_a_group():
    m = CacheManager([FULL, FULL, WIN, None, FULL], [None] * 5, 16, 8, 2)
    assert len(m.groups) == 2
    assert m.groups[0].entries == [0, 1, 4] and m.groups[1].entries == [2]
    assert m.entry_group[3] is None and m.entry_group[4] == (0, 2)


def test_window_group_gives_pages_back():
    m = CacheManager([FULL, WIN], [None, None], page_size=8, n_pages=16, max_requests=1)
    m.admit("a")
    for step, n in enumerate([30, 1, 1, 1, 20, 1]):
        assert m.reserve("a", n)
        m.commit("a", n)
        m.check()
        n_tok = m.requests["a"].n_tokens
        full, win = m.table_of("a", 0), m.table_of("a", 1)
        assert len(full) == len(win) == -(-n_tok // 8) and all(p >= 0 for p in full)
        # a page is dead once its last position is <= n_tok - window
        for i, p in enumerate(win):
            assert (p < 0) == ((i + 1) * 8 - 1 <= n_tok - 20), (step, i)
    assert m.free_pages()[1] > m.free_pages()[0]
    m.release("a")
    assert m.free_pages() == [16, 16]
    m.check()


def test_commit_beyond_reservation_is_refused():
    m = CacheManager([FULL], [None], 16, 4, 1)
    m.admit("a")
    m.reserve("a", 5)
    with pytest.raises(ValueError, match="reserved"):
        m.commit("a", 6)


def test_slots_and_state():
    m = CacheManager([FULL], [StateSpec((3,), torch.float32)], 16, 4, 2, device=None)
    a, b = m.admit("a"), m.admit("b")
    assert {a.slot, b.slot} == {0, 1} and m.admit("c") is None
    with pytest.raises(ValueError, match="already live"):
        m.admit("a")
    m.release("a")
    assert m.admit("c").slot == a.slot
    m.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_accounting_whole(seed):
    rng = random.Random(seed)
    m = CacheManager([FULL, WIN, FULL], [None] * 3, page_size=4, n_pages=40, max_requests=5)
    live, next_id, refused = {}, 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            assert m.admit(next_id) is not None
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            before = m.free_pages()
            if m.reserve(rid, n):
                m.commit(rid, n)
                live[rid] += n
            else:
                refused += 1
                assert m.free_pages() == before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.requests[rid].n_tokens == n
            assert len(m.table_of(rid, 0)) >= -(-n // 4)
            for g in range(len(m.groups)):   # the array copy of a table never drifts from it
                assert m.table_array(rid, g).tolist() == m.table_of(rid, g)
    assert refused > 0  # the pool did run out
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.free_pages() == [40, 40] and m.n_free_slots == 5
    st = m.waste_stats()
    assert st["allocated_tokens"] == 0
