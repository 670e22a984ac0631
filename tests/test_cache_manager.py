"""Cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; groups have pools of their own; prefix reuse."""
import random

import pytest

from llm_steadyinfer_b200.cache import CacheLayout, CacheManager, OutOfPages, OutOfSlots, PageError, PagePool
from llm_steadyinfer_b200.parts.base import CacheNeed, StateNeed

FULL = CacheNeed(2, 16, None)
WIN = CacheNeed(2, 16, 20)


def manager(needs, page_size=4, num_pages=16, max_requests=4, states=None, prefix=False, cache_from=None):
    states = states or [None] * len(needs)
    return CacheManager(CacheLayout(needs, states, cache_from), page_size, num_pages, max_requests, prefix)


def test_pool_basics():
    p = PagePool(4)
    assert p.allocate(2) == [0, 1] and p.num_free == 2
    assert p.allocate(3) is None and p.num_free == 2           # all or nothing
    p.release(1)
    assert p.allocate(1) == [1]                               # last freed, first reused
    with pytest.raises(PageError):
        p.release(3)                                          # never taken
    p.release(0)
    with pytest.raises(PageError):
        p.release(0)                                          # freed twice
    with pytest.raises(PageError):
        p.retain(0)                                           # free and without content


def test_grow_commit_release_and_table_order():
    m = manager([FULL, FULL])
    assert len(m.groups) == 1 and m.groups[0].layers == [0, 1]
    m.admit("a")
    m.grow("a", 9)                       # 3 pages of 4
    assert m.table(0, "a") == [0, 1, 2]
    m.commit("a", 9)
    m.grow("a", 12)                      # still 3 pages
    assert m.table(0, "a") == [0, 1, 2]
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.grow("b", 4 * 14)              # 14 pages, 13 free: nothing is taken
    assert m.free_pages() == 13 and m.table(0, "b") == []
    m.release("a")
    assert m.free_pages() == 16
    m.grow("b", 5)
    assert m.table(0, "b") == [2, 1]      # freed pages are used again, last freed first
    m.check_invariant()


def test_slots():
    m = manager([FULL], max_requests=2, states=[StateNeed((3,))])
    assert m.admit("a") == 0 and m.slot("a") == 0
    m.admit("b")
    with pytest.raises(OutOfSlots):
        m.admit("c")
    m.release("a")
    m.admit("c")
    assert m.slot("c") == 0 and m.slot("b") == 1
    assert sorted(m.new_slots) == [0, 0, 1]
    m.check_invariant()


def test_window_group_gives_pages_back_and_has_its_own_pool():
    m = manager([FULL, WIN, FULL, WIN], page_size=4, num_pages=32)
    assert len(m.groups) == 2 and m.groups[0].layers == [0, 2] and m.groups[1].layers == [1, 3]
    m.admit("a")
    length = 0
    for n in (10, 7, 30, 1, 1, 25):
        m.grow("a", length + n)
        length += n
        m.commit("a", length)
        full, win = m.table(0, "a"), m.table(1, "a")
        assert all(p >= 0 for p in full) and len(full) == -(-length // 4)
        first_needed = max(0, length - 20 + 1)
        for b, p in enumerate(win):
            assert (p < 0) == ((b + 1) * 4 <= first_needed), (length, b, win)
        m.check_invariant()
    assert m.free_pages(1) > m.free_pages(0)
    assert m.can_truncate_to(40) == 0                 # a window cannot be cut back: recompute from 0
    assert m.truncate("a", 40) == 0 and m.table(1, "a") == []
    m.release("a")
    assert m.free_pages(0) == 32 and m.free_pages(1) == 32


def test_layer_reading_another_layers_cache():
    lay = CacheLayout([FULL, FULL, FULL], [None] * 3, [None, None, 0])
    assert lay.layer_group == [0, 0, 0] and lay.layer_index_in_group == [0, 1, 0] and lay.group_layers == [[0, 1]]
    with pytest.raises(ValueError):
        CacheLayout([FULL, FULL], [None] * 2, [1, 0])


def test_truncate_keeps_whole_pages():
    m = manager([FULL])
    m.admit("a"); m.grow("a", 14); m.commit("a", 14)
    assert m.truncate("a", 9) == 8 and m.table(0, "a") == [0, 1] and m.free_pages() == 14
    m.grow("a", 14)
    assert m.table(0, "a") == [0, 1, 3, 2]
    m.check_invariant()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariant(seed):
    rng = random.Random(seed)
    windowed = seed % 2 == 1
    m = manager([FULL, WIN] if windowed else [FULL], page_size=4, num_pages=24, max_requests=5, prefix=not windowed)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            toks = [rng.randrange(3) for _ in range(rng.randrange(1, 30))]
            held = m.admit(next_id, toks)
            assert held % 4 == 0 and held < len(toks)
            live[next_id] = {"toks": toks, "len": held}
            next_id += 1
        elif op < 0.7 and live:
            r = rng.choice(list(live))
            n = rng.randrange(1, 12)
            st = live[r]
            try:
                m.grow(r, st["len"] + n)
            except OutOfPages:
                before = [m.free_pages(g) for g in range(len(m.groups))]
                assert before == [m.free_pages(g) for g in range(len(m.groups))]
            else:
                st["len"] += n
                m.commit(r, st["len"])
                if rng.random() < 0.5:
                    m.remember_prefix(r, st["toks"])
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            live[r]["len"] = m.truncate(r, rng.randrange(0, live[r]["len"] + 1))
            assert m.length(r) == live[r]["len"]
        elif live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        m.check_invariant()
    for r in list(live):
        m.release(r)
    m.check_invariant()
    assert all(m.free_pages(g) == 24 for g in range(len(m.groups)))
    assert m.slots.num_free == 5


def test_prefix_chain_matches_only_equal_history():
    m = manager([FULL], page_size=4, num_pages=8, prefix=True)
    a = [1, 2, 3, 4, 5, 6, 7, 8, 9]
    m.admit("a", a); m.grow("a", 9); m.commit("a", 9); m.remember_prefix("a", a)
    assert len(m.match_prefix(a)) == 2                          # whole pages, one token left to compute
    assert len(m.match_prefix([1, 2, 3, 4, 5, 6, 7, 8])) == 1   # at least one token must be computed
    assert m.match_prefix([9, 9, 9, 9, 5, 6, 7, 8, 1]) == []    # equal block after another history: no match
    assert m.admit("b", a + [3]) == 8
    assert m.table(0, "b") == m.table(0, "a")[:2]
    m.release("a")
    m.check_invariant()
    assert m.free_pages() == 6                                   # two pages still held by b
    m.release("b")
    assert m.free_pages() == 8
    assert m.admit("c", a) == 8                                  # parked pages are taken back
    m.check_invariant()
    m.release("c")
    # when the pool needs them the parked pages lose their content
    m.admit("d"); m.grow("d", 32); m.commit("d", 32)
    assert m.match_prefix(a) == []
    m.release("d")
    m.check_invariant()
