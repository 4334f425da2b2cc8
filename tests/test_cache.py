"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of requests; window
groups give pages back as the window passes; state slots."""
import random

import pytest
import torch

from fusezap_core_b200.cache import CacheManager, KVNeed, OutOfPages, PageAllocator


def manager(needs=None, pages=16, page_size=4, max_len=64, states=None, requests=4):
    needs = needs or {0: KVNeed(2, 16, 0), 1: KVNeed(2, 16, 0)}
    return CacheManager(needs, states or {}, page_size, pages, requests, max_len, torch.float32, "cpu", allocate=bool(states))


def test_allocator_lifo_and_double_free():
    a = PageAllocator(4)
    p = a.allocate(3)
    assert p == [0, 1, 2] and a.num_free == 1
    a.free([1])
    assert a.allocate(1) == [1], "a page just given back is the next one handed out"
    with pytest.raises(OutOfPages):
        a.allocate(2)
    a.free([0])
    with pytest.raises(AssertionError, match="not held"):
        a.free([0])
    with pytest.raises(AssertionError, match="not held"):
        a.free([3 + 4])
    a.check()


def test_tables_slots_and_capacity():
    m = manager()
    assert len(m.groups) == 1 and m.groups[0].slots == [0, 1], "equal needs share one group and one table"
    assert m.capacity_tokens == 64 and m.max_pages_per_request == 16
    m.ensure("a", 5)
    assert m.table(0, "a") == [0, 1] and m.pages_needed("a", 8) == [0] and m.pages_needed("a", 9) == [1]
    m.commit("a", 5)
    m.ensure("b", 4); m.ensure("a", 9)
    assert m.table(0, "b") == [2] and m.table(0, "a") == [0, 1, 3]
    assert not m.can_ensure("c", 65) and m.can_ensure("c", 12 * 4) and not m.can_ensure("c", 12 * 4 + 1)
    with pytest.raises(OutOfPages):
        m.ensure("c", 60)
    assert not m.holds("c") and m.num_free_pages == 12, "a refused request holds nothing"
    m.free("a")
    m.ensure("c", 4)
    assert m.table(0, "c") == [3], "pages are used again, last freed first"
    m.free("b"); m.free("c"); m.free("nobody")
    assert m.num_free_pages == 16
    m.check()


def test_groups_with_different_needs_have_pages_of_their_own():
    m = manager({0: KVNeed(2, 16, 0), 1: KVNeed(2, 16, 8), 2: KVNeed(2, 16, 8), 3: KVNeed(1, 32, 0)})
    assert [g.slots for g in m.groups] == [[0], [1, 2], [3]] and m.slot_group == {0: 0, 1: 1, 2: 1, 3: 2}
    m.ensure("a", 30); m.commit("a", 30)
    full, win = m.table(0, "a"), m.table(1, "a")
    assert all(p >= 0 for p in full) and len(full) == 8
    # the next query (position 30) sees keys 23..30: pages 0..4 (positions < 20) are gone from the window group
    assert [p >= 0 for p in win] == [False] * 5 + [True] * 3
    assert m.groups[1].allocator.num_free == 16 - 3 and m.groups[0].allocator.num_free == 8
    m.ensure("a", 31); m.commit("a", 31)      # the next query (31) sees 24..31: page 5 (20..23) has passed
    assert m.table(1, "a")[5] == -1 and m.table(1, "a")[6] >= 0
    m.ensure("a", 35); m.commit("a", 35)      # the next query (35) sees 28..35: page 6 (24..27) has passed
    assert m.table(1, "a")[6] == -1 and m.table(1, "a")[7] >= 0 and m.table(1, "a")[8] >= 0
    m.check(); m.free("a"); m.check()
    assert all(g.allocator.num_free == 16 for g in m.groups)


def test_window_group_lets_a_long_request_live_in_few_pages():
    m = manager({0: KVNeed(1, 16, 8)}, pages=5, page_size=4, max_len=400)
    for n in range(1, 400):
        m.ensure("a", n); m.commit("a", n)
        assert 5 - m.num_free_pages <= 3
    m.check()


def test_state_slots():
    m = manager(states={(0, "s"): (3,), (1, "s"): (2, 2)}, requests=2)
    m.ensure("a", 3); m.ensure("b", 3)
    assert {m.state_slot("a"), m.state_slot("b")} == {0, 1}
    assert not m.can_ensure("c", 1), "no state slot left"
    m.states.tensors[(0, "s")][m.state_slot("a")] = 7.0
    slot = m.state_slot("a")
    m.free("a")
    m.ensure("c", 1)
    assert m.state_slot("c") == slot and float(m.states.tensors[(0, "s")][slot].abs().sum()) == 0.0, "a slot is zeroed when handed out"
    assert m.states.tensors[(1, "s")].shape == (2, 2, 2)
    m.check()
    plain = manager()
    plain.ensure("a", 1)
    assert plain.state_slot("a") == -1, "a model without state takes no slot"


@pytest.mark.parametrize("seed", range(6))
def test_random_lives(seed):
    """Random arrivals, growth, commits and departures over three groups: the invariants hold after every operation."""
    rng = random.Random(seed)
    m = manager({0: KVNeed(2, 16, 0), 1: KVNeed(2, 16, 6), 2: KVNeed(1, 32, 13)}, pages=24, page_size=4, max_len=96,
                states={(0, "s"): (2,)}, requests=5)
    lens: dict[int, int] = {}
    nxt = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(lens) < 7:
            lens[nxt] = 0; nxt += 1
        elif op < 0.8 and lens:
            r = rng.choice(list(lens))
            n = lens[r] + rng.choice((1, 1, 1, 2, 5, 17))
            if m.can_ensure(r, n):
                m.ensure(r, n); m.commit(r, n); lens[r] = n
            else:
                before = [g.allocator.num_free for g in m.groups]
                with pytest.raises((OutOfPages, ValueError)):
                    m.ensure(r, n)
                assert before == [g.allocator.num_free for g in m.groups], "a refused growth takes nothing"
        elif lens:
            r = rng.choice(list(lens))
            m.free(r); del lens[r]
        m.check()
        for r, n in lens.items():
            if n:
                assert all(p >= 0 for p in m.table(0, r)[: -(-n // 4)]) and len(m.table(0, r)) == -(-n // 4)
    for r in list(lens):
        m.free(r)
    m.check()
    assert all(g.allocator.num_free == 24 for g in m.groups) and m.states.num_free == 5


def test_state_slots_take_the_dtype_the_mixer_declares():
    cm = CacheManager({0: KVNeed(1, 16, 0)}, {(0, "s"): (5,), (1, "count"): ((2, 3), torch.int32), (2, "h"): ((4,), torch.bfloat16)},
                      4, 8, 3, 32, torch.float32, "cpu")
    t = cm.states.tensors
    assert t[(0, "s")].shape == (3, 5) and t[(0, "s")].dtype == torch.float32
    assert t[(1, "count")].shape == (3, 2, 3) and t[(1, "count")].dtype == torch.int32
    assert t[(2, "h")].dtype == torch.bfloat16
    cm.ensure("a", 3)
    slot = cm.state_slot("a")
    t[(1, "count")][slot] += 7
    cm.free("a")
    cm.ensure("b", 3)
    assert cm.state_slot("b") == slot and int(t[(1, "count")][slot].sum()) == 0, "a slot is zeroed when it is handed out"
