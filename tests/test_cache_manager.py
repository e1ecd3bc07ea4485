"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
pages of a window group come back while the request runs; freed pages are used again first."""
import random

import pytest
import torch

from rvllm_b200 import KvExhausted, SchedulerError
from rvllm_b200.cache import CacheManager, PagePool, SlotPool
from rvllm_b200.parts import KvCacheNeed, StateNeed

FULL = KvCacheNeed(2, 16, None)
WIN = KvCacheNeed(2, 16, 20)


def manager(num_pages=12, page=8, max_seqs=4, needs=None, allocate=False):
    needs = needs if needs is not None else {0: FULL, 1: WIN, 2: WIN, 3: FULL}
    return CacheManager(needs, num_pages, page, max_seqs, torch.float32, "cpu", allocate=allocate)


def test_pool_is_a_stack_and_refuses_double_free():
    p = PagePool(4)
    a = p.allocate(3, "x")
    assert a == [0, 1, 2] and p.num_free == 1
    p.release([1], "x")
    assert p.allocate(1, "y") == [1]                      # the page given back is the next handed out
    with pytest.raises(SchedulerError, match="held by"):
        p.release([1], "x")
    p.release([1], "y")
    with pytest.raises(SchedulerError, match="freed twice"):
        p.release([1], "y")
    with pytest.raises(KvExhausted) as e:
        p.allocate(5, "z")
    assert (e.value.needed_blocks, e.value.free_blocks) == (5, 2)
    p.check()


def test_groups_are_formed_by_need():
    m = manager()
    assert len(m.groups) == 2
    assert m.groups[0].cache_slots == [0, 3] and m.groups[1].cache_slots == [1, 2]
    assert m.view(3).group == 0 and m.view(2).group == 1
    m2 = manager(allocate=True, needs={0: FULL, 1: StateNeed((3, 5)), 2: None})
    assert m2.view(0).kv.shape == (12, 2, 2, 8, 16)
    assert m2.view(1).state.shape == (4, 3, 5) and m2.view(1).kv is None and m2.view(2).group is None
    assert CacheManager.bytes_per_page({0: FULL, 1: WIN}, 8, torch.bfloat16) == 2 * 2 * 2 * 8 * 16 * 2


def test_append_allocates_on_demand_and_all_or_nothing():
    m = manager(num_pages=4)
    m.admit("a")
    assert m.append("a", 5) == 0 and m.num_free_pages() == [3, 3]
    assert m.append("a", 3) == 5 and m.num_free_pages() == [3, 3]      # still inside the first page
    assert m.append("a", 1) == 8 and m.num_free_pages() == [2, 2]
    assert m.slot_mapping("a", 0, 7, 3) == [7, 8 * m.block_table("a", 0)[1], 8 * m.block_table("a", 0)[1] + 1]
    m.admit("b")
    with pytest.raises(KvExhausted):
        m.append("b", 8 * 3)                                            # needs 3, only 2 free
    assert m.num_free_pages() == [2, 2] and m.num_tokens("b") == 0      # nothing was taken
    assert m.can_append("b", 16) and not m.can_append("b", 17)
    assert not m.can_append("b", 16, reserved=[1, 0])
    m.check()


def test_window_pages_come_back_while_the_request_runs():
    m = manager(num_pages=8, needs={0: FULL, 1: WIN})
    m.admit("a")
    m.append("a", 50)                         # 7 pages in both groups
    assert m.num_free_pages() == [1, 1]
    freed = m.release_passed("a")
    # next query at position 50 sees keys > 50 - 20 = 30, i.e. from 31: pages 0..2 (positions 0..23) go
    assert freed == 3 and m.num_free_pages() == [1, 4]
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and all(p >= 0 for p in m.block_table("a", 1)[3:])
    assert all(p >= 0 for p in m.block_table("a", 0))
    with pytest.raises(SchedulerError, match="given back"):
        m.slot_mapping("a", 1, 10, 1)
    assert m.release_passed("a") == 0
    m.append("a", 9)                          # 59 tokens: 8 logical pages; the window group reuses a freed page
    assert m.num_free_pages() == [0, 3]
    m.release_passed("a")                     # keys from 40: page 4 (positions 32..39) goes too
    assert m.block_table("a", 1)[:5] == [-1] * 5
    m.check()
    m.free("a")
    assert m.num_free_pages() == [8, 8]
    m.check()


def test_state_slots_are_zeroed_on_admission():
    m = manager(allocate=True, needs={0: FULL, 1: StateNeed((3,))})
    s = m.admit("a")
    m.view(1).state[s] = 7.0
    m.free("a")
    s2 = m.admit("b")
    assert s2 == s and float(m.view(1).state[s2].abs().sum()) == 0.0
    for i in range(3):
        m.admit(f"x{i}")
    with pytest.raises(SchedulerError, match="slots"):
        m.admit("one too many")
    with pytest.raises(SchedulerError, match="already"):
        m.admit("b")


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page=4, max_seqs=5)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{next_id}"
            next_id += 1
            m.admit(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 15])
            if m.can_append(rid, n):
                start = m.append(rid, n)
                assert start == live[rid]
                live[rid] += n
                for g in range(2):
                    slots = m.slot_mapping(rid, g, start, n)
                    assert len(set(slots)) == n
                m.release_passed(rid)
            else:
                with pytest.raises(KvExhausted):
                    m.append(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        # a window group never holds more than the window plus the pages at its two edges
        for rid in live:
            held = sum(1 for p in m.block_table(rid, 1) if p >= 0)
            assert held <= 20 // 4 + 2
    for rid in list(live):
        m.free(rid)
    m.check()
    assert m.num_free_pages() == [24, 24] and m.slots.num_free == 5
    with pytest.raises(KeyError):
        m.free("r0")                                         # freeing twice is an error
