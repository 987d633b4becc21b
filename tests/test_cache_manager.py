"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; groups have pools of their own."""
import random

import pytest
import torch

from pih_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool, StateSlotPool
from pih_b200.parts import PagedKVNeed, StateNeed


def manager(needs, page_size=4, num_pages=16, max_requests=4, reads=None):
    return CacheManager(needs, reads or [None] * len(needs), page_size=page_size, num_pages=num_pages,
                        max_requests=max_requests, device=torch.device("cpu"), dtype=torch.float32)


FULL = PagedKVNeed(2, 8, None)
WIN = PagedKVNeed(2, 8, 6)


def test_pool_refuses_double_free_and_foreign_free():
    pool = PagePool(4)
    a = pool.allocate(2, "a")
    b = pool.allocate(1, "b")
    with pytest.raises(ValueError, match="belongs to"):
        pool.free(b, "a")
    pool.free(a, "a")
    with pytest.raises(ValueError, match="freed twice"):
        pool.free(a, "a")
    with pytest.raises(ValueError, match="named twice"):
        pool.free(b + b, "b")
    with pytest.raises(OutOfPages):
        pool.allocate(4, "c")
    assert pool.num_free == 3                       # a failed allocation changes nothing
    pool.check()


def test_freed_pages_are_used_again():
    pool = PagePool(3)
    first = pool.allocate(3, "a")
    pool.free(first[:2], "a")
    again = pool.allocate(2, "b")
    assert set(again) == set(first[:2]) and pool.pages_handed_out == 5


def test_slots():
    slots = StateSlotPool(2)
    s0, s1 = slots.acquire("a"), slots.acquire("b")
    with pytest.raises(OutOfSlots):
        slots.acquire("c")
    with pytest.raises(ValueError):
        slots.release(s0, "b")
    slots.release(s0, "a")
    with pytest.raises(ValueError):
        slots.release(s0, "a")
    assert slots.acquire("c") == s0 and s1 != s0
    slots.check()


def test_groups_by_need_and_shared_cache_entries():
    m = manager([FULL, WIN, FULL, None, WIN], reads=[None, None, None, 0, None])
    assert len(m.groups) == 2
    assert m.groups[0].entries == [0, 2] and m.groups[1].entries == [1, 4]
    assert m.entry_group[3] == m.entry_group[0]           # entry 3 reads entry 0's cache
    assert m.groups[0].kv.shape == (2, 16, 2, 2, 4, 8)
    assert m.bytes_per_token() == 4 * 2 * 2 * 8 * 4


def test_append_is_all_groups_or_none_and_commit_counts():
    m = manager([FULL, WIN], num_pages=3)
    m.add_request("a")
    m.append("a", 9)                                       # 3 pages in each group
    assert m.num_free_pages() == [0, 0]
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.append("b", 1)
    assert m.requests["b"].pages == [[], []] and m.requests["b"].pending == 0
    m.commit("a")
    assert m.requests["a"].num_tokens == 9
    # window 6, length 9: later queries read keys >= 4, page 0 (keys 0..3) went back in the window group only
    assert m.num_free_pages() == [0, 1] and m.requests["a"].pages[1][0] == -1
    with pytest.raises(OutOfPages):
        m.append("b", 3)                                   # room in the window group alone is not enough
    assert m.num_free_pages() == [0, 1] and m.requests["b"].pages == [[], []]
    m.release("a"), m.release("b")
    assert m.num_free_pages() == [3, 3]
    m.check()


def test_window_never_frees_a_page_that_a_later_query_reads():
    m = manager([WIN], page_size=4, num_pages=64)
    m.add_request("a")
    length = 0
    rnd = random.Random(0)
    while length < 150:
        n = rnd.choice([1, 1, 2, 5, 9])
        m.append("a", n)
        # every query of this step reads keys p-5..p; their pages must be held
        for p in range(length, length + n):
            for j in range(max(0, p - 5), p + 1):
                assert m.requests["a"].pages[0][j // 4] >= 0
        m.slot_mapping(0, "a", length, n)
        m.commit("a")
        length += n
        held = [p for p in m.requests["a"].pages[0] if p >= 0]
        assert len(held) <= 3                              # window 6 over pages of 4 spans at most 3 pages
        m.check()
    m.release("a")
    assert m.num_free_pages() == [64]


def test_random_orders_of_requests_keep_the_books():
    rnd = random.Random(1)
    m = manager([FULL, WIN, FULL], page_size=4, num_pages=24, max_requests=5)
    live, serial = {}, 0
    for _ in range(3000):
        op = rnd.random()
        if op < 0.15 and len(live) < 5:
            rid = f"r{serial}"
            serial += 1
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 3, 7, 13])
            before = m.num_free_pages()
            try:
                m.append(rid, n)
            except OutOfPages:
                assert m.num_free_pages() == before
                continue
            if rnd.random() < 0.1:
                m.rollback(rid)
            else:
                m.commit(rid)
                live[rid] += n
            assert m.requests[rid].num_tokens == live[rid]
        elif op < 0.9 and live:
            rid = rnd.choice(list(live))
            m.release(rid)
            del live[rid]
        elif live:
            rid = rnd.choice(list(live))
            m.reset(rid)
            live[rid] = 0
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.num_free_pages() == [24, 24] and m.slots.num_free == 5


def test_state_slots_are_zeroed_for_a_new_request():
    m = manager([FULL, StateNeed((3,), torch.float32)], max_requests=2)
    rc = m.add_request("a")
    m.state_tensors[1][rc.slot] = 7.0
    m.release("a")
    rc2 = m.add_request("b")
    assert rc2.slot == rc.slot and float(m.state_tensors[1][rc2.slot].abs().sum()) == 0.0


def test_block_table_rows_and_slot_mapping():
    m = manager([FULL], page_size=4, num_pages=8)
    m.add_request("a")
    m.append("a", 6)
    pages = list(m.requests["a"].pages[0])
    assert m.block_table_rows(0, ["a"], 3) == [pages + [-1]]
    assert m.slot_mapping(0, "a", 0, 6) == [pages[0] * 4 + i for i in range(4)] + [pages[1] * 4, pages[1] * 4 + 1]


def test_queued_steps_count_for_the_next_step_but_only_confirmed_ones_give_pages_back():
    m = manager([FULL, WIN], page_size=4, num_pages=8)
    m.add_request("a")
    m.append("a", 9)
    m.commit("a", confirmed=False)                         # queued on the device, its error word not seen yet
    rc = m.requests["a"]
    assert rc.num_tokens == 9 and rc.confirmed_tokens == 0 and rc.unconfirmed == [9]
    assert m.num_free_pages() == [5, 5]                    # the window group keeps page 0 until the step is confirmed
    m.append("a", 1)                                       # the next step starts behind the queued tokens
    assert m.slot_mapping(1, "a", 9, 1) == [rc.pages[1][2] * 4 + 1]
    m.commit("a", confirmed=False)
    m.confirm("a")
    assert rc.confirmed_tokens == 9 and m.num_free_pages() == [5, 6] and rc.pages[1][0] == -1
    m.confirm("a")
    assert rc.confirmed_tokens == 10 and rc.unconfirmed == []
    with pytest.raises(ValueError, match="no queued step"):
        m.confirm("a")
    m.check()


def test_rollback_of_queued_steps_returns_to_the_confirmed_length():
    m = manager([FULL, WIN], page_size=4, num_pages=8)
    m.add_request("a")
    m.append("a", 6)
    m.commit("a")
    held = [list(pl) for pl in m.requests["a"].pages]
    for n in (5, 1):
        m.append("a", n)
        m.commit("a", confirmed=False)
    m.append("a", 3)                                       # a third step, not even queued
    m.rollback("a")                                        # plain rollback: only the append is undone
    rc = m.requests["a"]
    assert rc.num_tokens == 12 and rc.unconfirmed == [5, 1] and rc.pending == 0
    m.rollback("a", unconfirmed=True)                      # ... and now the queued steps too
    assert rc.num_tokens == rc.confirmed_tokens == 6 and rc.unconfirmed == []
    assert [list(pl) for pl in rc.pages] == held
    m.check()
    m.append("a", 2)
    with pytest.raises(ValueError, match="queued steps to confirm"):
        m.commit("a", confirmed=False), m.append("a", 1), m.commit("a")
    m.release("a")
    m.check()
    assert m.num_free_pages() == [8, 8]


def test_rollback_puts_the_state_slot_back_as_it_was_before_the_step():
    m = manager([FULL, StateNeed((3,), torch.float32)], max_requests=2)
    slot = m.add_request("a").slot
    state = m.state_tensors[1]
    m.append("a", 2)
    state[slot] = 1.0                                      # the step's mixer advanced the state
    m.commit("a")
    m.append("a", 1)
    state[slot] = 2.0
    m.rollback("a")                                        # the step failed half-way: the old state is back
    assert state[slot].tolist() == [1.0] * 3
    # queued steps: the state goes back to what it was at the confirmed length
    for value in (3.0, 4.0):
        m.append("a", 1)
        state[slot] = value
        m.commit("a", confirmed=False)
    m.confirm("a")                                         # the step that wrote 3.0 succeeded
    m.append("a", 1)
    state[slot] = 5.0
    m.rollback("a", unconfirmed=True)
    assert state[slot].tolist() == [3.0] * 3 and m.requests["a"].num_tokens == 3


def test_random_orders_with_queued_steps_keep_the_books():
    rnd = random.Random(7)
    m = manager([FULL, WIN], page_size=4, num_pages=24, max_requests=4)
    live, serial = {}, 0                                   # rid -> [confirmed length, queued counts]
    for _ in range(3000):
        op = rnd.random()
        if op < 0.15 and len(live) < 4:
            rid = f"r{serial}"
            serial += 1
            m.add_request(rid)
            live[rid] = [0, []]
        elif op < 0.6 and live:
            rid = rnd.choice(list(live))
            n = rnd.choice([1, 1, 2, 5, 11])
            try:
                m.append(rid, n)
            except OutOfPages:
                continue
            if len(live[rid][1]) < 2 and rnd.random() < 0.7:
                m.commit(rid, confirmed=False)
                live[rid][1].append(n)
            elif not live[rid][1]:
                m.commit(rid)
                live[rid][0] += n
            else:
                m.rollback(rid)
        elif op < 0.8 and live:
            rid = rnd.choice(list(live))
            if live[rid][1]:
                m.confirm(rid)
                live[rid][0] += live[rid][1].pop(0)
        elif op < 0.9 and live:
            rid = rnd.choice(list(live))
            m.rollback(rid, unconfirmed=True)
            live[rid][1] = []
        elif live:
            rid = rnd.choice(list(live))
            m.release(rid)
            del live[rid]
        for rid, (confirmed, queued) in live.items():
            rc = m.requests[rid]
            assert rc.confirmed_tokens == confirmed and rc.num_tokens == confirmed + sum(queued)
            # every key that a query from the confirmed length on may read is still held
            for j in range(max(0, confirmed - 5), rc.num_tokens):
                assert rc.pages[1][j // 4] >= 0
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.num_free_pages() == [24, 24]
