"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; groups; reading another run's cache
(after the reference's tests/unit/test_kv.py:16-58)."""

from __future__ import annotations

import random

import pytest
import torch

from turingserve_b200.cache import CacheManager, NoFreePages, PageAllocator, RunNeeds
from turingserve_b200.parts.base import CacheNeed, StateNeed

FULL = CacheNeed(2, 16, None)
WIN = CacheNeed(2, 16, 24)


def test_allocator_never_hands_out_the_null_page_and_reuses_fifo():
    a = PageAllocator(5)
    got = [a.allocate() for _ in range(4)]
    assert got == [1, 2, 3, 4] and a.num_free == 0
    with pytest.raises(NoFreePages):
        a.allocate()
    a.free(3)
    a.free(1)
    assert [a.allocate(), a.allocate()] == [3, 1]                 # first freed, first reused
    with pytest.raises(ValueError):
        a.free(0)
    a.free(2)
    with pytest.raises(ValueError, match="twice"):
        a.free(2)
    a.check()


@pytest.mark.parametrize("n,pages", [(1, 1), (15, 1), (16, 1), (17, 2), (32, 2), (33, 3)])
def test_pages_and_slots(n, pages):
    m = CacheManager([RunNeeds(FULL, None)], 16, 10, 4)
    rc = m.admit("a")
    assert m.pages_needed(rc, n) == [pages]
    m.grow(rc, n)
    m.advance(rc, n)
    assert len(rc.tables[0]) == pages
    assert m.slot_of(rc, 0, n - 1) == rc.tables[0][(n - 1) // 16] * 16 + (n - 1) % 16
    m.grow(rc, 0)
    assert len(rc.tables[0]) == pages                              # growing is idempotent


def test_groups_are_formed_by_need_and_shared_runs_own_nothing():
    needs = [RunNeeds(FULL, None), RunNeeds(WIN, None), RunNeeds(FULL, None), RunNeeds(FULL, None, cache_from=1),
             RunNeeds(None, StateNeed((3,))), RunNeeds(WIN, StateNeed((2, 2), torch.float32))]
    m = CacheManager(needs, 8, 9, 3, torch.float32, "cpu")
    assert [g.runs for g in m.groups] == [[0, 2], [1, 5]]
    assert m.groups[0].pool.shape == (2, 2, 9, 2, 8, 16)
    v0, v1, v3, v4 = m.view(0), m.view(1), m.view(3), m.view(4)
    assert v0.group == 0 and v0.writable and v1.group == 1
    assert v3.group == 1 and not v3.writable and v3.k.data_ptr() == v1.k.data_ptr()
    assert v4 is None
    assert m.states[4].shape == (4, 3) and m.states[5].shape == (4, 2, 2) and m.states[0] is None  # 3 requests + the null slot
    with pytest.raises(ValueError, match="has none"):
        CacheManager([RunNeeds(None, None), RunNeeds(FULL, None, cache_from=0)], 8, 4, 2)


def test_state_slots_are_zeroed_on_admission_and_reused():
    m = CacheManager([RunNeeds(None, StateNeed((4,)))], 8, 4, 2, torch.float32, "cpu")
    a, b = m.admit("a"), m.admit("b")
    assert {a.slot, b.slot} == {0, 1} and not m.has_free_slot()
    with pytest.raises(NoFreePages):
        m.admit("c")
    m.states[0][a.slot] = 7.0
    m.release(a)
    c = m.admit("c")
    assert c.slot == a.slot and torch.all(m.states[0][c.slot] == 0)
    with pytest.raises(ValueError, match="twice"):
        m.release(a)
    m.check()


def test_window_gives_pages_back_as_it_passes_them():
    m = CacheManager([RunNeeds(FULL, None), RunNeeds(WIN, None)], 8, 40, 2)
    rc = m.admit("a")
    held = []
    for step_tokens in [20, 1, 1, 30, 1, 7, 50, 1]:
        m.grow(rc, step_tokens)
        m.advance(rc, step_tokens)
        n = rc.num_tokens
        full, win = rc.tables
        assert all(p != 0 for p in full) and len(full) == -(-n // 8)
        first_needed = max(0, n - 24 + 1)                         # oldest key the next query may see
        for p, page in enumerate(win):
            if (p + 1) * 8 <= first_needed:
                assert page == 0, f"page {p} should have been given back at length {n}"
            else:
                assert page != 0, f"page {p} still holds visible keys at length {n}"
        held.append(sum(1 for p in win if p))
        m.check()
    assert max(held[3:]) <= 24 // 8 + 7                           # bounded by window + a portion, not by length
    assert m.num_free(1) > m.num_free(0)
    m.release(rc)
    assert m.num_free(0) == m.num_free(1) == 39


def test_grow_is_all_or_nothing():
    m = CacheManager([RunNeeds(FULL, None), RunNeeds(WIN, None)], 8, 5, 2)       # 4 usable pages each
    a = m.admit("a")
    assert m.can_grow(a, 32) and not m.can_grow(a, 33) and not m.can_grow(a, 32, keep_free=1)
    assert m.can_grow(None, 32) and not m.can_grow(None, 33)
    with pytest.raises(NoFreePages):
        m.grow(a, 40)
    assert a.tables == [[], []] and m.num_free(0) == 4
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    m = CacheManager([RunNeeds(FULL, StateNeed((2,))), RunNeeds(WIN, None), RunNeeds(FULL, None, cache_from=0)],
                     rng.choice([4, 8, 16]), rng.randint(12, 40), 5, torch.float32, "cpu")
    if seed % 2:
        for g in m.groups:
            g.allocator.shuffle_free_list(rng)
    live = {}
    n = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.has_free_slot():
            n += 1
            live[f"r{n}"] = m.admit(f"r{n}")
        elif op < 0.8 and live:
            rc = rng.choice(list(live.values()))
            k = rng.choice([1, 1, 1, 2, 7, 16, 33])
            if m.can_grow(rc, k):
                m.grow(rc, k)
                m.advance(rc, k)
            else:
                with pytest.raises(NoFreePages):
                    m.grow(rc, k)
        elif live:
            rid = rng.choice(list(live))
            m.release(live.pop(rid))
        m.check()
        for rc in live.values():                                   # every visible position has a real page
            for gi, g in enumerate(m.groups):
                lo = 0 if g.need.window is None else max(0, rc.num_tokens - g.need.window + 1)
                for pos in range(lo, rc.num_tokens):
                    assert rc.tables[gi][pos // m.page_size] != 0
    for rc in list(live.values()):
        m.release(rc)
    m.check()
    assert all(g.allocator.num_free == g.allocator.num_usable for g in m.groups)
