"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows release pages; state slots; what happens when pages run out (no GPU)."""

import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

from libmir_b200 import KvCachePressure, KvCapacity, NoFreeSlot, build_spec
from libmir_b200.cache import CacheManager, PagePool
from libmir_b200.config.spec import FixedState, PagedKv
from libmir_b200.models.decoder import CacheEntryPlan, DecoderModel
from libmir_b200.parts.base import BuildEnv
from tiny_configs import TINY_A, TINY_C


def plan_of(config):
    return DecoderModel(build_spec(config), BuildEnv(torch.float32, torch.device("meta"))).cache_plan()


def test_pool_fifo_and_double_free():
    pool = PagePool(4)
    first = pool.take(3)
    assert first == [0, 1, 2] and pool.free == 1
    pool.give_back([1])
    assert pool.take(2) == [3, 1] and pool.reused == 1     # oldest freed first; page 1 is used again
    with pytest.raises(RuntimeError, match="not held"):
        pool.give_back([1, 1])
    with pytest.raises(RuntimeError, match="only"):
        pool.take(5)


def test_decode_allocates_exactly_at_a_page_edge():
    manager = CacheManager(plan_of(TINY_A), page_size=4, num_pages=8, max_requests=2)
    seq = manager.admit("r")
    manager.grow(seq, 4); manager.commit(seq, 4)
    assert len(seq.tables[0]) == 1
    manager.grow(seq, 5); manager.commit(seq, 5)            # length == blocks * page_size -> one more page
    assert len(seq.tables[0]) == 2
    for length in (6, 7, 8):
        manager.grow(seq, length); manager.commit(seq, length)
        assert len(seq.tables[0]) == 2
    manager.check()


def test_capacity_and_pressure_take_nothing():
    manager = CacheManager(plan_of(TINY_A), page_size=4, num_pages=4, max_requests=3)
    a, b = manager.admit("a"), manager.admit("b")
    manager.grow(a, 9)
    with pytest.raises(KvCachePressure):
        manager.grow(b, 8)
    assert b.tables[0] == [] and manager.groups[0].pool.free == 1
    with pytest.raises(KvCapacity):
        manager.grow(b, 17)
    manager.release("a")
    manager.grow(b, 16)
    assert manager.groups[0].pool.free == 0 and manager.groups[0].pool.reused == 3
    manager.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    manager = CacheManager(plan_of(TINY_C), page_size=8, num_pages=24, max_requests=2)
    full, windowed = manager.groups
    assert windowed.window == 40
    seq = manager.admit("r")
    length = 0
    for portion in (30, 30, 30, 1, 1, 1, 50):
        manager.grow(seq, length + portion)
        length += portion
        manager.commit(seq, length)
        # keys a later query (position >= length) can see: j >= length - window + 1
        first_needed = max(0, length - 40 + 1)
        table = seq.tables[1]
        for block, page in enumerate(table):
            if block < first_needed // 8:
                assert page == -1
            else:
                assert page >= 0
        assert all(page >= 0 for page in seq.tables[0])
        manager.check()
    assert full.pool.held == -(-length // 8) and windowed.pool.held <= 40 // 8 + 2
    manager.release("r")
    assert full.pool.free == 24 and windowed.pool.free == 24


def test_slots_and_fixed_state_entries():
    plan = [CacheEntryPlan(0, PagedKv(2, 16, None), 0, True), CacheEntryPlan(1, FixedState((4, 8)), 1, True),
            CacheEntryPlan(2, PagedKv(2, 16, None), 0, False), CacheEntryPlan(3, None, 3, True)]
    manager = CacheManager(plan, page_size=4, num_pages=4, max_requests=2)
    assert manager.state_entries == {1: FixedState((4, 8))}
    assert manager.entry_group == {0: 0, 2: 0} and manager.entry_local == {0: 0, 2: 0}
    assert len(manager.groups[0].entries) == 1                     # the reader owns no storage
    a, b = manager.admit("a"), manager.admit("b")
    assert {a.slot, b.slot} == {0, 1} and manager.take_fresh_slots() == [a.slot, b.slot]
    with pytest.raises(NoFreeSlot):
        manager.admit("c")
    manager.release("a")
    c = manager.admit("c")
    assert c.slot == a.slot and manager.take_fresh_slots() == [c.slot]
    with pytest.raises(ValueError, match="already live"):
        manager.admit("c")
    with pytest.raises(KeyError):
        manager.release("zzz")
    manager.check()


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10_000), page_size=st.sampled_from([1, 4, 8, 16]), pages=st.integers(6, 40),
       windowed=st.booleans())
def test_random_orders_never_lose_or_double_hold_a_page(seed, page_size, pages, windowed):
    rng = random.Random(seed)
    manager = CacheManager(plan_of(TINY_C if windowed else TINY_A), page_size, pages, max_requests=4)
    lengths = {}
    counter = 0
    for _ in range(200):
        action = rng.random()
        if action < 0.25 and manager.free_slots:
            name = f"r{counter}"
            counter += 1
            manager.admit(name)
            lengths[name] = 0
        elif action < 0.85 and lengths:
            name = rng.choice(sorted(lengths))
            seq = manager.live[name]
            portion = rng.choice([1, 1, 1, 2, 3, 7, 16, 33])
            before = [list(t) for t in seq.tables]
            free_before = [g.pool.free for g in manager.groups]
            try:
                manager.grow(seq, lengths[name] + portion)
            except (KvCachePressure, KvCapacity):
                assert [list(t) for t in seq.tables] == before           # nothing was taken
                assert [g.pool.free for g in manager.groups] == free_before
            else:
                lengths[name] += portion
                manager.commit(seq, lengths[name])
        elif lengths:
            name = rng.choice(sorted(lengths))
            manager.release(name)
            del lengths[name]
        manager.check()
    for name in list(lengths):
        manager.release(name)
    manager.check()
    assert all(g.pool.free == g.pool.count for g in manager.groups) and manager.free_slots == 4
