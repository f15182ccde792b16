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


def test_pool_counts_holders_of_shared_pages():
    pool = PagePool(3)
    a, b = pool.take(2)
    pool.mark_cached(a)                                      # the index's own reference
    assert pool.holders(a) == 2 and pool.reclaimable == 0 and pool.available == 1
    pool.give_back([a])                                      # only the index holds it now
    assert pool.holders(a) == 1 and pool.reclaimable == 1 and pool.available == 2 and pool.free == 1
    pool.retain(a); pool.retain(a)                           # two requests share it
    assert pool.holders(a) == 3 and pool.reclaimable == 0
    with pytest.raises(RuntimeError, match="cannot be evicted"):
        pool.evict(a)
    pool.give_back([a, a])
    pool.evict(a)
    assert pool.free == 2 and not pool.is_cached(a) and pool.holders(a) == 0
    with pytest.raises(RuntimeError, match="not held"):
        pool.retain(a)
    with pytest.raises(RuntimeError, match="cannot be cached"):
        pool.mark_cached(a)
    pool.mark_cached(b)
    with pytest.raises(RuntimeError, match="cannot be cached"):
        pool.mark_cached(b)
    pool.give_back([b])
    with pytest.raises(RuntimeError, match="not held"):
        pool.give_back([b])
    pool.check()


def prefix_manager(pages=8, page_size=4, requests=4):
    return CacheManager(plan_of(TINY_A), page_size, pages, requests, prefix_cache=True, model_key="m")


def feed(manager, name, tokens, portion=5):
    """Admit a request and cache all of `tokens` in portions; returns the sequence."""
    seq = manager.admit(name, tokens)
    while seq.length < len(tokens):
        step = tokens[seq.length:seq.length + portion]
        manager.grow(seq, seq.length + len(step))
        manager.commit(seq, seq.length + len(step), step)
    return seq


def test_prefix_pages_are_found_shared_and_leave_one_token_to_compute():
    manager = prefix_manager()
    prompt = list(range(50, 64))                             # 14 tokens: three full pages and two tokens
    a = feed(manager, "a", prompt)
    assert a.prefix_tokens == 0 and len(manager.prefix) == 3
    manager.check()
    b = manager.admit("b", prompt)                           # while a is live: its pages are shared
    assert b.length == 12 and b.prefix_tokens == 12 and b.tables[0] == a.tables[0][:3]
    assert [manager.groups[0].pool.holders(p) for p in b.tables[0]] == [3, 3, 3]
    manager.release("a")
    manager.check()
    c = manager.admit("c", prompt[:12])                      # all of it is cached: the last page is computed again
    assert c.length == 8
    d = manager.admit("d", prompt[:5] + [7] + prompt[6:])    # differs inside the second page
    assert d.length == 4 and d.tables[0] == b.tables[0][:1]
    manager.release("b"); manager.release("c"); manager.release("d")
    pool = manager.groups[0].pool
    assert pool.free == 5 and pool.available == 8 and pool.reclaimable == 3
    e = manager.admit("e")                                   # no tokens given: nothing is looked up
    assert e.length == 0 and e.tables[0] == []
    manager.check()
    assert manager.stats()["prefix_hit_tokens"] == 12 + 8 + 4 and manager.stats()["cached_prefix_pages"] == 3


def test_a_page_is_found_only_behind_its_own_prefix_and_its_own_model():
    manager = prefix_manager()
    feed(manager, "a", [1, 2, 3, 4, 5, 6, 7, 8, 9])
    manager.release("a")
    assert manager.admit("b", [9, 9, 9, 9, 5, 6, 7, 8, 9]).length == 0      # same second page, other first page
    other = CacheManager(plan_of(TINY_A), 4, 8, 4, prefix_cache=True, model_key="other")
    other.prefix = manager.prefix                                              # (same index, another model's key)
    assert other.admit("c", [1, 2, 3, 4, 5, 6, 7, 8, 9]).length == 0


def test_cached_pages_are_evicted_oldest_first_and_never_while_a_request_holds_them():
    manager = prefix_manager(pages=6)
    old = list(range(100, 109))                              # two full pages each
    new = list(range(200, 209))
    feed(manager, "old", old); manager.release("old")
    feed(manager, "new", new); manager.release("new")
    pool = manager.groups[0].pool
    assert len(manager.prefix) == 4 and pool.free == 2 and pool.available == 6
    holder = manager.admit("holder", old)                    # holds old's two pages (and makes them the newest)
    assert holder.length == 8
    big = manager.admit("big")
    manager.grow(big, 16)                                    # four pages: two free ones and new's two
    assert manager.prefix_evictions == 2 and len(manager.prefix) == 2
    assert set(holder.tables[0]).isdisjoint(big.tables[0])
    with pytest.raises(KvCachePressure):
        manager.grow(holder, 9)                              # nothing free, nothing evictable
    manager.check()
    manager.release("big")
    assert manager.admit("again", new).length == 0           # new's pages are gone
    assert manager.admit("still", old).length == 8
    manager.check()


def test_clearing_the_prefix_cache_frees_what_no_request_holds():
    manager = prefix_manager()
    feed(manager, "gone", list(range(9))); manager.release("gone")
    live = feed(manager, "live", list(range(20, 29)))
    pool = manager.groups[0].pool
    assert len(manager.prefix) == 4 and pool.free == 3
    assert manager.clear_prefix() == 4 and len(manager.prefix) == 0
    assert pool.free == 5 and pool.reclaimable == 0 and [pool.holders(p) for p in live.tables[0]] == [1, 1, 1]
    manager.check()
    assert manager.admit("b", list(range(20, 29))).length == 0
    manager.grow(live, 13); manager.commit(live, 13, [1, 2, 3, 4])           # it goes on remembering from here
    assert len(manager.prefix) == 1
    manager.release("live"); manager.release("b")
    manager.check()


def test_unknown_tokens_stop_the_remembering_not_the_request():
    manager = prefix_manager()
    seq = manager.admit("a", [1, 2, 3, 4, 5])
    manager.grow(seq, 5); manager.commit(seq, 5, [1, 2, 3, 4, 5])
    manager.grow(seq, 9); manager.commit(seq, 9)             # decoded on the device: ids unknown here
    assert seq.tokens is None and len(manager.prefix) == 1
    manager.grow(seq, 13); manager.commit(seq, 13, [1, 1, 1, 1])
    assert len(manager.prefix) == 1
    manager.check()


def test_prefix_cache_is_off_where_pages_do_not_keep_every_token():
    windowed = CacheManager(plan_of(TINY_C), 4, 8, 2, prefix_cache=True)
    assert windowed.prefix is None and windowed.admit("a", [1, 2, 3, 4, 5, 6]).length == 0
    plan = [CacheEntryPlan(0, PagedKv(2, 16, None), 0, True), CacheEntryPlan(1, FixedState((4, 8)), 1, True)]
    assert CacheManager(plan, 4, 8, 2, prefix_cache=True).prefix is None


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10_000), page_size=st.sampled_from([1, 4, 8]), pages=st.integers(6, 30))
def test_random_orders_with_a_prefix_cache_share_only_what_is_the_same(seed, page_size, pages):
    """The pages' contents are modelled on the host: every cached token position holds a digest of the tokens up to
    it.  A request that takes over cached pages must find in them what it would have computed itself, and no request
    ever writes into a page that another holder can see."""
    rng = random.Random(seed)
    manager = CacheManager(plan_of(TINY_A), page_size, pages, max_requests=4, prefix_cache=True, model_key="m")
    pool = manager.groups[0].pool
    prompts = [[rng.randrange(3) for _ in range(rng.randrange(1, 40))] for _ in range(4)]
    contents = {}                                            # (page, offset) -> digest of the tokens up to there
    todo = {}                                                # live request -> tokens it will be fed
    counter = 0

    def digest(tokens, upto):
        return hash(tuple(tokens[:upto + 1]))

    for _ in range(300):
        action = rng.random()
        if action < 0.3 and manager.free_slots:
            name = f"r{counter}"
            counter += 1
            base = rng.choice(prompts)
            tokens = base[:rng.randrange(1, len(base) + 1)] + [rng.randrange(3) for _ in range(rng.randrange(0, 12))]
            seq = manager.admit(name, tokens if rng.random() < 0.9 else None)
            assert seq.length % page_size == 0 and seq.length < len(tokens)
            for position in range(seq.length):               # what it took over is what it would have computed
                page = seq.tables[0][position // page_size]
                assert contents[(page, position % page_size)] == digest(tokens, position)
            todo[name] = tokens
        elif action < 0.85 and todo:
            name = rng.choice(sorted(todo))
            seq, tokens = manager.live[name], todo[name]
            if seq.length == len(tokens):
                tokens.append(rng.randrange(3))              # decode one more
            portion = tokens[seq.length:seq.length + rng.choice([1, 1, 2, 3, 7, 16])]
            try:
                manager.grow(seq, seq.length + len(portion))
            except (KvCachePressure, KvCapacity):
                manager.check()
                continue
            for position in range(seq.length, seq.length + len(portion)):
                page = seq.tables[0][position // page_size]
                assert pool.holders(page) == 1               # nobody else sees the page that is written
                contents[(page, position % page_size)] = digest(tokens, position)
            manager.commit(seq, seq.length + len(portion), portion if rng.random() < 0.9 else None)
        elif todo:
            name = rng.choice(sorted(todo))
            manager.release(name)
            del todo[name]
        manager.check()
    for name in list(todo):
        manager.release(name)
    manager.check()
    assert pool.available == pool.count and manager.free_slots == 4
    assert pool.free + len(manager.prefix) == pool.count
