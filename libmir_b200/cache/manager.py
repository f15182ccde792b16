"""The cache manager: pages for keys and values, block tables per request, state slots per request.

Host-side bookkeeping only; the device memory the ids refer to is in cache/storage.py, so the manager
can be tested without a GPU.

Groups.  Schedule entries (layer runs) with the same needs share a group: (kv_heads, head_dim, window)
for paged keys/values.  Each group has its own PagePool and each request has one block table per
group; one page id addresses the same slot range in every entry of the group, as libmir's block id
addresses every layer (runtime/src/kv/write.rs:7-10).  A group without a window keeps every token; a
group with a window gives pages back as soon as no later query can see them.

Lengths.  `length` is the number of tokens whose keys are in the cache.  A step first `grow`s the
request to length + count (pages for the new tokens, all groups or none), runs, then `commit`s the new
length, which is also when windowed groups release what fell out of the window.

Table layout.  A request's table for a group is indexed by position // page_size for all positions
from 0; entries whose page was released hold -1.

What is given back when: `release` returns every page and the state slot (request finished, cancelled
or preempted); `commit` returns pages a window has passed; a failed `grow` takes nothing.
libmir: runtime/src/kv/state/mod.rs:96-116 (decode append allocates exactly when length == blocks *
block_size), kv/state/prefill.rs:45-118 (all-or-nothing with rollback), kv/cache/pressure.rs:5-33 and
runtime/src/error.rs:24-27 (KvCapacity vs KvCachePressure).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..config.spec import FixedState, PagedKv
from ..errors import KvCachePressure, KvCapacity, NoFreeSlot
from .pages import PagePool
from .prefix import PrefixIndex, page_key


@dataclass
class GroupInfo:
    """One group of schedule entries with the same paged needs."""

    index: int
    requirement: PagedKv
    entries: List[int]             # schedule entries that own storage in this group
    pool: PagePool

    @property
    def window(self) -> Optional[int]:
        return self.requirement.window


@dataclass
class Sequence_:
    """One live request's hold on the cache."""

    request_id: object
    slot: int
    length: int = 0                                   # tokens cached (committed)
    reserved: int = 0                                 # length pages have been allocated for
    tables: List[List[int]] = field(default_factory=list)      # per group: page id or -1 per block
    first_live: List[int] = field(default_factory=list)        # per group: first block not yet released
    serial: int = 0                                   # unique over the manager's life (ids and slots are reused)
    tokens: Optional[List[int]] = None                # with a prefix cache: the ids of the cached tokens (None: unknown)
    keys: List[bytes] = field(default_factory=list)   # with a prefix cache: the key of every full page so far
    prefix_tokens: int = 0                            # tokens this request found cached when it was admitted


class CacheManager:
    def __init__(self, plan: Sequence, page_size: int, num_pages: int, max_requests: int,
                 prefix_cache: bool = False, model_key: str = ""):
        """`plan` is DecoderModel.cache_plan(): one CacheEntryPlan per schedule entry.  `prefix_cache`: full pages
        are remembered by the tokens they hold (cache/prefix.py) and shared by requests that start alike; it takes
        effect where every cached token stays in its page for the request's life and nothing else is kept per
        request: one group of pages without a window, no fixed-size state."""
        if page_size <= 0 or max_requests <= 0:
            raise ValueError("page_size and max_requests must be greater than zero")
        self.page_size = page_size
        self.max_requests = max_requests
        self.groups: List[GroupInfo] = []
        self.entry_group: Dict[int, int] = {}          # schedule entry -> group (paged entries)
        self.entry_local: Dict[int, int] = {}          # schedule entry -> index of its storage within the group
        self.state_entries: Dict[int, FixedState] = {} # schedule entry -> fixed state it owns
        by_requirement: Dict[PagedKv, GroupInfo] = {}
        for item in plan:
            if isinstance(item.requirement, PagedKv):
                if item.source == item.entry:
                    group = by_requirement.get(item.requirement)
                    if group is None:
                        group = GroupInfo(len(self.groups), item.requirement, [], PagePool(num_pages))
                        by_requirement[item.requirement] = group
                        self.groups.append(group)
                    self.entry_local[item.entry] = len(group.entries)
                    group.entries.append(item.entry)
                    self.entry_group[item.entry] = group.index
            elif isinstance(item.requirement, FixedState) and item.source == item.entry:
                self.state_entries[item.entry] = item.requirement
        for item in plan:                              # readers of another entry's cache
            if item.source != item.entry and isinstance(item.requirement, PagedKv):
                self.entry_group[item.entry] = self.entry_group[item.source]
                self.entry_local[item.entry] = self.entry_local[item.source]
        capable = len(self.groups) == 1 and self.groups[0].window is None and not self.state_entries
        self.prefix: Optional[PrefixIndex] = PrefixIndex() if prefix_cache and capable else None
        self._model_key = model_key.encode()
        self.prefix_hit_tokens = 0                     # tokens that admitted requests found cached
        self.prefix_evictions = 0
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._serial = 0                               # counts admissions: ids and slots are reused, serials are not
        self.live: Dict[object, Sequence_] = {}
        self.fresh_slots: List[int] = []               # slots handed out since the device last zeroed state

    # -- admission ---------------------------------------------------------------
    def admit(self, request_id, tokens: Optional[Sequence[int]] = None) -> Sequence_:
        """A new live request.  With a prefix cache and the tokens it will be fed: the longest run of full pages that
        hold exactly its first tokens is taken over (shared, not copied), `length` starts behind them, and at least
        one token is left to compute."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._serial += 1
        sequence = Sequence_(request_id, slot, tables=[[] for _ in self.groups], first_live=[0] * len(self.groups),
                             serial=self._serial)
        self.live[request_id] = sequence
        self.fresh_slots.append(slot)
        if self.prefix is not None:
            sequence.tokens = []
            if tokens is not None:
                pool, table, page = self.groups[0].pool, sequence.tables[0], self.page_size
                parent = None
                for block in range((len(tokens) - 1) // page):
                    key = page_key(self._model_key, parent, tokens[block * page:(block + 1) * page])
                    cached = self.prefix.get(key)
                    if cached is None:
                        break
                    pool.retain(cached)
                    table.append(cached)
                    sequence.keys.append(key)
                    parent = key
                cached_tokens = len(table) * page
                sequence.tokens = [int(t) for t in tokens[:cached_tokens]]
                sequence.length = sequence.reserved = sequence.prefix_tokens = cached_tokens
                self.prefix_hit_tokens += cached_tokens
        return sequence

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # -- pages ---------------------------------------------------------------------
    def _blocks_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_needed(self, sequence: Sequence_, new_length: int) -> List[int]:
        """Per group, how many more pages the request needs to hold tokens up to new_length."""
        return [max(0, self._blocks_for(new_length) - len(table)) for table in sequence.tables]

    def peak_pages(self, length: int, group: GroupInfo, portion: int) -> int:
        """Most pages of `group` that a request of `length` tokens holds at once when it is fed in
        portions of at most `portion` tokens."""
        if group.window is None:
            return self._blocks_for(length)
        span = min(length, group.window + portion)
        return min(self._blocks_for(length), span // self.page_size + 2)

    def can_grow(self, sequence: Sequence_, new_length: int, spare: Optional[List[int]] = None) -> bool:
        need = self.pages_needed(sequence, new_length)
        spare = spare or [0] * len(self.groups)
        return all(n <= g.pool.available - s for n, g, s in zip(need, self.groups, spare))

    def grow(self, sequence: Sequence_, new_length: int) -> None:
        """Allocate pages so that tokens up to new_length fit, in every group or in none."""
        if new_length < sequence.length:
            raise ValueError("a request cannot shrink")
        need = self.pages_needed(sequence, new_length)
        for n, group, table, first in zip(need, self.groups, sequence.tables, sequence.first_live):
            if n == 0:
                continue
            live_now = len(table) - first                    # the blocks before `first` were given back
            if live_now + n > group.pool.count:
                raise KvCapacity(live_now + n, group.pool.count, f"group {group.index}")
            if n > group.pool.available:
                raise KvCachePressure(n, group.pool.available, f"group {group.index}")
        for n, group, table in zip(need, self.groups, sequence.tables):
            self._reclaim(group, n)
            table.extend(group.pool.take(n))
        sequence.reserved = max(sequence.reserved, new_length)

    def _reclaim(self, group: GroupInfo, n: int) -> None:
        """Make n pages free by dropping cached prefixes that no request holds, the least recently used first."""
        if n <= group.pool.free or self.prefix is None:
            return
        for key, page in self.prefix.oldest_first():
            if group.pool.holders(page) == 1:
                self.prefix.remove(key)
                group.pool.evict(page)
                self.prefix_evictions += 1
                if n <= group.pool.free:
                    return

    def clear_prefix(self) -> int:
        """Forget every cached prefix (libmir: Engine::clear_prefix_cache, src/engine/mod.rs:187-200).  Pages that live
        requests hold stay theirs; the rest are free again.  Returns how many pages were forgotten."""
        if self.prefix is None:
            return 0
        pool, dropped = self.groups[0].pool, 0
        for key, page in self.prefix.oldest_first():
            self.prefix.remove(key)
            pool.forget(page)
            dropped += 1
        return dropped

    def commit(self, sequence: Sequence_, new_length: int, tokens: Optional[Sequence[int]] = None) -> None:
        """The tokens up to new_length are now cached; release what windows have passed.  `tokens`: the ids that were
        just cached (with a prefix cache, the pages they complete are remembered; without them the request's later
        pages are not)."""
        if self.groups and new_length > len(sequence.tables[0]) * self.page_size:
            raise ValueError("commit beyond the pages that were grown")
        if self.prefix is not None and sequence.tokens is not None:
            if tokens is None or len(sequence.tokens) + len(tokens) != new_length:
                sequence.tokens = None                         # what the pages hold from here on is not known
            else:
                sequence.tokens.extend(int(t) for t in tokens)
                pool, table, page = self.groups[0].pool, sequence.tables[0], self.page_size
                for block in range(len(sequence.keys), new_length // page):
                    parent = sequence.keys[-1] if sequence.keys else None
                    key = page_key(self._model_key, parent, sequence.tokens[block * page:(block + 1) * page])
                    sequence.keys.append(key)
                    if self.prefix.get(key, touch=False) is None and not pool.is_cached(table[block]):
                        self.prefix.insert(key, table[block])
                        pool.mark_cached(table[block])
        sequence.length = new_length
        for index, group in enumerate(self.groups):
            if group.window is None:
                continue
            # a later query at position p >= new_length sees keys j > p - window >= new_length - window
            dead_keys = new_length - group.window + 1       # keys < dead_keys are never read again
            dead_blocks = max(0, dead_keys // self.page_size)
            table = sequence.tables[index]
            first = sequence.first_live[index]
            if dead_blocks > first:
                group.pool.give_back(page for page in table[first:dead_blocks] if page >= 0)
                for block in range(first, dead_blocks):
                    table[block] = -1
                sequence.first_live[index] = dead_blocks

    def release(self, request_id) -> None:
        """Give back every page and the slot of a request."""
        sequence = self.live.pop(request_id, None)
        if sequence is None:
            raise KeyError(f"request {request_id!r} is not live")
        for group, table in zip(self.groups, sequence.tables):
            group.pool.give_back(page for page in table if page >= 0)
            table.clear()
        self._free_slots.append(sequence.slot)

    def take_fresh_slots(self) -> List[int]:
        """Slots admitted since the last call: their fixed-size state must start at zero."""
        fresh, self.fresh_slots = self.fresh_slots, []
        return fresh

    # -- reports -------------------------------------------------------------------
    def stats(self) -> dict:
        return {
            "page_size": self.page_size,
            "live_requests": len(self.live),
            "free_slots": len(self._free_slots),
            "groups": [{"window": g.window, "kv_heads": g.requirement.kv_heads, "head_dim": g.requirement.head_dim,
                        "value_head_dim": g.requirement.value_dim,
                        "entries": len(g.entries), "pages": g.pool.count, "free": g.pool.available,
                        "high_water": g.pool.high_water, "reused": g.pool.reused} for g in self.groups],
            "cached_prefix_pages": len(self.prefix) if self.prefix is not None else 0,
            "prefix_hit_tokens": self.prefix_hit_tokens, "prefix_evictions": self.prefix_evictions,
        }

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost or held twice."""
        for index, group in enumerate(self.groups):
            group.pool.check()
            holders: Dict[int, list] = {}
            for sequence in self.live.values():
                for page in sequence.tables[index]:
                    if page < 0:
                        continue
                    holders.setdefault(page, []).append(sequence.request_id)
            cached = set(self.prefix.pages()) if self.prefix is not None and index == 0 else set()
            if self.prefix is not None and len(cached) != len(self.prefix):
                raise RuntimeError("a page is in the prefix index under two keys")
            for page, who in holders.items():
                if len(who) > 1 and page not in cached:
                    raise RuntimeError(f"page {page} of group {index} is held by {who!r} and is no cached prefix")
            for page in set(holders) | cached:
                expected = len(holders.get(page, [])) + (1 if page in cached else 0)
                if group.pool.holders(page) != expected or group.pool.is_cached(page) != (page in cached):
                    raise RuntimeError(f"page {page} of group {index}: the pool counts {group.pool.holders(page)} "
                                       f"holders, tables and index hold it {expected} times")
            if len(set(holders) | cached) != group.pool.held:
                raise RuntimeError(f"group {index}: the pool says {group.pool.held} pages are held, tables and index "
                                   f"hold {len(set(holders) | cached)}")
        slots = [s.slot for s in self.live.values()] + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise RuntimeError(f"state slots are lost or held twice: {sorted(slots)}")
