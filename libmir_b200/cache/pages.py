"""One pool of cache pages: ids 0 .. count-1, a FIFO free list, and a count of holders per page.

libmir's block manager (runtime/src/kv/cache/mod.rs:32-52,118-153) keeps a free VecDeque of block ids and a
reference count per block.  Here too: a page is free (no holder, on the free list) or held by one or more
holders.  Holders are requests (a page in a block table) and, when prefixes are cached, the prefix index, which
holds one reference of its own on every page it knows (`mark_cached`).  A cached page that only the index
holds is `reclaimable`: it counts as available and goes back to the free list when pages are needed
(`evict`).  Giving back a page that is not held, or taking one that is, raises at once.
"""

from __future__ import annotations

from collections import deque
from typing import Iterable, List


class PagePool:
    def __init__(self, count: int):
        if count <= 0:
            raise ValueError("a page pool needs at least one page")
        self.count = count
        self._free = deque(range(count))
        self._holders = [0] * count
        self._cached = [False] * count
        self.reclaimable = 0       # cached pages that only the prefix index holds
        self.high_water = 0
        self.reused = 0            # pages handed out that had been held before
        self._ever_held = [False] * count

    @property
    def free(self) -> int:
        """Pages on the free list right now."""
        return len(self._free)

    @property
    def available(self) -> int:
        """Pages a request can get: the free ones and those that only the prefix index holds."""
        return len(self._free) + self.reclaimable

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def holders(self, page: int) -> int:
        return self._holders[page]

    def is_cached(self, page: int) -> bool:
        return self._cached[page]

    def take(self, n: int) -> List[int]:
        """n pages, oldest-freed first; the caller checks `free` before (all-or-nothing)."""
        if n > len(self._free):
            raise RuntimeError(f"PagePool.take({n}) with only {len(self._free)} free pages")
        out = []
        for _ in range(n):
            page = self._free.popleft()
            if self._holders[page] != 0:
                raise RuntimeError(f"page {page} was on the free list while held")
            self._holders[page] = 1
            if self._ever_held[page]:
                self.reused += 1
            self._ever_held[page] = True
            out.append(page)
        self.high_water = max(self.high_water, self.held)
        return out

    def retain(self, page: int) -> None:
        """One more holder of a page that is held already (a request that shares a cached prefix)."""
        if not 0 <= page < self.count or self._holders[page] == 0:
            raise RuntimeError(f"page {page} is retained but is not held")
        if self._cached[page] and self._holders[page] == 1:
            self.reclaimable -= 1
        self._holders[page] += 1

    def give_back(self, pages: Iterable[int]) -> None:
        """One holder less for each page; a page without holders goes to the free list."""
        for page in pages:
            if not 0 <= page < self.count or self._holders[page] == 0:
                raise RuntimeError(f"page {page} is given back but is not held")
            if self._cached[page] and self._holders[page] == 1:
                raise RuntimeError(f"page {page} is given back but is not held (only the prefix index holds it)")
            self._holders[page] -= 1
            if self._holders[page] == 0:
                self._free.append(page)
            elif self._cached[page] and self._holders[page] == 1:
                self.reclaimable += 1

    def mark_cached(self, page: int) -> None:
        """The prefix index takes a reference of its own on a held page."""
        if not 0 <= page < self.count or self._holders[page] == 0 or self._cached[page]:
            raise RuntimeError(f"page {page} cannot be cached (holders {self._holders[page]}, cached {self._cached[page]})")
        self._holders[page] += 1
        self._cached[page] = True

    def evict(self, page: int) -> None:
        """The prefix index drops a page that nobody else holds: it is free again."""
        if not 0 <= page < self.count or not self._cached[page] or self._holders[page] != 1:
            raise RuntimeError(f"page {page} cannot be evicted (holders {self._holders[page]}, cached {self._cached[page]})")
        self.forget(page)

    def forget(self, page: int) -> None:
        """The prefix index drops its reference; the page is free again unless requests still hold it."""
        if not 0 <= page < self.count or not self._cached[page]:
            raise RuntimeError(f"page {page} is not cached")
        self._cached[page] = False
        self._holders[page] -= 1
        if self._holders[page] == 0:
            self.reclaimable -= 1
            self._free.append(page)

    def check(self) -> None:
        """Every page is either free exactly once or held; the reclaimable count is what the flags say."""
        seen = [0] * self.count
        for page in self._free:
            seen[page] += 1
        for page in range(self.count):
            if seen[page] + (1 if self._holders[page] > 0 else 0) != 1:
                raise RuntimeError(f"page {page}: on the free list {seen[page]} times, holders={self._holders[page]}")
            if self._cached[page] and self._holders[page] == 0:
                raise RuntimeError(f"page {page} is cached but has no holder")
        counted = sum(1 for page in range(self.count) if self._cached[page] and self._holders[page] == 1)
        if counted != self.reclaimable:
            raise RuntimeError(f"{counted} pages are reclaimable, the pool counts {self.reclaimable}")
