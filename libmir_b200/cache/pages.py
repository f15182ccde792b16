"""One pool of cache pages: ids 0 .. count-1, a FIFO free list, and a record of who holds what.

libmir's block manager (runtime/src/kv/cache/mod.rs:32-52) keeps a free VecDeque of block ids and a
reference count per block.  Here a page has exactly one holder (no prefix sharing), so the record is
a flag per page; giving back a page that is not held, or taking one that is, raises at once.
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
        self._held = [False] * count
        self.high_water = 0
        self.reused = 0            # pages handed out that had been held before
        self._ever_held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def take(self, n: int) -> List[int]:
        """n pages, oldest-freed first; the caller checks `free` before (all-or-nothing)."""
        if n > len(self._free):
            raise RuntimeError(f"PagePool.take({n}) with only {len(self._free)} free pages")
        out = []
        for _ in range(n):
            page = self._free.popleft()
            if self._held[page]:
                raise RuntimeError(f"page {page} was on the free list while held")
            self._held[page] = True
            if self._ever_held[page]:
                self.reused += 1
            self._ever_held[page] = True
            out.append(page)
        self.high_water = max(self.high_water, self.held)
        return out

    def give_back(self, pages: Iterable[int]) -> None:
        for page in pages:
            if not 0 <= page < self.count or not self._held[page]:
                raise RuntimeError(f"page {page} is given back but is not held")
            self._held[page] = False
            self._free.append(page)

    def check(self) -> None:
        """Every page is either free exactly once or held; raises if not."""
        seen = [0] * self.count
        for page in self._free:
            seen[page] += 1
        for page in range(self.count):
            if seen[page] + (1 if self._held[page] else 0) != 1:
                raise RuntimeError(f"page {page}: on the free list {seen[page]} times, held={self._held[page]}")
