"""Full pages of prompts (and of what was generated after them) remembered by what they hold, so that a request
that starts with the same tokens takes them instead of computing them again.

A page's key is a hash of the model's key, the key of the page before it and the page's token ids: a chain, so a
page is found only behind the very prefix it was computed behind (libmir: BlockHash::from_tokens,
runtime/src/kv/block.rs:48-58, blake3 there, blake2b here).  The index keeps its entries in order of use, oldest
first; the cache manager evicts from that end the pages that nobody but the index holds when requests need pages
(runtime/src/kv/prefix.rs:20-121, kv/cache/pressure.rs:5-33).
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from typing import Iterable, Iterator, Optional, Sequence, Tuple


def page_key(model_key: bytes, parent: Optional[bytes], tokens: Sequence[int]) -> bytes:
    digest = hashlib.blake2b(digest_size=16)
    digest.update(model_key)
    if parent is not None:
        digest.update(parent)
    digest.update(struct.pack(f"<{len(tokens)}I", *tokens))
    return digest.digest()


class PrefixIndex:
    def __init__(self):
        self._pages: "OrderedDict[bytes, int]" = OrderedDict()    # key -> page, oldest use first

    def __len__(self) -> int:
        return len(self._pages)

    def get(self, key: bytes, touch: bool = True) -> Optional[int]:
        page = self._pages.get(key)
        if page is not None and touch:
            self._pages.move_to_end(key)
        return page

    def insert(self, key: bytes, page: int) -> None:
        if key in self._pages:
            raise RuntimeError("the prefix index already has this key")
        self._pages[key] = page

    def remove(self, key: bytes) -> int:
        return self._pages.pop(key)

    def oldest_first(self) -> Iterator[Tuple[bytes, int]]:
        return iter(list(self._pages.items()))

    def pages(self) -> Iterable[int]:
        return self._pages.values()
