"""Device memory behind the cache manager's ids.

Per group one allocation for the keys, [entries, pages * page_size, kv_heads, head_dim], and one for the
values, [entries, pages * page_size, kv_heads, value_dim], in the engine's dtype, so a page id is the same
offset in every layer run of the group (libmir keeps one K and one V buffer per layer with widths of their
own, cuda/src/backend/kv/storage/mod.rs:17-25,47-89; token-major NHD layout as there).
Per schedule entry with fixed-size state: [max_requests, *shape], one record per request slot.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .manager import CacheManager

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class CacheView:
    """What one schedule entry's mixer gets."""

    group: Optional[int] = None            # index of the paged group, None if the entry has no pages
    k_pages: Optional[torch.Tensor] = None  # [pages * page_size, kv_heads, head_dim]
    v_pages: Optional[torch.Tensor] = None
    page_size: int = 0
    writes: bool = True                     # False: the entry reads another entry's cache
    state: Optional[torch.Tensor] = None    # [max_requests, *shape] fixed-size state, indexed by slot


class CacheStorage:
    def __init__(self, manager: CacheManager, plan, dtype: torch.dtype, device: torch.device):
        self.manager = manager
        self.key_buffers, self.value_buffers = [], []
        for group in manager.groups:
            r = group.requirement
            rows = group.pool.count * manager.page_size
            self.key_buffers.append(torch.zeros((len(group.entries), rows, r.kv_heads, r.head_dim), dtype=dtype,
                                                device=device))
            self.value_buffers.append(torch.zeros((len(group.entries), rows, r.kv_heads, r.value_dim), dtype=dtype,
                                                  device=device))
        self.buffers = self.key_buffers + self.value_buffers
        self.states: Dict[int, torch.Tensor] = {}
        for entry, requirement in manager.state_entries.items():
            self.states[entry] = torch.zeros((manager.max_requests, *requirement.shape),
                                             dtype=_DTYPES[requirement.dtype], device=device)
        self.views: Dict[int, CacheView] = {}
        for item in plan:
            view = CacheView(writes=item.source == item.entry)
            if item.entry in manager.entry_group:
                group = manager.entry_group[item.entry]
                local = manager.entry_local[item.entry]
                view.group = group
                view.k_pages = self.key_buffers[group][local]
                view.v_pages = self.value_buffers[group][local]
                view.page_size = manager.page_size
            if item.source in self.states:
                view.state = self.states[item.source]
            self.views[item.entry] = view

    def zero_slots(self, slots) -> None:
        """Fixed-size state of newly admitted requests starts at zero."""
        if not slots or not self.states:
            return
        index = torch.tensor(slots, dtype=torch.long, device=next(iter(self.states.values())).device)
        for state in self.states.values():
            state.index_fill_(0, index, 0)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers) + \
            sum(s.numel() * s.element_size() for s in self.states.values())
