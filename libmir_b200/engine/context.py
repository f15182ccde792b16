"""What a step hands to the parts: the packed rows' metadata on the device, and scratch memory.

Nothing here is specific to a mixer.  The packed-row description follows libmir's PagedPrefillBatch
(cuda/src/backend/kv/prefill_batch/mod.rs:82-139): per row of the batch (one request's portion)
query_starts, context length after the step, block table; per token its request row, absolute
position and cache slot.  A decoded token is a portion of one token (cuda/src/engine/model/generation/
graph.rs:112-121).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..parts.base import PartContext


class Arena:
    """Scratch memory of a step: a bump allocator over buffers that are kept between steps.

    `reset` starts a new step.  When a step needs more than the arena holds, another buffer is added
    (a device allocation) and kept, so steps of a size seen before allocate nothing; shapes replayed
    from a CUDA graph always find the addresses they were captured with because allocation order is
    deterministic.
    """

    ALIGN = 256

    def __init__(self, device: torch.device, chunk_bytes: int = 64 << 20):
        self.device = device
        self.chunk_bytes = chunk_bytes
        self.chunks: List[torch.Tensor] = []
        self.chunk = 0
        self.offset = 0
        self._views: dict = {}       # (chunk, offset, dtype, shape) -> (view, padded bytes): steps repeat their sizes

    def reset(self) -> None:
        self.chunk = 0
        self.offset = 0

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        key = (self.chunk, self.offset, dtype, shape)
        known = self._views.get(key)
        if known is not None:                       # the same request at the same place as in an earlier step
            self.offset += known[1]
            return known[0]
        view = self._alloc_new(shape, dtype)
        if self.chunk == key[0]:                    # (it fitted into the chunk it was asked in)
            if len(self._views) > 65536:
                self._views.clear()
            self._views[key] = (view, self.offset - key[1])
        return view

    def _alloc_new(self, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for dim in shape:
            count *= int(dim)
        nbytes = count * dtype.itemsize
        padded = -(-max(nbytes, 1) // self.ALIGN) * self.ALIGN
        while True:
            if self.chunk >= len(self.chunks):
                self.chunks.append(torch.empty(max(self.chunk_bytes, padded), dtype=torch.uint8, device=self.device))
            buffer = self.chunks[self.chunk]
            if self.offset + padded <= buffer.numel():
                view = buffer[self.offset:self.offset + nbytes].view(dtype).view(*shape)
                self.offset += padded
                return view
            self.chunk += 1
            self.offset = 0

    def bytes(self) -> int:
        return sum(chunk.numel() for chunk in self.chunks)


@dataclass
class GroupContext:
    """Per cache group: where each token's key/value goes and each row's block table."""

    block_table: torch.Tensor           # int32 [rows, width]; -1 where a page was released
    slot_mapping: torch.Tensor          # int32 [tokens]; page * page_size + position % page_size, -1 = no write
    table_width: int = 0


@dataclass
class StepContext(PartContext):
    num_tokens: int
    num_rows: int
    tokens: torch.Tensor                # int32 [T]
    positions: torch.Tensor             # int32 [T] absolute position of each token in its request
    row_of_token: torch.Tensor          # int32 [T]
    query_starts: torch.Tensor          # int32 [R + 1]
    context_lens: torch.Tensor          # int32 [R] tokens of the request cached after this step
    state_slots: torch.Tensor           # int32 [R] the request's fixed-size state slot
    groups: List[GroupContext]
    views: Dict[int, object]            # schedule entry -> CacheView
    arena: Arena
    dtype: torch.dtype
    # host copies, for launch geometry and for parts that walk requests on the host
    host_query_starts: Sequence[int] = ()
    host_start_positions: Sequence[int] = ()
    host_state_slots: Sequence[int] = ()
    max_context: int = 0
    max_portion: int = 0
    decode_only: bool = False
    # Rows are ordered with the single-token rows first: rows [0, single_rows) have one token each, and token r is
    # row r's; single_context is the longest context among them.
    single_rows: int = 0
    single_context: int = 0
    page_size: int = 0
    # (residual data_ptr, rows, sums-of-squares tensor, tiles, weighted rows, norm weight data_ptr) or None
    residual_stats: Optional[tuple] = None
    # The norm that will be applied to the residual right after the part that runs now has added into it (set by
    # the block), and the one that the next block in the schedule starts with (set by the model); None if unknown.
    upcoming_norm: Optional[object] = None
    norm_after_block: Optional[object] = None

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.arena.alloc(shape, dtype)

    def note_residual_stats(self, residual: torch.Tensor, sumsq: Optional[torch.Tensor], tiles: int,
                            weighted: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None) -> None:
        """Remember (or forget, with None) that `sumsq` holds the sums of squares of `residual` as it is now and
        `weighted` its rows times `norm_weight`.  Whoever changes the residual calls this; the norm with that
        weight may then be folded into the product that follows it."""
        if sumsq is None or weighted is None or norm_weight is None:
            self.residual_stats = None
        else:
            self.residual_stats = (residual.data_ptr(), residual.shape[0], sumsq, tiles, weighted,
                                   norm_weight.data_ptr())

    def stats_for(self, residual: torch.Tensor, norm_weight: torch.Tensor):
        stats = self.residual_stats
        if (stats is not None and stats[0] == residual.data_ptr() and stats[1] == residual.shape[0]
                and stats[5] == norm_weight.data_ptr()):
            return stats[2], stats[3], stats[4]
        return None

    def accumulate(self, x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor,
                   bias: Optional[torch.Tensor] = None) -> None:
        """residual += x . weight^T (+ bias).  If a foldable norm is known to follow (`upcoming_norm`) and the
        product can do it, it also leaves what that norm needs to be folded into the next product."""
        norm = self.upcoming_norm
        norm_weight = norm.weight if (norm is not None and norm.foldable) else None
        if (not kernels.FUSE_NORM_INTO_PRODUCT or norm_weight is None or self.dtype != torch.bfloat16
                or residual.shape[0] > kernels.few_rows_max()
                or norm_weight.numel() != residual.shape[1]):
            kernels.linear(x, weight, residual, bias, accumulate=True)
            self.residual_stats = None
            return
        tiles = kernels.sumsq_tiles(residual.shape[1])
        sumsq = self.alloc((tiles, kernels.NORM_STAT_STRIDE), torch.float32)
        weighted = self.alloc(tuple(residual.shape), torch.bfloat16)
        wrote = kernels.linear(x, weight, residual, bias, accumulate=True, sumsq_out=sumsq,
                               weighted_out=(weighted, norm_weight))
        self.note_residual_stats(residual, sumsq if wrote else None, tiles, weighted, norm_weight)

    def cache_view(self, entry: int):
        return self.views.get(entry)
