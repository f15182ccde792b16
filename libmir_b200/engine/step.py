"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

One path for every mix: portions of prompts beside single decoded tokens, cut anywhere.  A step runs
only the tokens it is given, reads everything older from the cache, and returns 32-bit logits at the
requested places.  libmir's equivalent is CudaEngine::execute_generation_step ->
CudaMoeModelSession::prefill_packed_chunk + finish_packed_prefill_rows
(cuda/src/engine/execution/step.rs:14-88, cuda/src/backend/model/session/prefill/packed.rs:23-89,
output.rs:112-178), which returns only last-position results; here any position may be asked for.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage
from ..errors import KernelError, KvCachePressure, KvCapacity, SchedulerError
from .context import Arena, GroupContext, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the local places whose logits are wanted."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


class DecodeTimings:
    """What libmir attaches to the outputs of a decode step while decode profiling is on (runtime DecodeTimings,
    cuda/src/engine/profile.rs:7-46): how long the step took on the host (taking pages, the upload, the launches) and
    on the device (between two events on the step's stream), and how many rows it had."""

    def __init__(self, backend_execution: float, batch_rows: int, started: torch.cuda.Event, stopped: torch.cuda.Event):
        self.backend_execution = backend_execution      # seconds on the host
        self.batch_rows = batch_rows
        self._events = (started, stopped)
        self._device: Optional[float] = None

    @property
    def device_execution(self) -> float:
        """Seconds on the device (waits for the step to be over the first time it is asked for)."""
        if self._device is None:
            self._events[1].synchronize()
            self._device = self._events[0].elapsed_time(self._events[1]) / 1e3
        return self._device

    def as_dict(self) -> dict:
        return {"backend_execution": self.backend_execution, "device_execution": self.device_execution,
                "batch_rows": self.batch_rows}


@dataclass
class StepResult:
    logits: Optional[torch.Tensor]          # float32 [wanted, vocab] on the device; valid until the next step
    rows: List[tuple]                       # (request_id, local index) for each logits row, in order
    num_tokens: int = 0
    tokens: Optional[torch.Tensor] = None   # int32 [wanted] sampled tokens on the device, if samplers were given
    timings: Optional[DecodeTimings] = None  # of a decode step, while decode profiling is on


class StepRunner:
    """Owns the device state of one loaded model: cache storage, scratch, staging buffers."""

    def __init__(self, model, manager: CacheManager, storage: CacheStorage, device: torch.device,
                 decode_graphs: bool = False):
        self.model = model
        self.manager = manager
        self.storage = storage
        self.device = device
        self.decode_graphs = decode_graphs
        self.profile_decode = False          # Model.set_profile_decode
        self.decode_timings: List[DecodeTimings] = []   # of the profiled decode steps, oldest first (at most 4,096)
        self._graphs = None
        self._graphs_usable = False
        self.sampler = None
        if storage is not None:
            from ..sampling.sampler import DeviceSampler
            self.sampler = DeviceSampler(device, model.spec.vocab_size)
        self.arena = Arena(device)
        self._staging: List[Optional[torch.Tensor]] = [None, None]
        self._staging_events: List[Optional[torch.cuda.Event]] = [None, None]
        self._device_meta: Optional[torch.Tensor] = None
        self._flip = 0
        self.steps = 0
        self.tokens_run = 0
        # After a captured decode step: (request ids, their sequences, the graph, the result's row keys, the samplers'
        # settings or None if all were greedy), so that the next step of the same requests, if none of them needs a
        # page, skips everything that cannot have changed (`_step_again`).  None after any other step.
        self._again = None
        self.steps_again = 0

    # -- metadata ------------------------------------------------------------------
    def _stage(self, arrays: List[np.ndarray]) -> List[torch.Tensor]:
        """Copy int32 arrays to the device through one pinned buffer and one transfer."""
        sizes = [a.size for a in arrays]
        offsets, total = [], 0
        for size in sizes:
            offsets.append(total)
            total += -(-max(size, 1) // 4) * 4          # keep every array 16-byte aligned
        self._flip ^= 1
        staging = self._staging[self._flip]
        if staging is None or staging.numel() < total:
            staging = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True)
            self._staging[self._flip] = staging
            self._staging_events[self._flip] = None
        event = self._staging_events[self._flip]
        if event is not None:
            event.synchronize()
        if self._device_meta is None or self._device_meta.numel() < total:
            self._device_meta = torch.empty(max(total, 4096), dtype=torch.int32, device=self.device)
        host = staging.numpy()
        for array, offset in zip(arrays, offsets):
            host[offset:offset + array.size] = array.reshape(-1)
        self._device_meta[:total].copy_(staging[:total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._staging_events[self._flip] = event
        return [self._device_meta[offset:offset + size] for offset, size in zip(offsets, sizes)]

    def build_context(self, entries: Sequence[StepEntry], sequences) -> tuple:
        manager = self.manager
        page = manager.page_size
        # Rows are packed with the single-token rows first (a stable order otherwise), so that a mixer can run
        # them as a batch of decoded tokens beside the prompt portions; what is wanted keeps the entries' order.
        given = list(entries)
        order = sorted(range(len(given)), key=lambda index: len(given[index].tokens) != 1)
        entries = [given[index] for index in order]
        sequences = [sequences[index] for index in order]
        counts = [len(e.tokens) for e in entries]
        total = sum(counts)
        rows = len(entries)
        single_rows = sum(1 for c in counts if c == 1)
        tokens = np.empty(total, dtype=np.int32)
        positions = np.empty(total, dtype=np.int32)
        row_of_token = np.empty(total, dtype=np.int32)
        query_starts = np.zeros(rows + 1, dtype=np.int32)
        context_lens = np.empty(rows, dtype=np.int32)
        state_slots = np.empty(rows, dtype=np.int32)
        wanted: dict = {}
        vocab = self.model.spec.vocab_size
        cursor = 0
        for r, (entry, seq, count) in enumerate(zip(entries, sequences, counts)):
            ids = np.asarray(entry.tokens, dtype=np.int64)
            if ids.size and (ids.min() < 0 or ids.max() >= vocab):
                raise SchedulerError(f"request {entry.request_id!r}: token id outside [0, {vocab})")
            tokens[cursor:cursor + count] = ids
            positions[cursor:cursor + count] = np.arange(seq.length, seq.length + count, dtype=np.int32)
            row_of_token[cursor:cursor + count] = r
            query_starts[r + 1] = cursor + count
            context_lens[r] = seq.length + count
            state_slots[r] = seq.slot
            for local in entry.want:
                if not 0 <= local < count:
                    raise SchedulerError(f"request {entry.request_id!r}: wanted place {local} is outside its "
                                         f"{count} tokens")
            wanted[order[r]] = [(cursor + local, (entry.request_id, local)) for local in entry.want]
            cursor += count
        want_rows: List[int] = []
        want_keys: List[tuple] = []
        for index in range(rows):                          # in the order the entries were given
            for packed_row, key in wanted[index]:
                want_rows.append(packed_row)
                want_keys.append(key)
        arrays = [tokens, positions, row_of_token, query_starts, context_lens, state_slots,
                  np.asarray(want_rows, dtype=np.int32)]
        widths = []
        for g, group in enumerate(manager.groups):
            width = max(1, max(len(seq.tables[g]) for seq in sequences))
            widths.append(width)
            table = np.full((rows, width), -1, dtype=np.int32)
            slots = np.empty(total, dtype=np.int32)
            for r, seq in enumerate(sequences):
                blocks = seq.tables[g]
                table[r, :len(blocks)] = blocks
                begin, end = query_starts[r], query_starts[r + 1]
                pos = positions[begin:end]
                pages = table[r, pos // page]
                slots[begin:end] = np.where(pages >= 0, pages * page + pos % page, -1)
            arrays += [table, slots]
        staged = self._stage(arrays)
        groups = []
        for g, width in enumerate(widths):
            groups.append(GroupContext(block_table=staged[7 + 2 * g].view(rows, width),
                                       slot_mapping=staged[8 + 2 * g], table_width=width))
        ctx = StepContext(
            num_tokens=total, num_rows=rows, tokens=staged[0], positions=staged[1], row_of_token=staged[2],
            query_starts=staged[3], context_lens=staged[4], state_slots=staged[5], groups=groups,
            views=self.storage.views, arena=self.arena, dtype=self.model.env.dtype,
            host_query_starts=query_starts.tolist(), host_start_positions=[seq.length for seq in sequences],
            host_state_slots=state_slots.tolist(), max_context=int(context_lens.max()) if rows else 0,
            max_portion=max(counts) if counts else 0, decode_only=all(c == 1 for c in counts),
            single_rows=single_rows, single_context=int(context_lens[:single_rows].max()) if single_rows else 0,
            page_size=page)
        return ctx, staged[6], want_keys

    # -- the step ----------------------------------------------------------------------
    def reserve(self, entries: Sequence[StepEntry]):
        """Host side of a step: check the batch and take the pages it needs, all or none.

        Raises KvCapacity when one request alone exceeds a pool, KvCachePressure when the pages are not
        free right now (nothing is taken in either case)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        manager = self.manager
        seen = set()
        sequences = []
        for entry in entries:
            if entry.request_id in seen:
                raise SchedulerError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            seq = manager.live.get(entry.request_id)
            if seq is None:
                raise SchedulerError(f"request {entry.request_id!r} is not live: admit it first")
            sequences.append(seq)
        limit = self.model.spec.max_positions
        for entry, seq in zip(entries, sequences):
            if seq.length + len(entry.tokens) > limit:
                raise SchedulerError(f"request {entry.request_id!r} would reach {seq.length + len(entry.tokens)} "
                                     f"tokens, max_position_embeddings is {limit}")
        needs = [manager.pages_needed(seq, seq.length + len(e.tokens)) for e, seq in zip(entries, sequences)]
        for g, group in enumerate(manager.groups):
            total_need = sum(n[g] for n in needs)
            if total_need <= group.pool.available:
                continue
            for need, seq in zip(needs, sequences):     # a request too large for the whole pool is a hard error
                alone = sum(1 for p in seq.tables[g] if p >= 0) + need[g]
                if alone > group.pool.count:
                    raise KvCapacity(alone, group.pool.count, f"group {g}")
            raise KvCachePressure(total_need, group.pool.available, f"group {g}")
        for entry, seq in zip(entries, sequences):
            manager.grow(seq, seq.length + len(entry.tokens))
        return entries, sequences

    def _graph_eligible(self, entries, samplers) -> bool:
        if not self.decode_graphs or samplers is None or len(samplers) != len(entries):
            return False
        if any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return False
        if any(s.repetition_penalty > 1.0 for s in samplers):
            return False
        if self._graphs is None:
            from .decode_graph import DecodeGraphs
            self._graphs = DecodeGraphs(self)
            self._graphs_usable = self._graphs.usable()
        return self._graphs_usable

    def _options(self, samplers) -> Optional[np.ndarray]:
        if all(s.greedy for s in samplers):
            return None
        from .. import kernels
        options = np.zeros(len(samplers), dtype=kernels.SAMPLE_OPTIONS)
        for r, s in enumerate(samplers):
            options[r] = (s.next_draw(), s.temperature, s.top_p, s.top_k, 0)
        return options

    def execute(self, entries: Sequence[StepEntry], sequences, samplers=None) -> StepResult:
        """Device side of a step: run the tokens from the cache, return logits at the wanted places
        and, when `samplers` has one sampler per wanted row, the sampled tokens."""
        self.storage.zero_slots(self.manager.take_fresh_slots())
        if self._graph_eligible(entries, samplers):
            graph = self._graphs.get(len(entries), sequences, 1, any(s.ranked for s in samplers))
            options = self._options(samplers)
            vocab = self.model.spec.vocab_size
            for entry in entries:
                if not 0 <= entry.tokens[0] < vocab:
                    raise SchedulerError(f"request {entry.request_id!r}: token id outside [0, {vocab})")
            graph.load([e.tokens[0] for e in entries], sequences, options)
            graph.replay()
            rows = len(entries)
            keys = [(e.request_id, 0) for e in entries]
            manager = self.manager
            if manager.prefix is None and len(manager.groups) == 1 and manager.groups[0].window is None:
                settings = None if options is None else [(s.temperature, s.top_p, s.top_k, s.repetition_penalty)
                                                         for s in samplers]
                self._again = ([e.request_id for e in entries], list(sequences), graph, keys, settings)
            return StepResult(graph.logits[:rows], keys, rows, graph.sampled[:rows])
        self.arena.reset()
        ctx, want_rows, want_keys = self.build_context(entries, sequences)
        residual = self.model.forward(ctx)
        candidates = None
        if samplers is not None and want_keys:
            from .. import kernels
            candidates = kernels.HeadCandidates.allocate(ctx.alloc, len(want_keys), self.model.spec.vocab_size)
        logits = self.model.logits(ctx, residual, want_rows, candidates=candidates) if want_keys else None
        tokens = None
        if samplers is not None and logits is not None:
            tokens = self.sampler.sample(logits, samplers, candidates)
        return StepResult(logits, want_keys, ctx.num_tokens, tokens)

    def commit(self, entries: Sequence[StepEntry], sequences) -> None:
        for entry, seq in zip(entries, sequences):
            self.manager.commit(seq, seq.length + len(entry.tokens), entry.tokens)

    def _step_again(self, entries: Sequence[StepEntry], samplers) -> Optional[StepResult]:
        """The step after a captured decode step of the same requests in the same order with the same sampling settings,
        each of which has room in its last page: the block tables, slots and sampling records on the device are as
        they must be, so only tokens, positions and draws are uploaded, the same graph is replayed and the lengths
        move on by one.  None if any of
        this does not hold; the ordinary path then runs (and says what is wrong, if something is)."""
        ids, sequences, graph, keys, settings = self._again
        if samplers is None or len(entries) != len(ids) or len(samplers) != len(ids):
            return None
        live, limit, vocab = self.manager.live, self.model.spec.max_positions, self.model.spec.vocab_size
        capacity = self.manager.page_size
        tokens = []
        for entry, rid, seq in zip(entries, ids, sequences):
            if entry.request_id != rid or len(entry.tokens) != 1 or len(entry.want) != 1 or entry.want[0] != 0 \
                    or live.get(rid) is not seq or seq.length >= len(seq.tables[0]) * capacity or seq.length >= limit \
                    or not 0 <= entry.tokens[0] < vocab:
                return None
            tokens.append(entry.tokens[0])
        if self.manager.fresh_slots:
            return None
        draws = None
        if settings is None:                                   # the rows were greedy: they must still be
            if any(not s.greedy or s.repetition_penalty > 1.0 for s in samplers):
                return None
        else:                                                  # the sampling records on the device but for the draws
            if any((s.temperature, s.top_p, s.top_k, s.repetition_penalty) != known
                   for s, known in zip(samplers, settings)):
                return None
            draws = [s.next_draw() for s in samplers]          # (one per row, as the ordinary path takes them)
        graph.load_again(tokens, sequences, draws)
        graph.replay()
        for seq in sequences:                                  # (no window to release pages, no prefix to remember)
            seq.length += 1
            seq.reserved = max(seq.reserved, seq.length)
        rows = len(ids)
        self.steps += 1
        self.steps_again += 1
        self.tokens_run += rows
        return StepResult(graph.logits[:rows], keys, rows, graph.sampled[:rows])

    def step(self, entries: Sequence[StepEntry], samplers=None) -> StepResult:
        """Run one batch: reserve pages, run the tokens, commit the new lengths.  With `samplers` (one
        per wanted row, in order) the result also holds the sampled tokens."""
        if self._again is not None and not self.profile_decode:
            result = self._step_again(entries, samplers)
            if result is not None:
                return result
        self._again = None
        profiled = self.profile_decode and bool(entries) and all(len(e.tokens) == 1 for e in entries)
        if profiled:
            started_at = time.perf_counter()
            started, stopped = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            started.record()
        entries, sequences = self.reserve(entries)
        if not entries:
            return StepResult(None, [], 0)
        result = self.execute(entries, sequences, samplers)
        self.commit(entries, sequences)
        self.steps += 1
        self.tokens_run += result.num_tokens
        if profiled:
            stopped.record()
            result.timings = DecodeTimings(time.perf_counter() - started_at, len(entries), started, stopped)
            self.decode_timings.append(result.timings)
            del self.decode_timings[:-4096]
        return result

    def decode_many(self, entries: Sequence[StepEntry], samplers, steps: int) -> torch.Tensor:
        """`steps` decode steps for the same requests with no host work in between: each step's sampled
        token is the next step's input on the device.  Pages for all the steps are taken first.  Returns
        the sampled tokens [steps, rows] (int32, host).  Greedy or seeded sampling without penalty only;
        stopping rules are the caller's to apply afterwards."""
        from .decode_graph import LOG_STEPS
        if steps > LOG_STEPS:
            raise SchedulerError(f"decode_many takes at most {LOG_STEPS} steps at a time")
        entries = list(entries)
        if not self._graph_eligible(entries, samplers):
            raise SchedulerError("decode_many needs decode graphs, one token per request and samplers "
                                 "without a repetition penalty")
        if any(not s.greedy for s in samplers):
            raise SchedulerError("decode_many draws nothing on the host: greedy samplers only")
        self._again = None
        ahead = [StepEntry(e.request_id, list(e.tokens) + [0] * (steps - 1), []) for e in entries]
        ahead, sequences = self.reserve(ahead)
        self.storage.zero_slots(self.manager.take_fresh_slots())
        graph = self._graphs.get(len(entries), sequences, steps, False)
        graph.load([e.tokens[0] for e in entries], sequences, None)
        graph.step_counter.zero_()
        for _ in range(steps):
            graph.replay()
        tokens = graph.token_log[:steps, :len(entries)].cpu()
        graph.step_counter.zero_()
        for entry, seq in zip(ahead, sequences):      # (the sampled ids stayed on the device: no tokens to remember)
            self.manager.commit(seq, seq.length + len(entry.tokens))
        self.steps += steps
        self.tokens_run += steps * len(entries)
        return tokens
