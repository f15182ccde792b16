"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  Single-threaded and deterministic (first come, first served), so that a trace
can be reproduced.

libmir runs one worker thread per model fed by a channel (src/scheduler/generation/mod.rs:29-121,
worker/mod.rs:80-116); the decisions taken here follow it where it has them:
  * every live request that has its prompt in the cache decodes one token per step; decode rows come
    first and the prompt portions get what is left of the budget,
    budget = max_batch_tokens - decode rows, at least 1 (worker/budget.rs:104-116, src/scheduler/step.rs:49-56);
  * portions are cut "completion first": the oldest unfinished prompt gets as much of the budget as
    it can use, then the next (cuda/src/engine/execution/prefill/round/mod.rs:115-202), each at most
    prefill_chunk_tokens long (cuda/src/backend/model/config.rs:3);
  * a finished request's pages and slot go back before the next admission (src/session/mod.rs:152-166);
  * stop on a stop token unless ignore_eos and not before min_tokens, or at max_tokens
    (src/generation/mod.rs:124-187).
When pages run out (libmir makes the caller wait and never preempts, src/model/cache/mod.rs:43-61):
  * a request that could never fit is refused at submission (KvCapacity);
  * a waiting request is admitted only when the pages of its whole prompt (plus reserve_tokens) are free;
  * when a running request cannot get the page it needs, the youngest running request is preempted:
    its pages are freed, and it goes back to the head of the waiting queue to be recomputed from its
    prompt and the tokens it had produced (out_of_pages="preempt"), or it is finished with reason
    "out_of_pages" (out_of_pages="finish").  If the request that cannot grow is alone, it is finished
    with "out_of_pages".
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from ..cache import CacheManager
from ..config.generation import GenerationSettings
from ..config.runtime import SchedulerConfig
from ..errors import KvCapacity, SchedulerError
from ..sampling.sampler import RequestSampler
from .step import StepEntry


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    settings: GenerationSettings
    sampler: RequestSampler
    on_token: Optional[Callable[[int], None]] = None
    output: List[int] = field(default_factory=list)
    fed: int = 0                         # tokens of prompt + output that are in the cache
    state: str = "waiting"               # waiting | running | finished
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_order: int = -1
    cancelled: bool = False
    cached_tokens: int = 0               # tokens it found in the prefix cache (over all its admissions)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.fed


@dataclass
class PlannedEntry:
    request: Request
    start: int
    count: int
    samples: bool                        # the portion ends at the request's last token: sample after it


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, max_positions: int,
                 run_step: Callable[[Sequence[StepEntry], Sequence[RequestSampler]], List[int]],
                 portion_multiple: int = 1):
        """`run_step(entries, samplers)` runs one batch and returns the sampled token of every entry
        that wants one (those with a non-empty `want`), in order, as host integers.  `portion_multiple`: what
        the model's parts ask of the cuts (a mixer that scans in chunks wants every portion but a request's last
        to be a multiple of its chunk); a portion that does not end its request's pending tokens is cut down to
        a multiple of it."""
        config.validate()
        if portion_multiple < 1:
            raise SchedulerError("portion_multiple must be at least 1")
        if portion_multiple > 1 and portion_multiple > min(config.prefill_chunk_tokens,
                                                          config.max_batch_tokens - config.max_batch_requests):
            raise SchedulerError(f"the model wants portions in multiples of {portion_multiple} tokens: "
                                 f"prefill_chunk_tokens and max_batch_tokens - max_batch_requests must be at least that")
        self.portion_multiple = portion_multiple
        self.manager = manager
        self.config = config
        self.max_positions = max_positions
        self.run_step = run_step
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._admissions = 0
        self.steps = 0
        self.log: List[dict] = []          # one record per step: what ran (for tests and metrics)

    # -- submission ------------------------------------------------------------------
    def submit(self, request: Request) -> None:
        if not request.prompt:
            raise SchedulerError("a request needs at least one prompt token")
        if len(request.prompt) >= self.max_positions:
            raise SchedulerError(f"prompt of {len(request.prompt)} tokens leaves no room under "
                                 f"max_position_embeddings {self.max_positions}")
        for group in self.manager.groups:
            floor = self.manager.peak_pages(len(request.prompt) + 1, group, self.config.prefill_chunk_tokens)
            if floor > group.pool.count:
                raise KvCapacity(floor, group.pool.count, f"group {group.index}")
        request.state = "waiting"
        request.sampler.observe(request.prompt)
        self.waiting.append(request)

    def cancel(self, request_id) -> None:
        for request in list(self.waiting) + self.running:
            if request.request_id == request_id:
                request.cancelled = True

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def abandon(self, reason: str = "aborted") -> None:
        """Finish every request that is still waiting or running and give back what it holds: what a caller does
        when a step raised, so that the cache manager it shares with later calls keeps no holder of this one."""
        for request in list(self.running) + list(self.waiting):
            self._finish(request, reason)

    def _portion(self, request: Request, budget: int) -> int:
        """How many of the request's pending tokens the next step takes under `budget`."""
        count = min(request.pending, budget, self.config.prefill_chunk_tokens)
        if count < request.pending and self.portion_multiple > 1:
            count -= count % self.portion_multiple
        return count

    # -- finishing -------------------------------------------------------------------
    def _finish(self, request: Request, reason: str) -> None:
        if request.state == "running":
            self.manager.release(request.request_id)
            self.running.remove(request)
        elif request.state == "waiting":
            self.waiting.remove(request)
        request.state = "finished"
        request.finish_reason = reason
        self.finished.append(request)

    def _preempt(self, request: Request) -> None:
        """Free everything the request holds; it is recomputed from prompt + output later."""
        self.manager.release(request.request_id)
        self.running.remove(request)
        request.state = "waiting"
        request.fed = 0
        request.preemptions += 1
        self.waiting.appendleft(request)

    # -- planning --------------------------------------------------------------------
    def _pages_free(self) -> List[int]:
        return [group.pool.available for group in self.manager.groups]

    def _need(self, request: Request, count: int) -> List[int]:
        seq = self.manager.live[request.request_id]
        return self.manager.pages_needed(seq, seq.length + count)

    def _admission_need(self, request: Request) -> List[int]:
        total = min(self.max_positions, len(request.prompt) + len(request.output) + self.config.reserve_tokens)
        return [self.manager.peak_pages(total, group, self.config.prefill_chunk_tokens)
                for group in self.manager.groups]

    def plan(self) -> List[PlannedEntry]:
        """Decide the next step.  May preempt or finish requests that cannot get pages, and admits
        waiting requests; takes no pages itself (the step does)."""
        config = self.config
        for request in [r for r in list(self.waiting) + list(self.running) if r.cancelled]:
            self._finish(request, "cancelled")
        while True:
            free = self._pages_free()
            planned: List[PlannedEntry] = []
            starved = None
            # 1. decode rows, oldest first
            decoders = [r for r in self.running if r.pending == 1 and r.fed >= len(r.prompt)]
            decoders = decoders[:min(config.max_batch_requests, config.max_batch_tokens)]
            for request in decoders:
                need = self._need(request, 1)
                if any(n > f for n, f in zip(need, free)):
                    starved = request
                    break
                free = [f - n for f, n in zip(free, need)]
                planned.append(PlannedEntry(request, request.fed, 1, True))
            if starved is not None:
                # a running request cannot get its next page: take pages from the youngest, or, if it
                # is alone, end it
                if not self._make_room():
                    self._finish(starved, "out_of_pages")
                continue
            budget = max(1, config.max_batch_tokens - len(planned)) if planned else config.max_batch_tokens
            # 2. portions of prompts already running, oldest first
            for request in self.running:
                if budget <= 0 or request in decoders or request.pending == 0:
                    continue
                count = self._portion(request, budget)
                if count <= 0:
                    continue
                need = self._need(request, count)
                if any(n > f for n, f in zip(need, free)):
                    # shrink the portion to the pages that are free
                    count = self._fit(request, count, free)
                    if count <= 0:
                        continue
                    need = self._need(request, count)
                free = [f - n for f, n in zip(free, need)]
                budget -= count
                planned.append(PlannedEntry(request, request.fed, count, count == request.pending))
            # 3. admit waiting requests in order while slots, pages and budget allow
            while (self.waiting and budget > 0 and self.manager.free_slots > 0
                   and len(self.running) < config.max_batch_requests):
                request = self.waiting[0]
                need_all = self._admission_need(request)
                if any(n > f for n, f in zip(need_all, free)) or self._portion(request, budget) <= 0:
                    break
                self.waiting.popleft()
                # (with a prefix cache the request may find the pages of its first tokens: they count as fed, and
                # as taken from what was free, though some of them were held by others anyway)
                sequence = self.manager.admit(request.request_id, request.tokens)
                request.fed = sequence.length
                request.cached_tokens += sequence.prefix_tokens
                free = [f - len(table) for f, table in zip(free, sequence.tables)]
                request.state = "running"
                request.admitted_order = self._admissions
                self._admissions += 1
                self.running.append(request)
                count = self._portion(request, budget)
                need = self._need(request, count)
                free = [f - n for f, n in zip(free, need)]
                budget -= count
                planned.append(PlannedEntry(request, request.fed, count, count == request.pending))
            if not planned and (self.running or self.waiting):
                # nothing fits: free something, or give up on the request that blocks
                if self._make_room():
                    continue
                blocked = self.running[0] if self.running else self.waiting[0]
                self._finish(blocked, "out_of_pages")
                continue
            return planned

    def _fit(self, request: Request, count: int, free: List[int]) -> int:
        """The longest portion <= count whose pages are free."""
        seq = self.manager.live[request.request_id]
        page = self.manager.page_size
        best = count
        for g, table in enumerate(seq.tables):
            room = (len(table) + free[g]) * page - seq.length
            best = min(best, room)
        if best < request.pending and self.portion_multiple > 1:
            best -= best % self.portion_multiple
        return max(0, best)

    def _make_room(self) -> bool:
        """Preempt (or finish) the youngest running request to free pages; False if there is no
        other request to take pages from."""
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda r: r.admitted_order)
        if self.config.out_of_pages == "finish":
            self._finish(victim, "out_of_pages")
        else:
            self._preempt(victim)
        return True

    # -- running ---------------------------------------------------------------------
    def step(self) -> List[PlannedEntry]:
        """Plan and run one step; returns what ran."""
        planned = self.plan()
        if not planned:
            return planned
        entries = []
        for item in planned:
            tokens = item.request.tokens[item.start:item.start + item.count]
            entries.append(StepEntry(item.request.request_id, tokens, [item.count - 1] if item.samples else []))
        samplers = [item.request.sampler for item in planned if item.samples]
        sampled = self.run_step(entries, samplers)
        for item in planned:
            item.request.fed += item.count
        self.log.append({"step": self.steps, "tokens": sum(i.count for i in planned),
                         "decode_rows": sum(1 for i in planned if i.count == 1 and i.start >= len(i.request.prompt)),
                         "entries": [(i.request.request_id, i.start, i.count) for i in planned]})
        self.steps += 1
        cursor = 0
        for item in planned:
            if not item.samples:
                continue
            token = int(sampled[cursor])
            cursor += 1
            request = item.request
            request.output.append(token)
            request.sampler.observe([token])
            if request.on_token is not None:
                request.on_token(token)
            settings = request.settings
            produced = len(request.output)
            if (not settings.ignore_eos and token in settings.stop_token_ids and produced >= settings.min_tokens):
                self._finish(request, "stop")
            elif produced >= settings.max_tokens:
                self._finish(request, "length")
            elif len(request.prompt) + produced >= self.max_positions:
                self._finish(request, "length")
        return planned

    def run(self, max_steps: Optional[int] = None) -> None:
        """Step until every submitted request has finished."""
        steps = 0
        while not self.idle:
            self.step()
            steps += 1
            if max_steps is not None and steps >= max_steps:
                break
