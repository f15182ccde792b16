"""Decode-only steps as captured CUDA graphs.

A step in which every request brings exactly one token and wants its logits sampled has a fixed shape
once the number of rows and the width of the block tables are rounded up to a bucket, so the whole
forward (cache-slot computation, embedding, layers, final norm, head, sampling, and moving the sampled
token into the next step's input) is captured once per bucket and replayed.  Per step the host copies
one small block (tokens, positions, slots, block tables, sampling options) to the device and reads the
sampled tokens back; `run_many` replays several steps without any host work in between.

libmir captures decode per bucket of rows {1, 2, 4, 5, 8, 10, 16, ...} and re-captures when split
attention's partition counts change (cuda/src/engine/batch/mod.rs:18-32,108-131,
cuda/src/backend/model/batch/capture.rs:26-54), and chains batch-1 decode on the device-resident token
(cuda/src/backend/model/graph/mod.rs:54-100, session/mod.rs:152-160).  Here kernels read lengths and tables
from device memory, and a bucket is keyed by (rows, table widths, ranked sampling): rows are rounded up to a
power of two or one and a half times one (17 live requests run 24 rows, 33 run 40), table widths to the pages
of the next 512 tokens, so that split attention launches about as many partitions as the longest context has
and a graph is captured anew once per 512 generated tokens.  The least recently used graphs are dropped
beyond MAX_GRAPHS.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from .context import GroupContext, StepContext

LOG_STEPS = 512            # sampled tokens kept on the device between host reads


MAX_GRAPHS = 32            # captured buckets kept per model
WIDTH_STEP_TOKENS = 512    # table widths above this many tokens are rounded up to the pages of a multiple of it


def _bucket(n: int, floor: int = 1) -> int:
    size = floor
    while size < n:
        size *= 2
    return size


def row_bucket(rows: int) -> int:
    """Rows of the captured batch for `rows` live requests: 1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 40, 48, 64, 96, ..."""
    if 32 < rows <= 40:
        return 40
    size = 1
    while size < rows:
        if size + size // 2 >= rows and size >= 2:
            return size + size // 2
        size *= 2
    return size


def width_bucket(pages: int, page_size: int) -> int:
    """Columns of the captured block table for requests of up to `pages` pages."""
    tokens = pages * page_size
    if tokens <= WIDTH_STEP_TOKENS:
        return _bucket(pages, 8)
    rounded = -(-tokens // WIDTH_STEP_TOKENS) * WIDTH_STEP_TOKENS
    return -(-rounded // page_size)


class DecodeGraph:
    def __init__(self, runner, rows: int, widths: Sequence[int], ranked: bool):
        self.runner = runner
        self.rows = rows
        self.widths = list(widths)
        self._written = [[None] * rows for _ in self.widths]      # per group and row: what its table holds
        self.ranked = ranked
        device = runner.device
        groups = len(widths)
        options_ints = rows * kernels.SAMPLE_OPTIONS.itemsize // 4
        # host-written block: sampling options (first: they hold 64-bit values and the block starts on a
        # 256-byte boundary), tokens, positions, state slots, one table per group
        sizes = [options_ints, rows, rows, rows] + [rows * w for w in widths]
        self._offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        upload = int(self._offsets[-1])
        # device-computed block: slot mapping per group, context lengths, and the constant index arrays
        self.meta = torch.zeros(upload + groups * rows + rows + rows + (rows + 1) + rows, dtype=torch.int32,
                                device=device)
        self.staging = torch.zeros(upload, dtype=torch.int32, pin_memory=True)
        self._host = self.staging.numpy()
        self._upload = upload
        cut = lambda index: self.meta[int(self._offsets[index]):int(self._offsets[index + 1])]
        self.options = cut(0).view(torch.uint8)
        self.tokens, self.positions, self.state_slots = cut(1), cut(2), cut(3)
        self.tables = [cut(4 + g).view(rows, widths[g]) for g in range(groups)]
        cursor = upload
        self.slot_mappings = []
        for _ in range(groups):
            self.slot_mappings.append(self.meta[cursor:cursor + rows])
            cursor += rows
        self.context_lens = self.meta[cursor:cursor + rows]; cursor += rows
        self.row_of_token = self.meta[cursor:cursor + rows]; cursor += rows
        self.query_starts = self.meta[cursor:cursor + rows + 1]; cursor += rows + 1
        self.want_rows = self.meta[cursor:cursor + rows]
        self.row_of_token.copy_(torch.arange(rows, dtype=torch.int32))
        self.query_starts.copy_(torch.arange(rows + 1, dtype=torch.int32))
        self.want_rows.copy_(torch.arange(rows, dtype=torch.int32))
        self.sampled = torch.zeros(rows, dtype=torch.int32, device=device)
        self.token_log = torch.zeros(LOG_STEPS, rows, dtype=torch.int32, device=device)
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.logits: Optional[torch.Tensor] = None
        self.sort_keys = None
        if ranked:
            self.sort_keys = torch.empty(kernels.ranked_scratch_keys(rows, runner.model.spec.vocab_size),
                                         dtype=torch.int64, device=device)
        # what the head's kernel leaves for the sampling kernel (each row's largest logit is among them)
        self.candidates = kernels.HeadCandidates.allocate(
            lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=device), rows, runner.model.spec.vocab_size)
        self.host_tokens = torch.zeros(rows, dtype=torch.int32, pin_memory=True)
        self.launches_per_replay = 0
        self.replays = 0
        self._copied = None
        self._fast_tokens, self._fast_positions = self._host_part(1), self._host_part(2)
        self._live_rows = -1                       # rows the upload block was last filled for
        self._greedy_options = False               # whether its sampling records are the greedy defaults
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._capture()

    # -- host views of the upload block --------------------------------------------------
    def _host_part(self, index: int) -> np.ndarray:
        return self._host[int(self._offsets[index]):int(self._offsets[index + 1])]

    def _context(self) -> StepContext:
        runner = self.runner
        groups = [GroupContext(block_table=self.tables[g], slot_mapping=self.slot_mappings[g],
                               table_width=self.widths[g]) for g in range(len(self.widths))]
        page = runner.manager.page_size
        return StepContext(
            num_tokens=self.rows, num_rows=self.rows, tokens=self.tokens, positions=self.positions,
            row_of_token=self.row_of_token, query_starts=self.query_starts, context_lens=self.context_lens,
            state_slots=self.state_slots, groups=groups, views=runner.storage.views, arena=runner.arena,
            dtype=runner.model.env.dtype, host_query_starts=list(range(self.rows + 1)),
            host_start_positions=[0] * self.rows, host_state_slots=[0] * self.rows,
            max_context=max(self.widths) * page if self.widths else 0, max_portion=1, decode_only=True,
            page_size=page)

    def _body(self) -> None:
        runner = self.runner
        runner.arena.reset()
        ctx = self._context()
        for g in range(len(self.widths)):
            kernels.decode_prepare(self.positions, self.tables[g], runner.manager.page_size, self.slot_mappings[g],
                                   self.context_lens)
        residual = runner.model.forward(ctx)
        self.logits = runner.model.logits(ctx, residual, self.want_rows, candidates=self.candidates)
        kernels.sample(self.logits, self.options, self.sampled, self.sort_keys, self.ranked, self.candidates)
        kernels.decode_advance(self.sampled, self.tokens, self.positions, self.token_log, self.step_counter)

    def _capture(self) -> None:
        # every row is padding while warming up and capturing: nothing is written to the cache
        self._host[:] = 0
        self._host_part(2)[:] = -1
        greedy = np.zeros(self.rows, dtype=kernels.SAMPLE_OPTIONS)
        greedy["top_p"] = 1.0
        self._host_part(0)[:] = greedy.view(np.int32)
        self.meta[:self._upload].copy_(self.staging)
        stream = torch.cuda.Stream(device=self.runner.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                self._body()                       # builds library plans and grows the arena before capture
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        before = kernels.launches()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._body()
        self.launches_per_replay = kernels.launches() - before
        self.graph = graph
        self.step_counter.zero_()

    # -- running -----------------------------------------------------------------------------
    def load(self, tokens: Sequence[int], sequences, options: Optional[np.ndarray]) -> None:
        """Fill the upload block for the live rows (the rest is padding) and copy it to the device."""
        n = len(tokens)
        if self._copied is not None:
            self._copied.synchronize()             # the previous copy has read the pinned block
        host_tokens, host_positions, host_slots = self._host_part(1), self._host_part(2), self._host_part(3)
        host_tokens[:n] = tokens
        host_positions[:n] = [seq.length for seq in sequences]
        host_slots[:n] = [seq.slot for seq in sequences]
        if n != self._live_rows:                   # (the padding rows are as the last call left them otherwise)
            host_tokens[n:] = 0
            host_positions[n:] = -1
            host_slots[n:] = 0
            self._live_rows = n
        if options is None:
            if not self._greedy_options:
                records = self._host_part(0).view(kernels.SAMPLE_OPTIONS)
                records["draw"], records["temperature"], records["top_p"], records["top_k"] = 0.0, 0.0, 1.0, 0
                self._greedy_options = True
        else:
            self._host_part(0).view(kernels.SAMPLE_OPTIONS)[:n] = options
            self._greedy_options = False
        # Block tables only grow at the end (and lose their head to a window): a row whose request, length and
        # first live block are what was written last time is left as it is.
        for g, width in enumerate(self.widths):
            table = self._host_part(4 + g).reshape(self.rows, width)
            written = self._written[g]
            for r, seq in enumerate(sequences):
                blocks = seq.tables[g]
                state = (seq.serial, len(blocks), seq.first_live[g])
                if written[r] == state:
                    continue
                previous = written[r]
                if previous is not None and previous[0] == seq.serial and previous[2] == seq.first_live[g] \
                        and previous[1] <= len(blocks):
                    table[r, previous[1]:len(blocks)] = blocks[previous[1]:]     # only the new blocks
                else:
                    table[r, :len(blocks)] = blocks
                    table[r, len(blocks):] = -1
                written[r] = state
            for r in range(n, self.rows):
                if written[r] is not None:
                    table[r] = 0
                    written[r] = None
        self.meta[:self._upload].copy_(self.staging, non_blocking=True)
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record()

    def load_again(self, tokens: Sequence[int], sequences, draws: Optional[Sequence[float]] = None) -> None:
        """The upload for the same rows with the same sampling settings as the last `load`, none of which got a page
        since: only the tokens, the positions and (for samplers that draw) the draws differ."""
        n = len(tokens)
        self._copied.synchronize()                 # the previous copy has read the pinned block
        self._fast_tokens[:n] = tokens
        self._fast_positions[:n] = [seq.length for seq in sequences]
        if draws is not None:
            self._host_part(0).view(kernels.SAMPLE_OPTIONS)["draw"][:n] = draws
        self.meta[:self._upload].copy_(self.staging, non_blocking=True)
        self._copied.record()

    def replay(self) -> None:
        self.graph.replay()
        self.replays += 1
        kernels.REPLAYED_LAUNCHES += self.launches_per_replay


class DecodeGraphs:
    """The buckets captured so far for one StepRunner."""

    def __init__(self, runner):
        self.runner = runner
        self.graphs: Dict[Tuple, DecodeGraph] = {}

    def usable(self) -> bool:
        """Every part must read the batch from device memory only and never wait for the device (graph_safe),
        since a replay cannot see what the host knew at capture time."""
        return all(getattr(part, "graph_safe", False) for part in self.runner.model.parts())

    def get(self, rows: int, sequences, extra_tokens: int, ranked: bool) -> DecodeGraph:
        page = self.runner.manager.page_size
        widths = []
        for g in range(len(self.runner.manager.groups)):
            need = max(-(-(seq.length + extra_tokens) // page) for seq in sequences)
            need = max(need, max(len(seq.tables[g]) for seq in sequences))
            widths.append(width_bucket(need, page))
        key = (row_bucket(rows), tuple(widths), ranked)
        graph = self.graphs.pop(key, None)
        if graph is None:
            graph = DecodeGraph(self.runner, key[0], widths, ranked)
            while len(self.graphs) >= MAX_GRAPHS:
                self.graphs.pop(next(iter(self.graphs)))        # the least recently used (dicts keep insertion order)
        self.graphs[key] = graph                                # (re-inserted: the most recently used is last)
        return graph
