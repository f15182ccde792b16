"""Sampling of a batch of logits rows on the device.

Modes, per row (libmir src/generation/sampling.rs:49-88, runtime/src/sampling/mod.rs:46-135):
greedy (temperature <= epsilon or top_k == 1), full-vocabulary temperature sampling, and ranked
sampling with top-p and/or top-k; a repetition penalty rewrites the row's logits first
(runtime/src/sampling/candidate.rs:92-107).  The kernels are in csrc/sampling.cu.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..config.generation import DEFAULT_SEED, GenerationSettings
from .rng import SplitMix64

FLT_EPSILON = 1.1920929e-07


@dataclass
class RequestSampler:
    """Per-request sampling state: options, the generator, and the distinct tokens seen (for the penalty)."""

    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    seed: int = DEFAULT_SEED

    def __post_init__(self):
        self.rng = SplitMix64(self.seed)
        self.seen: set = set()

    @classmethod
    def from_settings(cls, settings: GenerationSettings, seed: Optional[int] = None) -> "RequestSampler":
        return cls(settings.temperature, settings.top_p, settings.top_k, settings.repetition_penalty,
                   DEFAULT_SEED if seed is None else seed)

    @property
    def greedy(self) -> bool:
        return self.temperature <= FLT_EPSILON or self.top_k == 1

    @property
    def ranked(self) -> bool:
        return not self.greedy and not (self.top_k == 0 and self.top_p >= 1.0)

    def observe(self, tokens) -> None:
        if self.repetition_penalty > 1.0:
            self.seen.update(int(t) for t in tokens)

    def next_draw(self) -> float:
        return 0.0 if self.greedy else self.rng.next_unit()


class DeviceSampler:
    def __init__(self, device: torch.device, vocab_size: int):
        self.device = device
        self.vocab_size = vocab_size
        self._sort_keys: Optional[torch.Tensor] = None
        self._greedy_options: Optional[torch.Tensor] = None
        self._tokens: Optional[torch.Tensor] = None

    def _token_buffer(self, rows: int) -> torch.Tensor:
        if self._tokens is None or self._tokens.numel() < rows:
            self._tokens = torch.empty(max(rows, 64), dtype=torch.int32, device=self.device)
        return self._tokens[:rows]

    def greedy_options(self, rows: int) -> torch.Tensor:
        """Device options of an all-greedy batch; built once, so greedy steps copy nothing to the device."""
        if self._greedy_options is None or self._greedy_options.numel() < rows * kernels.SAMPLE_OPTIONS.itemsize:
            count = max(rows, 256)
            host = np.zeros(count, dtype=kernels.SAMPLE_OPTIONS)
            host["top_p"] = 1.0
            self._greedy_options = torch.from_numpy(host.view(np.uint8)).to(self.device)
        return self._greedy_options

    def sample(self, logits: torch.Tensor, samplers: Sequence[RequestSampler], candidates=None) -> torch.Tensor:
        """One token per row; returns an int32 device tensor [rows] (valid until the next call).  `candidates`:
        what the head's kernel left beside these logits (kernels.HeadCandidates); not used once a penalty has
        changed the logits."""
        rows = logits.shape[0]
        assert rows == len(samplers)
        tokens = self._token_buffer(rows)
        if all(s.greedy and s.repetition_penalty <= 1.0 for s in samplers):
            kernels.sample(logits, self.greedy_options(rows), tokens, candidates=candidates)
            return tokens
        penalised = [(r, s) for r, s in enumerate(samplers) if s.repetition_penalty > 1.0 and s.seen]
        if penalised:
            ids = np.concatenate([np.fromiter(s.seen, dtype=np.int32) for _, s in penalised])
            id_rows = np.concatenate([np.full(len(s.seen), r, dtype=np.int32) for r, s in penalised])
            penalties = np.ones(rows, dtype=np.float32)
            for r, s in penalised:
                penalties[r] = s.repetition_penalty
            kernels.repetition_penalty(logits, torch.from_numpy(ids).to(self.device),
                                       torch.from_numpy(id_rows).to(self.device),
                                       torch.from_numpy(penalties).to(self.device))
        host = np.zeros(rows, dtype=kernels.SAMPLE_OPTIONS)
        for r, s in enumerate(samplers):
            host[r] = (s.next_draw(), s.temperature, s.top_p, s.top_k, 0)
        options = torch.from_numpy(host.view(np.uint8)).to(self.device)
        needs_ranked = any(s.ranked for s in samplers)
        if needs_ranked:
            need = kernels.ranked_scratch_keys(rows, self.vocab_size)
            if self._sort_keys is None or self._sort_keys.numel() < need:
                self._sort_keys = torch.empty(need, dtype=torch.int64, device=self.device)
        kernels.sample(logits, options, tokens, self._sort_keys if needs_ranked else None, needs_ranked,
                       None if penalised else candidates)
        return tokens
