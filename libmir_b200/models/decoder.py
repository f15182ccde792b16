"""A decoder put together from a ModelSpec: embedding, blocks in schedule order, final norm, head.

This class is architecture-neutral: which mixer, feed-forward, norm and position encoding each layer
has, under which names its tensors are stored and in which order layers run is all in the ModelSpec.
Flow as in libmir's metal/src/engine/dense/swiglu/model.rs:117-131 and
cuda/src/backend/model/session/prefill/packed.rs:23-89 (packed rows, final norm and head only on the
rows whose logits are wanted).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import FixedState, ModelSpec, PagedKv, ParamSpec
from ..parts.base import BuildEnv, Part
from ..parts.block import build_block
from ..registry import build_part


@dataclass(frozen=True)
class CacheEntryPlan:
    """What schedule entry `entry` needs from the cache manager."""

    entry: int
    requirement: object            # PagedKv | FixedState | None
    source: int                    # the entry whose storage it uses (itself unless cache_of)
    writes: bool


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self.env = env
        self.blocks = [build_block(layer, env) for layer in spec.layers]
        self.final_norm = build_part(spec.final_norm, env)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self._runs_key, self._runs_list, self._native = None, [], {}

    # -- what the cache manager must provide ------------------------------------
    def cache_plan(self) -> List[CacheEntryPlan]:
        plan = []
        for index, entry in enumerate(self.spec.schedule):
            requirement = self.blocks[entry.layer].cache_requirement()
            if entry.cache_of is not None:
                other = self.blocks[self.spec.schedule[entry.cache_of].layer].cache_requirement()
                if other != requirement:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, whose shape "
                                     f"{other} differs from its own {requirement}")
                plan.append(CacheEntryPlan(index, requirement, entry.cache_of, False))
            else:
                plan.append(CacheEntryPlan(index, requirement, index, True))
        return plan

    # -- parameters ---------------------------------------------------------------
    def parameter_table(self) -> Dict[str, Tuple[object, str, ParamSpec]]:
        """Checkpoint name -> (owner, local name, ParamSpec) for every tensor of the model."""
        spec = self.spec
        table: Dict[str, Tuple[object, str, ParamSpec]] = {}
        table[spec.embedding.name] = (self, "embedding", ParamSpec((spec.embedding.vocab_size, spec.embedding.hidden_size)))
        for layer_spec, block in zip(spec.layers, self.blocks):
            for slot, part in block.parts():
                for local, param in part.parameters().items():
                    table[layer_spec.prefix + layer_spec.names[slot] + local] = (part, local, param)
        for local, param in self.final_norm.parameters().items():
            table[spec.final_norm_name + local] = (self.final_norm, local, param)
        if not spec.head.tied:
            table[spec.head.name] = (self, "head", ParamSpec((spec.head.vocab_size, spec.head.hidden_size)))
        return table

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every loaded tensor (by checkpoint name) to the part that owns it."""
        per_owner: Dict[int, Tuple[object, Dict[str, torch.Tensor]]] = {}
        for name, (owner, local, _) in self.parameter_table().items():
            if name in tensors:
                per_owner.setdefault(id(owner), (owner, {}))[1][local] = tensors[name]
        for owner, local_tensors in per_owner.values():
            if owner is self:
                self.embedding = local_tensors["embedding"].contiguous()
                self.head = local_tensors.get("head")
            else:
                owner.bind(local_tensors)
        if self.spec.head.tied:
            self.head = self.embedding
        self.head = self.head.contiguous()
        self._runs_key = None                       # descriptors of the layers hold pointers to the old tensors

    def parts(self) -> List[Part]:
        out: List[Part] = []
        for block in self.blocks:
            out.extend(part for _, part in block.parts())
        out.append(self.final_norm)
        return out

    def portion_multiple(self) -> int:
        """The least common multiple of what the parts ask of the scheduler's cuts (Part.portion_multiple)."""
        import math
        return math.lcm(*[max(1, int(part.portion_multiple)) for part in self.parts()])

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every layer of the schedule once, the final norm and the
        head; the embedding table is only gathered from."""
        total = 0
        for entry in self.spec.schedule:
            total += sum(part.weight_bytes() for _, part in self.blocks[entry.layer].parts())
        total += self.final_norm.weight_bytes() + self.head.numel() * self.head.element_size()
        return total

    # -- running --------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Run the tokens of the step; returns the 32-bit residual [T, H] after the last layer."""
        spec = self.spec
        residual = ctx.alloc((ctx.num_tokens, spec.hidden_size), torch.float32)
        kernels.embed(self.embedding, ctx.tokens, residual, spec.embedding.multiplier)
        for run in self._runs(ctx):
            if run.layers is not None:
                run.execute(ctx, residual)
                continue
            index = run.first
            entry = spec.schedule[index]
            # the norm that the next block in the schedule starts with: this block's last product may prepare it
            following = self.blocks[spec.schedule[index + 1].layer] if index + 1 < len(spec.schedule) else None
            ctx.norm_after_block = following.first_norm() if following is not None else None
            if index + 1 < len(spec.schedule) and self._native.get(index + 1) is not None:
                ctx.norm_after_block = None          # the executor that runs the next block starts from the residual
            self.blocks[entry.layer].forward(ctx, ctx.cache_view(index), residual)
        return residual

    def _runs(self, ctx) -> list:
        """The schedule cut into runs: consecutive entries whose blocks the native executor takes form one run (one
        native call), every other entry runs part by part from Python.  Built once per cache storage, since the
        descriptors hold pointers to its pages."""
        key = id(ctx.views)
        if self._runs_key == key:
            return self._runs_list
        from ..kernels.executor import LayerRun
        self._native = {}
        if kernels.NATIVE_LAYERS:
            for index, entry in enumerate(self.spec.schedule):
                self._native[index] = self.blocks[entry.layer].native_descriptor(ctx.cache_view(index))
        runs, index = [], 0
        while index < len(self.spec.schedule):
            if self._native.get(index) is None:
                runs.append(LayerRun(index, None, self.env.dtype))
                index += 1
                continue
            last = index
            while last + 1 < len(self.spec.schedule) and self._native.get(last + 1) is not None:
                last += 1
            runs.append(LayerRun(index, [self._native[i] for i in range(index, last + 1)], self.env.dtype))
            index = last + 1
        self._runs_key, self._runs_list = key, runs
        return runs

    def logits(self, ctx, residual: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None,
               candidates=None) -> torch.Tensor:
        """32-bit logits [len(rows), V] at the packed rows `rows` (an int32 device tensor).  `candidates`
        (kernels.HeadCandidates): filled by the head's kernel where it can, for the sampling that follows."""
        normed = self.final_norm.forward(ctx, residual, rows=rows)
        if out is None:
            out = ctx.alloc((rows.numel(), self.spec.vocab_size), torch.float32)
        kernels.head_logits(normed, self.head, out, candidates)
        return out
