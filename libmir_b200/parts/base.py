"""The interfaces of the parts a layer is put together from.

A part is built from its PartSpec (numbers only) and a BuildEnv (engine dtype, device).  It says
which tensors it wants (`parameters`), receives them (`bind`), and runs on packed rows.  No part
knows which model it is in, which layer it is, or how the step was cut: everything it may use about
the batch is in the StepContext (libmir_b200/engine/context.py).

    Norm          forward(ctx, x, out=None, rows=None) -> tensor in the engine dtype
                  x is the 32-bit residual [T, H]; rows optionally gathers a subset first.
    Mixer         cache_requirement() -> PagedKv | FixedState | None
                  forward(ctx, cache, x, residual) -> None      residual += mixer(x)
                  x is [T, H] in the engine dtype (already normed); cache is the CacheView of the
                  schedule entry being run (None if the mixer asked for none).
    FeedForward   forward(ctx, x, residual) -> None             residual += feed_forward(x)
    Position      owned by the mixer that uses it.  rotation() -> (table, rotary_dim) if the encoding is the
                  half-split rotation that the q/k kernel applies itself, else None, and then
                  apply(ctx, queries, keys) changes [T, heads, head_dim] views in place (after the per-head
                  norm, before keys go to their pages).
    Block         forward(ctx, cache, residual) -> None          one arrangement of the above

`parameters()` maps a name local to the part ("q_proj.weight") to a ParamSpec; the model joins it
with the layer's prefix and the slot's sub-prefix from LayerSpec.names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from ..config.spec import CacheRequirement, ParamSpec


@dataclass(frozen=True)
class BuildEnv:
    dtype: torch.dtype            # torch.bfloat16 or torch.float32: weights, activations and cache
    device: torch.device


class Part:
    """Base of every part."""

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def parameters(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named by `parameters` (optional ones may be absent), already on the
        device and in the dtype their ParamSpec.store asks for."""

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (for the roofline account)."""
        return 0

    # True if forward reads the batch only from device tensors of the context and never waits for the device:
    # decode steps of a model whose parts all say so are captured in CUDA graphs.
    graph_safe = False


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    def cache_requirement(self) -> CacheRequirement:
        return None

    def forward(self, ctx, cache, x: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Position(Part):
    def rotation(self):
        """(float32 table of rotary_dim / 2 inverse frequencies, rotary_dim) if this encoding is the half-split
        rotation by position * frequency, which the kernel that norms q and k and writes the cache applies
        itself; None for every other encoding, which `apply` then computes."""
        return None

    def apply(self, ctx, queries: torch.Tensor, keys: torch.Tensor) -> None:
        """Encode ctx.positions into queries [T, heads, head_dim] and keys [T, kv_heads, head_dim] in place
        (views of the packed projection in the engine dtype)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    def cache_requirement(self) -> CacheRequirement:
        return None

    def forward(self, ctx, cache, residual: torch.Tensor) -> None:
        raise NotImplementedError
