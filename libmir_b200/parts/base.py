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

What a part may use of the step is the PartContext below: scratch memory, the residual-adding product, and the
protocol by which an RMSNorm between two few-rows products is folded into them.  That protocol is declared here,
not discovered: a norm says `foldable`, a consumer says `takes_normed_residual`, and `Norm.forward` has the
`lazy` argument in its signature.

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


class PartContext:
    """What a step hands to every part.  The engine's StepContext (engine/context.py) derives from this and adds the
    packed rows' metadata; a part that needs nothing of the batch (a norm, a feed-forward) runs on this alone, with
    `ScratchContext` as the smallest concrete form.

    alloc(shape, dtype)                   scratch memory that lives until the step ends.
    accumulate(x, weight, residual, bias) residual += x . weight^T (+ bias) on the 32-bit residual stream; every
                                          branch adds its result through this, so that the product can also
                                          prepare the norm named by `upcoming_norm` (see below).
    stats_for(residual, norm_weight)      what such a product left for the norm with that weight, or None.
    cast_residual(residual)               the residual in the engine dtype, for an arrangement without a norm.

    Folded norms: before a part runs, its block sets `upcoming_norm` to the norm that will be applied to the
    residual right after the part has added into it (None if unknown); the model sets `norm_after_block` to the norm
    the next block of the schedule starts with.  Whoever changes the residual in another way sets
    `residual_stats = None`."""

    dtype: Optional[torch.dtype] = None
    upcoming_norm = None
    norm_after_block = None
    residual_stats = None

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def accumulate(self, x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor,
                   bias: Optional[torch.Tensor] = None) -> None:
        from .. import kernels
        kernels.linear(x, weight, residual, bias, accumulate=True)
        self.residual_stats = None

    def stats_for(self, residual: torch.Tensor, norm_weight: torch.Tensor):
        return None

    def cast_residual(self, residual: torch.Tensor) -> torch.Tensor:
        from .. import kernels
        if self.dtype is None or self.dtype == torch.float32:
            return residual
        out = self.alloc(residual.shape, self.dtype)
        kernels.cast(residual, out)
        return out


class ScratchContext(PartContext):
    """A context that offers scratch memory and nothing of a batch: enough to run a norm or a feed-forward alone."""

    def __init__(self, alloc, dtype: Optional[torch.dtype] = None):
        self._alloc = alloc
        self.dtype = dtype

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        return self._alloc(shape, dtype)


class Part:
    """Base of every part."""

    # True if forward accepts a kernels.NormedResidual as x (an RMSNorm that was not run as a kernel but is
    # folded into the part's first product); every other part gets the normed tensor.
    takes_normed_residual = False

    # What the part asks of how prompts are cut: every portion of a request but its last has a multiple of this
    # many tokens (a mixer that scans in chunks names its chunk here; attention and per-token parts take any cut).
    portion_multiple = 1

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
    # True if the norm is y = x * s * weight with one 32-bit scale s per row and a float32 `weight` attribute: the
    # products around it can then take it over (the one before leaves sums of squares and weighted rows, the one
    # after scales its results).  Only a foldable norm is ever called with lazy=True.
    foldable = False

    def forward(self, ctx, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, lazy: bool = False) -> torch.Tensor:
        """The normed rows in the engine dtype.  `lazy` (foldable norms only): the caller's next product can take
        a kernels.NormedResidual; return one if ctx.stats_for(x, weight) has what it needs."""
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

    def native_descriptor(self, cache):
        """What the native layer executor needs to run this block by itself (kernels.executor.LayerDesc), or None if
        the block's parts run one by one from Python."""
        return None

    def first_norm(self) -> Optional["Norm"]:
        """The norm this block applies to the incoming residual before anything else, or None: the block before
        it in the schedule may prepare it in its last product."""
        return None

    def forward(self, ctx, cache, residual: torch.Tensor) -> None:
        raise NotImplementedError
