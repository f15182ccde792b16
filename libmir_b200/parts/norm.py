"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, no (1 + w) form.

libmir cuda/kernels/rms_norm_bf16.cu:3-36; eps key and aliases models/src/layout/decoder/parse/mod.rs:82-86.
The input is the 32-bit residual stream; the weight is kept in 32-bit (exact for every stored dtype).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.spec import ParamSpec
from .base import Norm


class RmsNorm(Norm):
    graph_safe = True
    foldable = True       # y = x * s * w with one s per row: the products around it can take it over

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.weight: Optional[torch.Tensor] = None

    def parameters(self):
        return {"weight": ParamSpec((self.spec.size,), init="ones", store="float32")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, ctx, x, out=None, rows=None, lazy=False):
        """`lazy`: the caller's next product can take over this norm; if what it needs is at hand (the sums of
        squares of x and its rows times this norm's weight, written by the product that last added into x),
        return a NormedResidual instead of running a kernel."""
        if (lazy and kernels.FUSE_NORM_INTO_PRODUCT and out is None and rows is None
                and self.env.dtype == torch.bfloat16):
            stats = ctx.stats_for(x, self.weight)
            if stats is not None:
                return kernels.NormedResidual(x, self.weight, self.spec.eps, stats[0], stats[1], self.env.dtype,
                                              stats[2])
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.alloc((n_rows, self.spec.size), self.env.dtype)
        kernels.rms_norm(x, self.weight, self.spec.eps, out, rows)
        return out
