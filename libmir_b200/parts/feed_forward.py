"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), accumulated into the 32-bit residual.

Gate and up are one product on row-stacked [Wg; Wu] whose output row is [gate | up], as libmir's CUDA
engine does (cuda/src/backend/linear/pair.rs:36-64, cuda/src/backend/dense/feed_forward.rs:108-150).
silu is computed in 32-bit and is not rounded before the multiplication with up.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import ParamSpec
from .base import FeedForward


class SwiGlu(FeedForward):
    graph_safe = True
    takes_normed_residual = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.w_gate_up = self.w_down = None

    def parameters(self):
        s = self.spec
        return {
            "gate_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size)),
            "up_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size)),
            "down_proj.weight": ParamSpec((s.hidden_size, s.intermediate_size)),
        }

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0)
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, ctx, x, residual):
        s = self.spec
        tokens = x.shape[0]
        hidden = ctx.alloc((tokens, s.intermediate_size), self.env.dtype)
        kernels.gate_up_silu(x, self.w_gate_up, hidden, ctx.alloc)
        ctx.accumulate(hidden, self.w_down, residual)      # may also prepare the norm that follows
