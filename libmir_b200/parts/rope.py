"""Rotary position encoding, half-split layout: dims i and i + r/2 of the first r dims form a pair.

inverse frequency f_i = theta^(-2i/r) (libmir cuda/kernels/qkv_postprocess_bf16.cu:37-69), optionally
remapped by the llama3 piecewise rule (metal/src/engine/attention/rope.rs:58-96, keys
models/src/layout/decoder/rope.rs:61-95).  The table is computed once in 64-bit and held in 32-bit;
the angle position * f_i is a 32-bit product inside the kernel that applies it.
"""

from __future__ import annotations

import math

import torch

from .base import Position


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    index = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inverse = torch.pow(torch.tensor(theta, dtype=torch.float64), -index / rotary_dim)
    if scaling is not None:
        wavelength = 2.0 * math.pi / inverse
        ratio = scaling.original_max_position_embeddings / wavelength
        smooth = ((ratio - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)).clamp(0, 1)
        inverse = (inverse / scaling.factor) * (1.0 - smooth) + inverse * smooth
    return inverse.to(torch.float32)


class Rotary(Position):
    """Owned by a mixer; `table` is what its kernel multiplies positions with."""

    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2 or not 0 <= spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.rotary_dim = spec.rotary_dim
        self.table = inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling).to(env.device)

    def rotation(self):
        return self.table, self.rotary_dim
