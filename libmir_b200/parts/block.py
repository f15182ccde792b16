"""Arrangements of a mixer and a feed-forward in one layer.

pre_norm:  x += mixer(norm_1(x));  x += feed_forward(norm_2(x))
(metal/src/engine/dense/swiglu/layer.rs:123-166).  The residual stream x is 32-bit; each branch adds
its result into it (the matrix product's accumulate epilogue), so no separate add kernel runs.
A layer without feed-forward, or without one of the norms, leaves that step out.
"""

from __future__ import annotations

import torch

from ..registry import build_part
from .base import Block


class PreNormBlock(Block):
    SLOTS = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer_norm = build_part(spec.mixer_norm, env)
        self.mixer = build_part(spec.mixer, env)
        self.feed_forward_norm = build_part(spec.feed_forward_norm, env)
        self.feed_forward = build_part(spec.feed_forward, env)

    def parts(self):
        """(slot name, part) of every part this block holds."""
        return [(slot, getattr(self, slot)) for slot in self.SLOTS if getattr(self, slot) is not None]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def first_norm(self):
        """The norm this block applies to the incoming residual before anything else, or None."""
        return self.mixer_norm

    def native_descriptor(self, cache):
        """The layer as the native executor wants it (kernels.executor.LayerDesc), if every part of it is of the
        built-in kind that the executor runs (RMSNorm, softmax attention with the kernel's rotation or no position
        encoding, SwiGLU or no feed-forward) and its weights are bound; else None, and the parts run one by one."""
        from ..kernels.executor import LayerDesc, NormDesc
        from .attention import SoftmaxAttention
        from .feed_forward import SwiGlu
        from .norm import RmsNorm
        mixer, ff = self.mixer, self.feed_forward
        if type(mixer) is not SoftmaxAttention or type(self.mixer_norm) is not RmsNorm or cache is None \
                or cache.k_pages is None or mixer.w_qkv is None:
            return None
        if ff is not None and (type(ff) is not SwiGlu or type(self.feed_forward_norm) is not RmsNorm):
            return None
        rotation = mixer.position.rotation() if mixer.position is not None else (None, 0)
        if rotation is None or self.env.dtype not in (torch.bfloat16, torch.float32):
            return None
        s = mixer.spec
        if cache.k_pages.shape[1:] != (s.kv_heads, s.head_dim) or cache.v_pages.shape != cache.k_pages.shape \
                or not cache.k_pages.is_contiguous() or not cache.v_pages.is_contiguous():
            return None
        pointer = lambda tensor: None if tensor is None else tensor.data_ptr()
        norm = lambda part: NormDesc(part.weight.data_ptr(), part.spec.eps, part.spec.size)
        table, rotary_dim = rotation
        desc = LayerDesc()
        desc.mixer_norm = norm(self.mixer_norm)
        desc.w_qkv, desc.b_qkv, desc.w_o, desc.b_o = (pointer(mixer.w_qkv), pointer(mixer.b_qkv), pointer(mixer.w_o),
                                                      pointer(mixer.b_o))
        desc.q_norm, desc.k_norm, desc.inv_freq = pointer(mixer.q_norm), pointer(mixer.k_norm), pointer(table)
        desc.heads, desc.kv_heads, desc.head_dim, desc.rotary_dim = s.heads, s.kv_heads, s.head_dim, rotary_dim
        desc.window, desc.group, desc.writes_cache, desc.page_size = (int(s.window or 0), cache.group, int(cache.writes),
                                                                      cache.page_size)
        desc.scale, desc.qk_eps = s.scale, s.qk_norm_eps
        desc.k_pages, desc.v_pages, desc.cache_rows = cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), cache.k_pages.shape[0]
        if ff is not None:
            desc.ff_norm = norm(self.feed_forward_norm)
            desc.w_gate_up, desc.w_down, desc.inter = ff.w_gate_up.data_ptr(), ff.w_down.data_ptr(), ff.spec.intermediate_size
        return desc

    def forward(self, ctx, cache, residual):
        # Before a part runs, the context is told which norm follows it, so that its last product can prepare
        # that norm (parts.base.PartContext).
        after = ctx.norm_after_block
        x = (self._norm(self.mixer_norm, self.mixer, ctx, residual) if self.mixer_norm is not None
             else ctx.cast_residual(residual))
        ctx.residual_stats = None            # the mixer changes the residual; it may note new sums of squares
        ctx.upcoming_norm = self.feed_forward_norm if self.feed_forward is not None else after
        self.mixer.forward(ctx, cache, x, residual)
        if self.feed_forward is not None:
            x = (self._norm(self.feed_forward_norm, self.feed_forward, ctx, residual)
                 if self.feed_forward_norm is not None else ctx.cast_residual(residual))
            ctx.residual_stats = None
            ctx.upcoming_norm = after
            self.feed_forward.forward(ctx, x, residual)
        ctx.upcoming_norm = None

    @staticmethod
    def _norm(norm, consumer, ctx, residual):
        if consumer.takes_normed_residual and norm.foldable:
            return norm.forward(ctx, residual, lazy=True)
        return norm.forward(ctx, residual)


ARRANGEMENTS = {"pre_norm": PreNormBlock}


def build_block(layer_spec, env):
    from ..errors import RegistryError
    cls = ARRANGEMENTS.get(layer_spec.arrangement)
    if cls is None:
        raise RegistryError(f"unknown arrangement {layer_spec.arrangement!r}; known: {', '.join(sorted(ARRANGEMENTS))}")
    return cls(layer_spec, env)
