"""Arrangements of a mixer and a feed-forward in one layer.

pre_norm:  x += mixer(norm_1(x));  x += feed_forward(norm_2(x))
(metal/src/engine/dense/swiglu/layer.rs:123-166).  The residual stream x is 32-bit; each branch adds
its result into it (the matrix product's accumulate epilogue), so no separate add kernel runs.
A layer without feed-forward, or without one of the norms, leaves that step out.
"""

from __future__ import annotations

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
