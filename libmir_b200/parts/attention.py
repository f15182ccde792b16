"""Grouped-query softmax attention over the paged cache.

input [T, H] -> one packed projection [T, (Hq + 2 Hkv) D] (weights row-stacked [Wq; Wk; Wv] as libmir's
CUDA loader packs them, cuda/src/backend/linear/pack.rs:35-76) -> per-head q/k RMSNorm and rotary,
K and V written to their pages (one kernel) -> attention over the request's pages -> output projection
accumulated into the 32-bit residual.  Formulas: metal/src/engine/dense/swiglu/attention.rs:14-112.
Options, all from the spec: q/k-norm, q/k/v bias and output bias, window, scale, position encoding.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.spec import PagedKv, ParamSpec, TensorSource
from ..registry import build_part
from .base import Mixer


class SoftmaxAttention(Mixer):
    takes_normed_residual = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        self.q_width = s.heads * s.head_dim
        self.kv_width = s.kv_heads * s.head_dim
        self.position = build_part(s.position, env) if s.position is not None else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = None

    @property
    def graph_safe(self):
        return self.position is None or self.position.graph_safe

    def cache_requirement(self):
        return PagedKv(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    # names under which checkpoints store query, key and value as one row-stacked tensor [Wq; Wk; Wv]
    # (models/src/weights/binding/roles/parse.rs: "self_attn.qkv_proj.weight" | "self_attn.query_key_value.weight")
    FUSED_NAMES = ("qkv_proj", "query_key_value")

    def parameters(self):
        s = self.spec
        total = self.q_width + 2 * self.kv_width
        ranges = {"q_proj": (0, self.q_width), "k_proj": (self.q_width, self.q_width + self.kv_width),
                  "v_proj": (self.q_width + self.kv_width, total)}

        def fused(projection, suffix):
            return tuple(TensorSource(f"{name}.{suffix}", ranges[projection], total) for name in self.FUSED_NAMES)

        table = {f"{projection}.weight": ParamSpec((end - begin, s.hidden_size), sources=fused(projection, "weight"))
                 for projection, (begin, end) in ranges.items()}
        table["o_proj.weight"] = ParamSpec((s.hidden_size, self.q_width))
        if s.qkv_bias:
            for projection, (begin, end) in ranges.items():
                table[f"{projection}.bias"] = ParamSpec((end - begin,), sources=fused(projection, "bias"))
        if s.out_bias:
            table["o_proj.bias"] = ParamSpec((s.hidden_size,))
        if s.qk_norm:
            table["q_norm.weight"] = ParamSpec((s.head_dim,), init="ones", store="float32")
            table["k_norm.weight"] = ParamSpec((s.head_dim,), init="ones", store="float32")
        return table

    def bind(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.spec.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0)
        if self.spec.out_bias:
            self.b_o = tensors["o_proj.bias"].contiguous()
        if self.spec.qk_norm:
            self.q_norm = tensors["q_norm.weight"].contiguous()
            self.k_norm = tensors["k_norm.weight"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.b_qkv, self.b_o) if t is not None)

    def forward(self, ctx, cache, x, residual):
        s = self.spec
        tokens = x.shape[0]
        qkv = ctx.alloc((tokens, self.q_width + 2 * self.kv_width), self.env.dtype)
        group = ctx.groups[cache.group]
        rotation = self.position.rotation() if self.position is not None else (None, 0)
        if rotation is None:
            self.project_with_other_position(ctx, cache, group, x, qkv)
        else:
            self.project(ctx, cache, group, x, qkv, *rotation)
        mixed = ctx.alloc((tokens, self.q_width), self.env.dtype)
        self.attend(ctx, group, cache, qkv, mixed)
        ctx.accumulate(mixed, self.w_o, residual, self.b_o)      # may also prepare the norm that follows

    def project(self, ctx, cache, group, x, qkv, table, rotary_dim):
        """Projection, then per-head norm, rotation and cache write in one kernel."""
        s = self.spec
        kernels.linear(x, self.w_qkv, qkv, self.b_qkv, alloc=ctx.alloc)
        kernels.qk_rope_store(qkv, ctx.positions, group.slot_mapping, table, self.q_norm, self.k_norm,
                              cache.k_pages, cache.v_pages, s.heads, s.kv_heads, s.head_dim, rotary_dim,
                              s.qk_norm_eps, write_kv=cache.writes)

    def project_with_other_position(self, ctx, cache, group, x, qkv):
        """A position encoding that is no rotation of the kernel's: projection, then the per-head norms alone, then
        the encoding's own `apply` on the q and k views, then keys and values into their pages."""
        s = self.spec
        kernels.linear(x, self.w_qkv, qkv, self.b_qkv, alloc=ctx.alloc)
        if s.qk_norm:
            kernels.qk_rope_store(qkv, ctx.positions, None, None, self.q_norm, self.k_norm, None, None, s.heads,
                                  s.kv_heads, s.head_dim, 0, s.qk_norm_eps, keys_in_place=True)
        tokens = qkv.shape[0]
        queries = qkv[:, :self.q_width].view(tokens, s.heads, s.head_dim)
        keys = qkv[:, self.q_width:self.q_width + self.kv_width].view(tokens, s.kv_heads, s.head_dim)
        self.position.apply(ctx, queries, keys)
        if cache.writes:
            kernels.qk_rope_store(qkv, ctx.positions, group.slot_mapping, None, None, None, cache.k_pages,
                                  cache.v_pages, s.heads, s.kv_heads, s.head_dim, 0, s.qk_norm_eps, write_kv=True)

    def attend(self, ctx, group, cache, qkv, out):
        """Attention of every packed row over its request's pages; the kernel is chosen by dtype and size:
        bfloat16 with head_dim 64 or 128 runs on tensor cores (split over the keys when every row is a
        single decoded token), everything else runs the reference kernel."""
        s = self.spec
        if self.env.dtype == torch.bfloat16 and s.head_dim in kernels.FAST_HEAD_DIMS:
            # the single-token rows come first in the batch: they run as decoded tokens (keys split over CTAs, the
            # heads of a KV group in one CTA), the prompt portions after them as tiles of queries
            singles = ctx.num_rows if ctx.decode_only else ctx.single_rows
            if singles:
                longest = ctx.max_context if ctx.decode_only else ctx.single_context
                partition, count, floats = kernels.decode_attention_plan(singles, s.heads, s.kv_heads, s.head_dim,
                                                                         cache.page_size, longest)
                scratch = ctx.alloc((floats,), torch.float32) if floats else None
                kernels.decode_attention(qkv[:singles], out[:singles], cache.k_pages, cache.v_pages,
                                         group.block_table[:singles], ctx.positions, cache.page_size, s.heads,
                                         s.kv_heads, s.head_dim, s.scale, s.window, partition, count, scratch)
            if singles < ctx.num_rows:
                kernels.prefill_attention(qkv, out, cache.k_pages, cache.v_pages, group.block_table[singles:],
                                          ctx.query_starts[singles:], ctx.context_lens[singles:], cache.page_size,
                                          s.heads, s.kv_heads, s.head_dim, s.scale, s.window,
                                          portion_tokens=out.shape[0] - singles)
            return
        kernels.paged_attention_generic(qkv, out, cache.k_pages, cache.v_pages, group.block_table, ctx.row_of_token,
                                        ctx.positions, cache.page_size, s.heads, s.kv_heads, s.head_dim, s.scale,
                                        s.window)
