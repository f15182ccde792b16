"""The host's side of the native layer executor (csrc/executor.cu): descriptors of layers and of a step, and the
call that runs a run of layers.

A layer of the built-in kind (pre-norm block of RMSNorm, softmax attention with rotary positions or none, SwiGLU or
no feed-forward) describes itself once as a LayerDesc: pointers to its bound weights and to its cache pages, and its
numbers.  A step describes its packed rows and its scratch memory as a StepDesc.  `run_layers` hands both to native
code, which issues every launch of those layers; layers of any other kind run part by part from Python.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import List, Optional, Sequence

import torch

from ..errors import KernelError


class NormDesc(Structure):
    _fields_ = [("weight", c_void_p), ("eps", c_float), ("size", c_int)]


class LayerDesc(Structure):
    _fields_ = [
        ("mixer_norm", NormDesc),
        ("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_o", c_void_p), ("b_o", c_void_p),
        ("q_norm", c_void_p), ("k_norm", c_void_p), ("inv_freq", c_void_p),
        ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int), ("window", c_int),
        ("group", c_int), ("writes_cache", c_int), ("page_size", c_int),
        ("scale", c_float), ("qk_eps", c_float),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("cache_rows", c_longlong),
        ("ff_norm", NormDesc),
        ("w_gate_up", c_void_p), ("w_down", c_void_p),
        ("inter", c_int), ("pad", c_int),
    ]


class GroupDesc(Structure):
    _fields_ = [("block_table", c_void_p), ("slot_mapping", c_void_p), ("table_width", c_int), ("pad", c_int)]


class StepDesc(Structure):
    _fields_ = [
        ("bf16", c_int), ("tokens", c_int), ("rows", c_int), ("singles", c_int), ("single_context", c_int),
        ("max_context", c_int), ("decode_only", c_int), ("hidden", c_int),
        ("positions", c_void_p), ("row_of_token", c_void_p), ("query_starts", c_void_p), ("context_lens", c_void_p),
        ("groups", POINTER(GroupDesc)),
        ("n_groups", c_int), ("fuse_norm", c_int),
        ("residual", c_void_p), ("normed", c_void_p), ("qkv", c_void_p), ("mixed", c_void_p),
        ("hidden_act", c_void_p), ("gate_up", c_void_p),
        ("sumsq", c_void_p * 2), ("weighted", c_void_p * 2),
        ("attention_scratch", c_void_p), ("attention_scratch_floats", c_longlong),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("prefill_tensor_cores", c_int), ("prefill_tensor_core_min_portion", c_int),
        ("norm_after", c_void_p), ("stream", c_void_p),
    ]


_CHECKED: set = set()


def _entry(lib_name: str):
    from . import library
    lib = library(lib_name)
    if lib_name not in _CHECKED:
        sizes = [c_int(), c_int(), c_int()]
        lib.mir_executor_layout.argtypes = [POINTER(c_int)] * 3
        lib.mir_executor_layout.restype = c_int
        lib.mir_executor_layout(*[ctypes.byref(s) for s in sizes])
        expected = (ctypes.sizeof(LayerDesc), ctypes.sizeof(StepDesc), ctypes.sizeof(GroupDesc))
        if tuple(s.value for s in sizes) != expected:
            raise KernelError(f"the executor's descriptors are {[s.value for s in sizes]} bytes in the native library "
                              f"and {list(expected)} in Python: the two were built from different sources")
        lib.mir_run_layers.argtypes = [POINTER(LayerDesc), c_int, POINTER(StepDesc), c_void_p, c_void_p, c_void_p]
        lib.mir_run_layers.restype = c_int
        _CHECKED.add(lib_name)
    return lib


def layer_array(descriptors: Sequence[LayerDesc]):
    return (LayerDesc * len(descriptors))(*descriptors)


def run_layers(bf16: bool, layers, count: int, step: StepDesc) -> None:
    """Run `count` layers of the LayerDesc array on the step; raises KernelError with the native message."""
    lib = _entry("bf16" if bf16 else "core")
    status = lib.mir_run_layers(layers, count, ctypes.byref(step), None, None, None)
    if status != 0:
        raise KernelError(lib.mir_last_error().decode(errors="replace") or f"the layer executor failed with status {status}")


class LayerRun:
    """Consecutive schedule entries from `first` on.  With `layers` (their LayerDesc), the run is one call of the
    native executor; with None it is one entry whose parts run from Python."""

    def __init__(self, first: int, layers: Optional[List[LayerDesc]], dtype: torch.dtype):
        self.first = first
        self.layers = layers
        self.bf16 = dtype == torch.bfloat16
        self.dtype = dtype
        if layers is None:
            return
        self.array = layer_array(layers)
        self.count = len(layers)
        self.qkv_width = max((d.heads + 2 * d.kv_heads) * d.head_dim for d in layers)
        self.mixed_width = max(d.heads * d.head_dim for d in layers)
        self.inter = max(d.inter for d in layers)
        self.heads = max(d.heads for d in layers)
        self.head_dim = max(d.head_dim for d in layers)
        self.fast_attention = self.bf16 and any(d.head_dim in (64, 128) for d in layers)
        self.attention_shapes = sorted({(d.heads, d.kv_heads, d.head_dim, d.page_size) for d in layers
                                        if d.head_dim in (64, 128)})

    def execute(self, ctx, residual: torch.Tensor) -> None:
        """Scratch from the step's arena (one set for the whole run: the layers use it one after the other), the
        step's metadata, one native call."""
        from . import (FUSE_NORM_INTO_PRODUCT, PREFILL_TENSOR_CORE_MIN_PORTION,
                       PREFILL_TENSOR_CORES, NORM_STAT_STRIDE, _lt_workspace, _stream, decode_attention_plan,
                       few_rows_max, get_option, sumsq_tiles)
        tokens, hidden = residual.shape
        dtype = self.dtype
        step = StepDesc()
        step.bf16, step.tokens, step.rows, step.hidden = int(self.bf16), tokens, ctx.num_rows, hidden
        step.singles, step.single_context = ctx.single_rows, ctx.single_context
        step.max_context, step.decode_only = ctx.max_context, int(ctx.decode_only)
        step.positions, step.row_of_token = ctx.positions.data_ptr(), ctx.row_of_token.data_ptr()
        step.query_starts, step.context_lens = ctx.query_starts.data_ptr(), ctx.context_lens.data_ptr()
        groups = (GroupDesc * max(1, len(ctx.groups)))()
        for index, group in enumerate(ctx.groups):
            groups[index].block_table = group.block_table.data_ptr()
            groups[index].slot_mapping = group.slot_mapping.data_ptr()
            groups[index].table_width = group.block_table.shape[1]
        step.groups, step.n_groups = groups, len(ctx.groups)
        step.residual = residual.data_ptr()
        step.normed = ctx.alloc((tokens, hidden), dtype).data_ptr()
        step.qkv = ctx.alloc((tokens, self.qkv_width), dtype).data_ptr()
        step.mixed = ctx.alloc((tokens, self.mixed_width), dtype).data_ptr()
        if self.inter:
            step.hidden_act = ctx.alloc((tokens, self.inter), dtype).data_ptr()
            needs_pair = not self.bf16 or get_option("few_rows_max") < tokens < get_option("tensor_core_min_rows") \
                or hidden % 8 != 0
            if needs_pair:
                step.gate_up = ctx.alloc((tokens, 2 * self.inter), dtype).data_ptr()
        fold = self.bf16 and FUSE_NORM_INTO_PRODUCT and tokens <= few_rows_max()
        step.fuse_norm = int(fold)
        if fold:
            for index in range(2):
                step.sumsq[index] = ctx.alloc((sumsq_tiles(hidden), NORM_STAT_STRIDE), torch.float32).data_ptr()
                step.weighted[index] = ctx.alloc((tokens, hidden), torch.bfloat16).data_ptr()
        if self.fast_attention:
            singles = ctx.num_rows if ctx.decode_only else ctx.single_rows
            longest = ctx.max_context if ctx.decode_only else ctx.single_context
            floats = max(decode_attention_plan(singles, heads, kv_heads, head_dim, page_size, longest)[2]
                         for heads, kv_heads, head_dim, page_size in self.attention_shapes) if singles else 0
            if floats:
                step.attention_scratch = ctx.alloc((floats,), torch.float32).data_ptr()
                step.attention_scratch_floats = floats
        if self.bf16:
            workspace = _lt_workspace(residual.device)
            step.workspace, step.workspace_bytes = workspace.data_ptr(), workspace.numel()
        step.prefill_tensor_cores = int(PREFILL_TENSOR_CORES)
        step.prefill_tensor_core_min_portion = PREFILL_TENSOR_CORE_MIN_PORTION
        step.stream = _stream()
        run_layers(self.bf16, self.array, self.count, step)
        ctx.residual_stats = None
