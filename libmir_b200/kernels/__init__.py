"""Python launchers of the sm_100a kernels in libmir_b200/csrc.

Every function takes torch CUDA tensors, checks what the kernel cannot check itself (device, dtype,
contiguity), and launches on torch's current stream, so launches are captured when a CUDA graph is
being recorded.  There is no fallback: if the native library cannot be built or loaded, or a kernel
refuses its sizes, a KernelError is raised.
"""

from __future__ import annotations

import contextlib
import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build
from ..errors import KernelError

_LIBS: dict = {}
_VERBOSE_BUILD = True

_SIGNATURES = {
    "core": {
        "mir_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "mir_rms_norm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "mir_silu_mul": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "mir_add_bias": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "mir_cast": [c_int, c_void_p, c_void_p, c_size_t, c_void_p],
        "mir_qk_rope_store": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mir_paged_attention_generic": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                        c_void_p],
        "mir_gemm_f32": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                         c_void_p],
        "mir_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                       c_void_p, c_int, c_void_p],
        "mir_repetition_penalty": [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mir_decode_prepare": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "mir_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
    },
    "bf16": {
        "mir_decode_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                      c_longlong, c_void_p],
        "mir_decode_attention_paged_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                            c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_int, c_void_p, c_longlong, c_void_p],
        "mir_decode_attention_tc_takes": [c_int, c_int, c_int],
        "mir_head_logits_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_int, c_void_p, c_size_t, c_void_p, c_void_p],
        "mir_gemm_tc_stream_head_candidates": [c_int],
        "mir_decode_partition_keys": [c_int, c_int, c_int, c_int, c_int, c_int],
        "mir_decode_attention_plan": [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "mir_decode_attention_tc_error": [],
        "mir_prefill_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mir_prefill_attention_tc_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                          c_void_p],
        "mir_prefill_attention_tc_takes": [c_int, c_int],
        "mir_prefill_attention_tc_error": [],
        "mir_prefill_attention_tc_set_streams": [c_int],
        "mir_prefill_attention_tc_set_shared": [c_int],
        "mir_gemm_tc_stream_bf16": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mir_gemm_tc_stream_error": [],
        "mir_gemm_tc_stream_set_splits": [c_int, c_int, c_int],
        "mir_gemm_tc_bf16": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_void_p],
        "mir_gemm_tc_set_width": [c_int],
        "mir_gemm_tc_error": [],
        "mir_linear_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_void_p,
                            c_void_p],
        "mir_gate_up_silu_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float,
                                  c_void_p, c_void_p, c_size_t, c_void_p],
        "mir_set_option": [ctypes.c_char_p, c_int],
        "mir_get_option": [ctypes.c_char_p],
        "mir_gemm_bf16_lt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_void_p, c_size_t, c_void_p],
    },
}


def set_build_verbosity(verbose: bool) -> None:
    global _VERBOSE_BUILD
    _VERBOSE_BUILD = verbose


_TRACED = False


def use_traced_kernels() -> None:
    """Load the bfloat16 library with time stamps inside its kernels (csrc/trace.cuh) instead of the plain one.
    To be called before the first bfloat16 kernel runs; read_trace() returns what they recorded."""
    global _TRACED
    if "bf16" in _LIBS and not _TRACED:
        raise KernelError("use_traced_kernels: the plain bfloat16 library is loaded already")
    _TRACED = True


def read_trace() -> dict:
    """The records of the traced kernels since the last call, per group ("stream", "decode", "merge", "rope"):
    int64 arrays [records, 16] of %globaltimer nanoseconds (0 = not reached), [:, 14] a value, [:, 15] a tag; the
    sources say which time stamp is what.  Synchronises the device."""
    import numpy as np
    _require(_TRACED, "read_trace: call use_traced_kernels() first")
    lib = library("bf16")
    capacity = 4096
    host = (ctypes.c_ulonglong * (16 * capacity))()
    records = {}
    for group in ("stream", "decode", "merge", "rope"):
        reader = getattr(lib, f"mir_trace_read_{group}")
        reader.argtypes = [c_void_p, c_int]
        reader.restype = c_int
        count = reader(host, capacity)
        _require(count >= 0, f"read_trace: reading the {group} records failed")
        records[group] = np.array(host[: count * 16], dtype=np.uint64).reshape(count, 16).astype(np.int64)
    return records


def read_prompt_attention_trace():
    """Cycle stamps of the first CTA of the last tcgen05 prompt-attention launch (traced kernels only): an int64 array
    [256, 16]; row g is the CTA's g-th key tile, rows 200 + n the end of its n-th item; csrc/attention_tc.cu says
    which column is what.  0 = not reached.  Synchronises the device."""
    import numpy as np
    _require(_TRACED, "read_prompt_attention_trace: call use_traced_kernels() first")
    lib = library("bf16")
    rows = 256
    host = (ctypes.c_longlong * (16 * rows))()
    lib.mir_trace_read_prompt_tiles.argtypes = [c_void_p, c_int]
    lib.mir_trace_read_prompt_tiles.restype = c_int
    count = lib.mir_trace_read_prompt_tiles(host, rows)
    _require(count == rows, "read_prompt_attention_trace: reading the records failed")
    return np.array(host, dtype=np.int64).reshape(rows, 16)


def library(name: str) -> ctypes.CDLL:
    """The loaded native library `name`, compiled first if its sources changed or it was never built."""
    lib = _LIBS.get(name)
    if lib is not None:
        return lib
    path = _build.build("bf16_trace" if name == "bf16" and _TRACED else name, verbose=_VERBOSE_BUILD)
    try:
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)
    except OSError as error:
        raise KernelError(f"cannot load {path}: {error}") from error
    lib.mir_last_error.restype = ctypes.c_char_p
    lib.mir_last_error.argtypes = []
    for symbol, argtypes in _SIGNATURES.get(name, {}).items():
        function = getattr(lib, symbol)
        function.argtypes = argtypes
        function.restype = c_int
    _LIBS[name] = lib
    return lib


def set_programmatic_launch(mode) -> None:
    """How kernels are launched: 0 / False plainly; 1 / True all with programmatic stream serialization (a
    kernel's start overlaps the previous kernel's end; every kernel waits for its predecessor before it touches
    activations); 2 only the weight-streaming products, whose first weights are then on their way while the
    kernel before them drains."""
    for name in ("core", "bf16"):
        lib = library(name)
        lib.mir_set_pdl.argtypes = [c_int]
        lib.mir_set_pdl.restype = None
        lib.mir_set_pdl(int(mode))


def launch_counts(reset: bool = False) -> dict:
    """How often each kernel of the loaded libraries was launched, by the name its launcher gives
    ("decode_attention", "prefill_attention_tc", "paged_attention_generic", "tc_stream", "gemm_bf16_lt", ...).
    A launch recorded into a CUDA graph counts once, however often the graph is replayed."""
    counts: dict = {}
    for lib in _LIBS.values():
        lib.mir_launch_counts.argtypes = [ctypes.c_char_p, c_int]
        lib.mir_launch_counts.restype = c_int
        buffer = ctypes.create_string_buffer(lib.mir_launch_counts(None, 0))
        lib.mir_launch_counts(buffer, len(buffer))
        for line in buffer.value.decode().splitlines():
            name, _, count = line.partition("=")
            counts[name] = counts.get(name, 0) + int(count)
        if reset:
            lib.mir_reset_launch_counts.argtypes = []
            lib.mir_reset_launch_counts.restype = None
            lib.mir_reset_launch_counts()
    return counts


def loaded_libraries() -> dict:
    """Paths of the native libraries this process has loaded (for reports)."""
    return {name: lib._name for name, lib in _LIBS.items()}


# Whether an RMSNorm between two few-rows products is folded into them (NormedResidual): the product before it
# leaves the sums of squares and the weighted rows, the product after it scales its results.  Two kernels fewer
# per layer in a decode step.
FUSE_NORM_INTO_PRODUCT = True
# Whether layers of the built-in kind are run by the native executor (csrc/executor.cu), one call per run of such
# layers; False runs every layer part by part from Python (the same kernels, launched from the interpreter).
NATIVE_LAYERS = True
REPLAYED_LAUNCHES = 0   # launches that ran as part of replayed CUDA graphs (a replay counts what its capture counted)


def launches() -> int:
    """Kernels and library products launched so far by this process's native libraries, replays of captured graphs
    included (for reports)."""
    return sum(launch_counts().values()) + REPLAYED_LAUNCHES


MIR_CANNOT_FOLD = 4     # a product was given a folded norm's rows that it cannot take over (launchers.h)


def set_option(name: str, value: int) -> None:
    """A threshold of the bfloat16 product dispatch (csrc/ops_bf16.cu): few_rows_max, folded_norm_max_rows,
    tensor_core_min_rows, few_rows_modes (bits: store, accumulate, float32, SwiGLU), decode_tensor_cores,
    decode_partition_keys, decode_tc_partition_keys."""
    lib = library("bf16")
    _check(lib, lib.mir_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(library("bf16").mir_get_option(name.encode()))


@contextlib.contextmanager
def option(name: str, value: int):
    """An option of the native dispatch set for the duration of a `with` block (measurements, tests)."""
    before = get_option(name)
    set_option(name, value)
    try:
        yield
    finally:
        set_option(name, before)


def _check(lib: ctypes.CDLL, status: int) -> None:
    if status != 0:
        raise KernelError(lib.mir_last_error().decode(errors="replace") or f"kernel launch failed with status {status}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle (asked for at every launch, so by the short way where torch has one)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _is_bf16(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {tensor.dtype}")


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise KernelError(message)


def _cuda(*tensors) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("kernels take CUDA tensors only: there is no CPU path")


# --------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[r] = float(table[ids[r]]) * scale; out is the 32-bit residual [rows, hidden]."""
    _cuda(table, ids, out)
    rows, hidden = out.shape
    _require(table.is_contiguous() and out.is_contiguous() and ids.dtype == torch.int32 and ids.numel() == rows
             and out.dtype == torch.float32 and table.shape[1] == hidden, "embed: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_embed(_is_bf16(table), table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, hidden,
                              table.shape[0], scale, _stream()))


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight; x and weight are 32-bit."""
    _cuda(x, weight, out, rows)
    n_rows, hidden = out.shape
    _require(x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
             and x.shape[1] == hidden and weight.numel() == hidden, "rms_norm: bad arguments")
    if rows is not None:
        _require(rows.dtype == torch.int32 and rows.numel() == n_rows, "rms_norm: bad row index")
    else:
        _require(x.shape[0] >= n_rows, "rms_norm: fewer input rows than output rows")
    lib = library("core")
    _check(lib, lib.mir_rms_norm(_is_bf16(out), x.data_ptr(), weight.data_ptr(), out.data_ptr(), _ptr(rows), n_rows,
                                 hidden, eps, _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, I + c]."""
    _cuda(gate_up, out)
    rows, inter = out.shape
    _require(gate_up.shape == (rows, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous()
             and gate_up.dtype == out.dtype, "silu_mul: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_silu_mul(_is_bf16(out), gate_up.data_ptr(), out.data_ptr(), rows, inter, _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    _cuda(x, bias)
    rows, cols = x.shape
    _require(x.dtype == torch.float32 and x.is_contiguous() and bias.numel() == cols, "add_bias: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_add_bias(_is_bf16(bias), x.data_ptr(), bias.data_ptr(), rows, cols, _stream()))


CAST_KINDS = {(torch.float32, torch.bfloat16): 0, (torch.bfloat16, torch.float32): 1, (torch.float16, torch.bfloat16): 2,
              (torch.float16, torch.float32): 3}


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """Copy of equal shapes between what a checkpoint stores and what the engine keeps: float32 <-> bfloat16,
    float16 -> bfloat16 or float32 (load-time casts, libmir dense_cast.cu)."""
    _cuda(src, dst)
    _require(src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel(), "cast: bad arguments")
    kind = CAST_KINDS.get((src.dtype, dst.dtype))
    _require(kind is not None, f"cast: {src.dtype} -> {dst.dtype} is not supported")
    lib = library("core")
    _check(lib, lib.mir_cast(kind, src.data_ptr(), dst.data_ptr(), src.numel(), _stream()))


def random_normal(out: torch.Tensor, seed: int, deviation: float) -> None:
    """out (contiguous float32 or bfloat16, on the device) = deviation x normal deviates that depend on `seed` and
    the element's index only."""
    _cuda(out)
    _require(out.is_contiguous() and out.dtype in (torch.float32, torch.bfloat16), "random_normal: bad arguments")
    lib = library("core")
    lib.mir_random_normal.argtypes = [c_int, c_void_p, c_size_t, ctypes.c_ulonglong, c_float, c_void_p]
    lib.mir_random_normal.restype = c_int
    _check(lib, lib.mir_random_normal(int(out.dtype == torch.bfloat16), out.data_ptr(), out.numel(),
                                      seed & ((1 << 64) - 1), float(deviation), _stream()))


def decode_prepare(positions, block_table, page_size, slot_mapping, context_lens) -> None:
    """slot_mapping[r] and context_lens[r] of a decode batch from positions and block tables (on the device)."""
    rows = positions.numel()
    lib = library("core")
    _check(lib, lib.mir_decode_prepare(positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
                                       slot_mapping.data_ptr(), context_lens.data_ptr(), rows, _stream()))


def decode_advance(sampled, tokens, positions, token_log, step_counter) -> None:
    """tokens <- sampled, positions += 1, token_log[step] <- sampled, step += 1 (on the device)."""
    rows = tokens.numel()
    lib = library("core")
    _check(lib, lib.mir_decode_advance(sampled.data_ptr(), tokens.data_ptr(), positions.data_ptr(),
                                       token_log.data_ptr(), token_log.shape[0], step_counter.data_ptr(), rows,
                                       _stream()))


# --------------------------------------------------------------------------- attention
def qk_rope_store(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                  k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int, rotary_dim: int, eps: float, write_kv: bool = True,
                  keys_in_place: bool = False) -> None:
    """q/k-norm + rotary on the packed qkv rows in place for q, k and v into their pages.  `keys_in_place`:
    the keys are normed and rotated in place like the queries and nothing is written to the pages."""
    write_kv = write_kv and not keys_in_place
    _cuda(qkv, positions, slot_mapping, inv_freq, q_norm, k_norm, k_pages, v_pages)
    tokens = qkv.shape[0]
    _require(qkv.is_contiguous() and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim, "qk_rope_store: bad qkv")
    _require(positions.dtype == torch.int32 and positions.numel() >= tokens, "qk_rope_store: bad positions")
    _require(head_dim % 8 == 0, f"qk_rope_store: head_dim {head_dim} is not a multiple of 8")
    if rotary_dim:
        _require(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
                 "qk_rope_store: the angle table must hold rotary_dim / 2 float32 values")
    for norm in (q_norm, k_norm):
        _require(norm is None or (norm.dtype == torch.float32 and norm.numel() == head_dim),
                 "qk_rope_store: q/k norm weights must be float32 [head_dim]")
    if write_kv:
        _require(slot_mapping is not None and slot_mapping.dtype == torch.int32 and k_pages is not None
                 and v_pages is not None and k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype,
                 "qk_rope_store: cache pages of the activations' dtype and a slot mapping are needed")
    lib = library("core")
    _check(lib, lib.mir_qk_rope_store(_is_bf16(qkv), qkv.data_ptr(), positions.data_ptr(), _ptr(slot_mapping),
                                      _ptr(inv_freq), _ptr(q_norm), _ptr(k_norm), _ptr(k_pages), _ptr(v_pages),
                                      tokens, heads, kv_heads, head_dim, rotary_dim, eps,
                                      2 if keys_in_place else int(write_kv), _stream()))


def paged_attention_generic(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, row_of_token: torch.Tensor, positions: torch.Tensor,
                            page_size: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                            window: Optional[int]) -> None:
    """out[t, h] = softmax over the visible cached keys of token t's request; q is read from the packed qkv rows."""
    _cuda(qkv, out, k_pages, v_pages, block_table, row_of_token, positions)
    tokens = out.shape[0]
    _require(out.is_contiguous() and out.shape[1] == heads * head_dim and qkv.dtype == out.dtype
             and k_pages.dtype == out.dtype and v_pages.dtype == out.dtype, "paged_attention: bad tensors")
    _require(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
             and row_of_token.dtype == torch.int32 and positions.dtype == torch.int32, "paged_attention: bad metadata")
    lib = library("core")
    _check(lib, lib.mir_paged_attention_generic(
        _is_bf16(out), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], row_of_token.data_ptr(), positions.data_ptr(), tokens,
        page_size, heads, kv_heads, head_dim, scale, int(window or 0), _stream()))


FAST_HEAD_DIMS = (64, 128)      # what the tensor-core attention kernels take; other sizes use the reference kernel


def decode_attention_plan(rows: int, heads: int, kv_heads: int, head_dim: int, page_size: int, max_context: int) -> tuple:
    """(keys per partition, partitions, floats of scratch) for the attention of `rows` single tokens whose longest
    context (or block-table width) is max_context keys.  The plan is native (csrc/ops_bf16.cu:
    mir_decode_attention_plan), the same for the Python launcher and the layer executor: the tcgen05 kernel where
    it takes the sizes (partitions chosen by the cost of its waves, or decode_tc_partition_keys), else the mma.sync
    kernel with partitions of decode_partition_keys."""
    partition, count, floats = ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    lib = library("bf16")
    _check(lib, lib.mir_decode_attention_plan(rows, heads, kv_heads, head_dim, page_size, max_context,
                                              ctypes.byref(partition), ctypes.byref(count), ctypes.byref(floats)))
    return partition.value, count.value, floats.value


def decode_attention_scratch_floats(rows: int, heads: int, head_dim: int, num_partitions: int) -> int:
    """What the kernels that take one partition per CTA want (decode_attention_plan says what a call will use)."""
    return 0 if num_partitions <= 1 else rows * heads * num_partitions * (head_dim + 2)


def decode_attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor, page_size: int, heads: int, kv_heads: int,
                     head_dim: int, scale: float, window: Optional[int], partition: int, num_partitions: int,
                     scratch: Optional[torch.Tensor]) -> None:
    """bf16 split-KV attention for a batch of single tokens (row r of qkv belongs to request row r)."""
    _cuda(qkv, out, k_pages, v_pages, block_table, positions, scratch)
    rows = out.shape[0]
    _require(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
             and v_pages.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == heads * head_dim,
             "decode_attention: bfloat16 tensors are needed")
    _require(block_table.dtype == torch.int32 and block_table.is_contiguous() and positions.dtype == torch.int32
             and positions.numel() >= rows and block_table.shape[0] >= rows, "decode_attention: bad metadata")
    _require(scratch is None or scratch.dtype == torch.float32, "decode_attention: scratch must be float32")
    lib = library("bf16")
    _require(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[0] == v_pages.shape[0],
             "decode_attention: the cache tensors must be contiguous [token rows, kv_heads, head_dim]")
    _check(lib, lib.mir_decode_attention_paged_bf16(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), rows, page_size, heads, kv_heads, head_dim,
        scale,
        int(window or 0), partition, num_partitions, _ptr(scratch), 0 if scratch is None else scratch.numel(),
        _stream()))


# Whether prompt portions run the tcgen05 attention kernel where it takes the sizes (head_dim 128, pages of 8 to
# 128 keys that divide 128) and the portions average at least PREFILL_TENSOR_CORE_MIN_PORTION tokens.
PREFILL_TENSOR_CORES = True
PREFILL_TENSOR_CORE_MIN_PORTION = 32


def prefill_attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, query_starts: torch.Tensor, context_lens: torch.Tensor,
                      page_size: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                      window: Optional[int], tensor_cores: Optional[bool] = None,
                      portion_tokens: Optional[int] = None) -> None:
    """bf16 tensor-core attention for any mix of portions (row r owns tokens query_starts[r]..query_starts[r+1]
    of the packed qkv and out; the rows may be a part of the batch, `portion_tokens` then says how many tokens
    they have together).  `tensor_cores`: True runs the tcgen05 kernel, False the mma.sync kernel, None chooses."""
    _cuda(qkv, out, k_pages, v_pages, block_table, query_starts, context_lens)
    tokens = out.shape[0]
    rows = context_lens.numel()
    _require(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
             and v_pages.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == heads * head_dim,
             "prefill_attention: bfloat16 tensors are needed")
    _require(block_table.dtype == torch.int32 and block_table.is_contiguous() and query_starts.dtype == torch.int32
             and context_lens.dtype == torch.int32 and query_starts.numel() == rows + 1
             and block_table.shape[0] >= rows, "prefill_attention: bad metadata")
    lib = library("bf16")
    if tensor_cores is None:
        portion_tokens = tokens if portion_tokens is None else portion_tokens
        tensor_cores = (PREFILL_TENSOR_CORES and portion_tokens >= PREFILL_TENSOR_CORE_MIN_PORTION * rows
                        and bool(lib.mir_prefill_attention_tc_takes(head_dim, page_size))
                        and k_pages.is_contiguous() and v_pages.is_contiguous() and scale > 0)
    if tensor_cores:
        _require(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape,
                 "prefill_attention: the tcgen05 kernel reads contiguous [rows, kv_heads, head_dim] pages")
        _check(lib, lib.mir_prefill_attention_tc_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
            block_table.data_ptr(), block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows, tokens,
            page_size, heads, kv_heads, head_dim, scale, int(window or 0), _stream()))
        return
    _check(lib, lib.mir_prefill_attention_bf16(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows, tokens, page_size, heads,
        kv_heads, head_dim, scale, int(window or 0), _stream()))


def set_prefill_softmax_streams(streams: int) -> None:
    """For measurements: over how many softmax streams the tcgen05 attention splits a row's key tiles, 1 or 2."""
    lib = library("bf16")
    _check(lib, lib.mir_prefill_attention_tc_set_streams(int(streams)))


def set_prefill_shared_reference(shared: bool) -> None:
    """For measurements: whether the two softmax streams of the tcgen05 prompt attention share a row's reference and
    one output accumulator (the default) or keep a softmax each over their tiles."""
    lib = library("bf16")
    _check(lib, lib.mir_prefill_attention_tc_set_shared(1 if shared else 0))


def decode_attention_error() -> int:
    """0 unless a bounded wait of the tcgen05 decode attention kernel ran out (synchronises the device)."""
    return int(library("bf16").mir_decode_attention_tc_error())


def decode_attention_takes_tensor_cores(head_dim: int, page_size: int, partition: int) -> bool:
    """Whether single decoded tokens of these sizes run the tcgen05 kernel (and the option decode_tensor_cores is on)."""
    lib = library("bf16")
    return bool(lib.mir_get_option(b"decode_tensor_cores")) and \
        bool(lib.mir_decode_attention_tc_takes(head_dim, page_size, partition))


def prefill_attention_error() -> int:
    """0, or which role of the tcgen05 attention gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_prefill_attention_tc_error())


# --------------------------------------------------------------------------- matrix products
_LT_WORKSPACE: dict = {}
LT_WORKSPACE_BYTES = 64 * 1024 * 1024


def _lt_workspace(device) -> torch.Tensor:
    key = (device.type, device.index)
    buffer = _LT_WORKSPACE.get(key)
    if buffer is None:
        buffer = torch.empty(LT_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _LT_WORKSPACE[key] = buffer
    return buffer


class NormedResidual:
    """An RMSNorm of the 32-bit residual stream that is folded into the few-rows products around it.
    `weighted` holds bf16(residual * norm weight) and `sumsq`, per 16-column tile of the residual and per token,
    the sum of squares; both were written by the product that last updated the residual.  The product that takes
    this as its x multiplies each token's results by rsqrt(mean of squares + eps).  Anything else that needs the
    normed rows calls `materialize`."""

    def __init__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, sumsq: torch.Tensor, tiles: int,
                 dtype: torch.dtype, weighted: torch.Tensor):
        self.residual, self.weight, self.eps, self.sumsq, self.tiles, self.dtype = residual, weight, eps, sumsq, tiles, dtype
        self.weighted = weighted
        self.shape = residual.shape

    def materialize(self, alloc) -> torch.Tensor:
        out = alloc(tuple(self.residual.shape), self.dtype)
        rms_norm(self.residual, self.weight, self.eps, out)
        return out


def sumsq_tiles(columns: int) -> int:
    """How many 16-column tiles the accumulate epilogue writes sums of squares for."""
    return -(-columns // 16)


def linear(x, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           accumulate: bool = False, sumsq_out: Optional[torch.Tensor] = None, alloc=None,
           weighted_out: Optional[tuple] = None) -> bool:
    """out = (out if accumulate) + x . weight^T (+ bias).

    float32 tensors: the 32-bit FMA kernel.  bfloat16 x and weight: the native dispatch (csrc/ops_bf16.cu) runs up
    to few_rows_max (32) rows on the weight-streaming kernel and more on cuBLASLt, both with 32-bit accumulation;
    out is bfloat16 or float32.  x and out may be row-strided views; weight is [out_features, in_features].  x may
    be a NormedResidual (then `alloc` must be given in case it has to be materialised).  With `sumsq_out` (float32
    [ceil(N / 16), NORM_STAT_STRIDE]) and `weighted_out` = (bfloat16 [M, N], float32 norm weight [N]) an
    accumulating few-rows product also writes the sums of squares of the rows it updates and those rows times the
    weight; the return value says whether it did."""
    lazy = x if isinstance(x, NormedResidual) else None
    rows = lazy.weighted if lazy is not None else x
    _cuda(rows, weight, out, bias)
    m, k = rows.shape
    n = weight.shape[0]
    _require(weight.shape[1] == k and out.shape == (m, n) and rows.stride(1) == 1 and out.stride(1) == 1
             and weight.is_contiguous(), "linear: shapes or strides do not fit")
    if rows.dtype == torch.float32:
        _require(weight.dtype == torch.float32 and out.dtype == torch.float32
                 and (bias is None or bias.dtype == torch.float32), "linear: float32 takes float32 everywhere")
        lib = library("core")
        _check(lib, lib.mir_gemm_f32(x.data_ptr(), x.stride(0), weight.data_ptr(), k, _ptr(bias), out.data_ptr(),
                                     out.stride(0), m, n, k, 1.0 if accumulate else 0.0, _stream()))
        return False
    _require(rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16, "linear: x and weight must share a dtype")
    _require(out.dtype == torch.float32 or not accumulate, "linear: only a float32 output accumulates")
    if bias is not None and bias.dtype != out.dtype:
        _require(out.dtype == torch.float32 and accumulate, "linear: bias dtype must match out")
        add_bias(out, bias)
        bias = None
    stats, weighted, next_weight = None, None, None
    if sumsq_out is not None and weighted_out is not None and sumsq_out.numel() >= sumsq_tiles(n) * NORM_STAT_STRIDE:
        stats, (weighted, next_weight) = sumsq_out, weighted_out
        _cuda(stats, weighted, next_weight)
        _require(stats.dtype == torch.float32 and weighted.dtype == torch.bfloat16 and weighted.shape == (m, n)
                 and weighted.stride(1) == 1 and next_weight.dtype == torch.float32 and next_weight.numel() == n
                 and next_weight.is_contiguous(), "linear: weighted rows are bfloat16 [M, N], the weight float32 [N]")
    lib = library("bf16")
    workspace = _lt_workspace(rows.device)
    wrote = c_int(0)

    def call(source, folded):
        return lib.mir_linear_bf16(
            source.data_ptr(), source.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0),
            int(out.dtype == torch.float32), int(accumulate), m, n, k,
            folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
            folded.eps if folded is not None else 0.0, _ptr(stats), _ptr(next_weight), _ptr(weighted),
            weighted.stride(0) if weighted is not None else 0, workspace.data_ptr(), workspace.numel(), _stream(),
            ctypes.addressof(wrote))

    status = call(rows, lazy)
    if status == MIR_CANNOT_FOLD and lazy is not None:
        status = call(lazy.materialize(alloc), None)
    _check(lib, status)
    return bool(wrote.value)


def tensor_core_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                       bias: Optional[torch.Tensor] = None, accumulate: bool = False, swiglu: bool = False) -> None:
    """The tcgen05 product for many bfloat16 rows: out = x . weight^T (+ bias) as bfloat16, or as float32
    (added to out if `accumulate`); with `swiglu`, weight is [gate rows; up rows] and
    out[M, I] = silu(x w_gate^T) * (x w_up^T) in one kernel."""
    _cuda(x, weight, out, bias)
    m, k = x.shape
    _require(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
             and weight.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == m,
             "tensor_core_linear: bfloat16 x [M, K] and weight [N, K] are needed")
    lib = library("bf16")
    if swiglu:
        inter = out.shape[1]
        _require(weight.shape[0] == 2 * inter and out.dtype == torch.bfloat16 and bias is None and not accumulate,
                 "tensor_core_linear: the SwiGLU epilogue takes [2 I, K] weights, no bias, and writes bfloat16")
        mode, n, up_offset = MODE_SWIGLU, inter, inter
    else:
        n, up_offset = weight.shape[0], 0
        _require(out.shape[1] == n and (bias is None or bias.dtype == out.dtype)
                 and (out.dtype == torch.float32 or not accumulate),
                 "tensor_core_linear: out must be [M, N]; bias shares its dtype; only float32 accumulates")
        mode = MODE_STORE if out.dtype == torch.bfloat16 else (MODE_ACCUM if accumulate else MODE_F32)
    _check(lib, lib.mir_gemm_tc_bf16(mode, x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(),
                                     out.stride(0), m, n, k, up_offset, _stream()))


def stream_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  accumulate: bool = False, swiglu: bool = False, folded: Optional["NormedResidual"] = None,
                  sumsq_out: Optional[torch.Tensor] = None, weighted_out: Optional[tuple] = None) -> None:
    """The tcgen05 weight-streaming product for 1 to 128 bfloat16 rows (see tensor_core_linear for the modes).
    `folded`: x is folded.weighted and each token's results are scaled by the folded norm; `sumsq_out`,
    `weighted_out` as in linear (accumulate, up to 32 rows)."""
    if folded is not None:
        x = folded.weighted
    _cuda(x, weight, out, bias)
    m, k = x.shape
    _require(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
             and weight.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == m
             and 0 < m <= STREAM_MAX_ROWS, "stream_linear: 1..128 bfloat16 rows x [M, K] and weight [N, K] are needed")
    lib = library("bf16")
    if swiglu:
        inter = out.shape[1]
        _require(weight.shape[0] == 2 * inter and out.dtype == torch.bfloat16 and bias is None and not accumulate,
                 "stream_linear: the SwiGLU epilogue takes [2 I, K] weights, no bias, and writes bfloat16")
        mode, n, up_offset = MODE_SWIGLU, inter, inter
    else:
        n, up_offset = weight.shape[0], 0
        _require(out.shape[1] == n and (bias is None or bias.dtype == out.dtype)
                 and (out.dtype == torch.float32 or not accumulate),
                 "stream_linear: out must be [M, N]; bias shares its dtype; only float32 accumulates")
        mode = MODE_STORE if out.dtype == torch.bfloat16 else (MODE_ACCUM if accumulate else MODE_F32)
    rows, next_weight = weighted_out if weighted_out is not None else (None, None)
    if rows is not None:
        _cuda(rows, next_weight)
        _require(rows.dtype == torch.bfloat16 and rows.shape == (m, n) and rows.stride(1) == 1
                 and next_weight.dtype == torch.float32 and next_weight.numel() == n and next_weight.is_contiguous(),
                 "stream_linear: weighted rows are bfloat16 [M, N], the norm weight float32 [N]")
    _check(lib, lib.mir_gemm_tc_stream_bf16(
        mode, x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), m, n, k,
        up_offset, folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
        folded.eps if folded is not None else 0.0, _ptr(sumsq_out), _ptr(next_weight), _ptr(rows),
        rows.stride(0) if rows is not None else 0, _stream()))


STREAM_MAX_ROWS = 128


def stream_linear_error() -> int:
    """0, or which role of the weight-streaming product gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_gemm_tc_stream_error())


def tensor_core_linear_error() -> int:
    """0, or which role of the tcgen05 product gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_gemm_tc_error())


NORM_STAT_STRIDE = 32        # tokens per row of the sums-of-squares arrays (kNormStatStride of the kernels)
MODE_STORE, MODE_ACCUM, MODE_F32, MODE_SWIGLU = 0, 1, 2, 3


def few_rows_max() -> int:
    """Up to how many rows products run the weight-streaming kernel, which can also take over RMSNorms."""
    return min(get_option("few_rows_max"), get_option("folded_norm_max_rows"), STREAM_MAX_ROWS)


def gate_up_silu(x, w_gate_up: torch.Tensor, out: torch.Tensor, scratch_alloc) -> None:
    """out[M, I] = silu(x w_gate^T) * (x w_up^T) with w_gate_up = [w_gate; w_up] of shape [2 I, K].

    bfloat16: the native dispatch (csrc/ops_bf16.cu) runs up to few_rows_max (32) rows on the weight-streaming
    kernel (x may be a NormedResidual, a norm folded into this product) and from tensor_core_min_rows (128) rows on
    the tcgen05 many-rows kernel, one kernel each, the [M, 2 I] intermediate never written; between them the library
    product followed by the SiLU-multiply kernel.  float32: the 32-bit product and that kernel.
    `scratch_alloc(shape, dtype)` provides the intermediate where one is needed."""
    lazy = x if isinstance(x, NormedResidual) else None
    rows = lazy.weighted if lazy is not None else x
    m, k = rows.shape
    inter = out.shape[1]
    _cuda(rows, w_gate_up, out)
    _require(w_gate_up.shape == (2 * inter, k) and out.shape[0] == m and out.is_contiguous()
             and w_gate_up.is_contiguous() and rows.stride(1) == 1, "gate_up_silu: shapes do not fit")
    if rows.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        gate_up = scratch_alloc((m, 2 * inter), rows.dtype)
        linear(x, w_gate_up, gate_up)
        silu_mul(gate_up, out)
        return
    _require(out.dtype == torch.bfloat16, "gate_up_silu: bfloat16 rows give a bfloat16 result")
    lib = library("bf16")
    workspace = _lt_workspace(rows.device)
    needs_scratch = get_option("few_rows_max") < m < get_option("tensor_core_min_rows") or k % 8 != 0 \
        or rows.stride(0) % 8 != 0 or rows.data_ptr() % 16 != 0

    def call(source, folded):
        scratch = scratch_alloc((m, 2 * inter), torch.bfloat16) if needs_scratch else None
        return lib.mir_gate_up_silu_bf16(
            source.data_ptr(), source.stride(0), w_gate_up.data_ptr(), out.data_ptr(), m, inter, k,
            folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
            folded.eps if folded is not None else 0.0, _ptr(scratch), workspace.data_ptr(), workspace.numel(), _stream())

    status = call(rows, lazy)
    if status == MIR_CANNOT_FOLD and lazy is not None:
        status = call(lazy.materialize(scratch_alloc), None)
    _check(lib, status)


# --------------------------------------------------------------------------- sampling
SAMPLE_OPTIONS = np.dtype([("draw", "<f8"), ("temperature", "<f4"), ("top_p", "<f4"), ("top_k", "<i4"),
                           ("pad", "<i4")])


def ranked_scratch_keys(rows: int, vocab: int) -> int:
    """How many 64-bit keys of scratch top-k / top-p sampling needs for `rows` rows."""
    padded = 1
    while padded < vocab:
        padded <<= 1
    return rows * padded


class HeadCandidates:
    """What the output head's kernel can leave beside the logits (head_logits): per row the largest finite logit of
    every 32 columns and its column.  `valid` says whether the last product that was given these buffers filled
    them; sample() then finds each row's largest logit among them instead of among the whole vocabulary."""

    def __init__(self, values: torch.Tensor, indices: torch.Tensor):
        self.values, self.indices, self.valid = values, indices, False

    @staticmethod
    def count(vocab: int) -> int:
        return -(-vocab // 128) * 4

    @classmethod
    def allocate(cls, alloc, rows: int, vocab: int) -> "HeadCandidates":
        return cls(alloc((rows, cls.count(vocab)), torch.float32), alloc((rows, cls.count(vocab)), torch.int32))


def head_logits(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                candidates: Optional[HeadCandidates] = None) -> None:
    """out[M, V] (float32) = x . weight^T, the output head.  bfloat16 rows up to few_rows_max go through the
    weight-streaming kernel, whose epilogue also fills `candidates` (and sets candidates.valid); every other case is
    linear() and leaves candidates.valid False."""
    if candidates is not None:
        candidates.valid = False
    if candidates is None or x.dtype != torch.bfloat16:
        linear(x, weight, out)
        return
    _cuda(x, weight, out, candidates.values, candidates.indices)
    m, k = x.shape
    n = weight.shape[0]
    _require(weight.dtype == torch.bfloat16 and weight.shape[1] == k and weight.is_contiguous()
             and out.dtype == torch.float32 and out.shape == (m, n) and x.stride(1) == 1 and out.stride(1) == 1,
             "head_logits: bfloat16 x [M, K] and weight [V, K], float32 out [M, V]")
    _require(candidates.values.shape == candidates.indices.shape and candidates.values.shape[0] >= m
             and candidates.values.is_contiguous() and candidates.indices.is_contiguous()
             and candidates.values.dtype == torch.float32 and candidates.indices.dtype == torch.int32,
             "head_logits: candidates are float32 values and int32 indices of one shape [rows, count]")
    lib = library("bf16")
    workspace = _lt_workspace(x.device)
    wrote = c_int(0)
    _check(lib, lib.mir_head_logits_bf16(x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), m, n,
                                         k, candidates.values.data_ptr(), candidates.indices.data_ptr(),
                                         candidates.values.shape[1], workspace.data_ptr(), workspace.numel(), _stream(),
                                         ctypes.addressof(wrote)))
    candidates.valid = bool(wrote.value)


def sample(logits: torch.Tensor, options: torch.Tensor, tokens: torch.Tensor,
           sort_keys: Optional[torch.Tensor] = None, needs_ranked: bool = False,
           candidates: Optional[HeadCandidates] = None) -> None:
    """tokens[r] = one token from row r of the 32-bit logits; options is a uint8 view of SAMPLE_OPTIONS records.
    `candidates` (valid, from the product that wrote these very logits): where each row's largest logit is found."""
    _cuda(logits, options, tokens, sort_keys)
    rows, vocab = logits.shape
    _require(logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.dtype == torch.int32
             and tokens.numel() >= rows and options.numel() * options.element_size() >= rows * SAMPLE_OPTIONS.itemsize,
             "sample: bad arguments")
    capacity = 0 if sort_keys is None else sort_keys.numel() * sort_keys.element_size() // 8
    use = candidates is not None and candidates.valid and candidates.values.shape[0] >= rows
    lib = library("core")
    _check(lib, lib.mir_sample(logits.data_ptr(), logits.stride(0), rows, vocab, options.data_ptr(), _ptr(sort_keys),
                               capacity, int(needs_ranked), tokens.data_ptr(),
                               candidates.values.data_ptr() if use else None,
                               candidates.indices.data_ptr() if use else None,
                               candidates.values.shape[1] if use else 0, _stream()))


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, id_rows: torch.Tensor,
                       penalties: torch.Tensor) -> None:
    _cuda(logits, ids, id_rows, penalties)
    rows, vocab = logits.shape
    _require(logits.dtype == torch.float32 and ids.dtype == torch.int32 and id_rows.dtype == torch.int32
             and penalties.dtype == torch.float32 and penalties.numel() >= rows and ids.numel() == id_rows.numel(),
             "repetition_penalty: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_repetition_penalty(logits.data_ptr(), logits.stride(0), vocab, ids.data_ptr(),
                                           id_rows.data_ptr(), penalties.data_ptr(), ids.numel(), _stream()))
