"""The decode-attention entry point for callers that cannot allocate (csrc/no_alloc.h).

It keeps the partitions' partial results in an array built into the library instead of in scratch that
the caller provides.  Here it is called through its exported C symbol, twice in a row with different
inputs (the second call finds the first call's leftovers in the array), and compared with the ordinary
entry point given scratch of its own.  This file is collected last on purpose, so that a run that stops
at the first failure has already run every other test; it also passes when run alone."""

import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 2 * 1024 * 1024            # MIR_STATIC_SCRATCH_FLOATS of csrc/no_alloc.h


def entry_point():
    from libmir_b200 import kernels
    path = kernels.library("bf16")._name
    lib = ctypes.CDLL(path)                                   # the exported C symbol, not the Python launcher
    function = lib.mir_decode_attention_bf16_static
    c = ctypes
    function.argtypes = [c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p,
                         c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_float, c.c_int, c.c_int, c.c_int, c.c_void_p]
    function.restype = c.c_int
    lib.mir_last_error.restype = c.c_char_p
    return lib, function


def make_case(seed, rows, heads, kv_heads, dim, page, lengths):
    generator = torch.Generator().manual_seed(seed)
    blocks = [-(-n // page) for n in lengths]
    total = sum(blocks) + 3
    order = torch.randperm(total, generator=generator)
    k_pool = (torch.randn(total * page, kv_heads, dim, generator=generator) * 1.5).bfloat16().cuda()
    v_pool = torch.randn(total * page, kv_heads, dim, generator=generator).bfloat16().cuda()
    table = torch.zeros(rows, max(blocks), dtype=torch.int32)
    cursor = 0
    for r, count in enumerate(blocks):
        table[r, :count] = order[cursor:cursor + count].int()
        cursor += count
    qkv = torch.randn(rows, (heads + 2 * kv_heads) * dim, generator=generator).bfloat16().cuda()
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    return qkv, k_pool, v_pool, table.cuda(), positions


@pytest.mark.parametrize("dim, window", [(128, None), (64, None), (128, 200), (64, 96)])
def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row(dim, window):
    """Both entry points run the same deterministic kernels with the same launch geometry, so their results must
    be the same bits: a scratch array that is too small, or used at a wrong offset, changes some of them.  The
    second call has fewer partitions than the first, so the partial results that the first call left lie inside
    the range that a wrong merge would read."""
    from libmir_b200 import kernels
    lib, static_entry = entry_point()
    heads, kv_heads, page, partition = 16, 4, 16, 128
    scale = 1.0 / math.sqrt(dim)
    for call, lengths in enumerate([[700, 33, 512, 129], [64, 300, 17, 260]]):
        rows = len(lengths)
        qkv, k_pool, v_pool, table, positions = make_case(100 + call, rows, heads, kv_heads, dim, page, lengths)
        count = -(-max(lengths) // partition)
        floats = kernels.decode_attention_scratch_floats(rows, heads, dim, count)
        assert 0 < floats <= STATIC_FLOATS
        expected = torch.empty(rows, heads * dim, device="cuda", dtype=torch.bfloat16)
        with kernels.option("decode_tensor_cores", 0):     # the ordinary entry point of the same (mma.sync) kernel
            kernels.decode_attention(qkv, expected, k_pool, v_pool, table, positions, page, heads, kv_heads, dim, scale,
                                     window, partition, count, torch.empty(floats, device="cuda"))
        got = torch.full_like(expected, 7.0)
        status = static_entry(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                              table.data_ptr(), table.shape[1], positions.data_ptr(), rows, page, heads, kv_heads,
                              dim, scale, int(window or 0), partition, count, torch.cuda.current_stream().cuda_stream)
        assert status == 0, lib.mir_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, expected), (f"call {call}: {int((got != expected).sum())} values differ, max |diff| "
                                            f"{float((got.float() - expected.float()).abs().max()):.3e}")


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib, static_entry = entry_point()
    rows, heads, dim, count = 64, 64, 128, 16                              # 64 * 64 * 16 * 130 floats > 2 Mi
    status = static_entry(None, 0, None, None, None, None, 1, None, rows, 16, heads, 8, dim, 1.0, 0, 128, count, None)
    assert status == 1
    message = lib.mir_last_error().decode()
    assert "needs 8519680 floats" in message and "holds 2097152" in message


def test_static_scratch_entry_point_refuses_sizes_whose_product_overflows():
    """Arguments so large that rows * heads * partitions * (head_dim + 2) leaves 64 bits must be refused like any
    call that does not fit, not wrap around to a small number that passes the size check."""
    lib, static_entry = entry_point()
    huge = 2 ** 31 - 1
    for rows, heads, count in [(65535, huge - huge % 8, huge), (65536, 64, 16), (4, huge - huge % 8, huge)]:
        status = static_entry(None, 0, None, None, None, None, 1, None, rows, 16, heads, 8, 128, 1.0, 0, 128, count,
                              None)
        assert status == 1, (rows, heads, count)
