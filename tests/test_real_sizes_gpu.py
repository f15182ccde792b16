"""The kernels at the layer sizes the benchmark times (Qwen3-4B: hidden 2,560, 32 heads / 8 KV heads of 128,
intermediate 9,728, vocabulary 151,936), each against a 32-bit product or plain attention of the same bfloat16
inputs computed on the GPU by torch (the oracle only): grids larger than the machine, persistent loops past their
first tile, clusters over the whole vocabulary.  A fault that shows only at large grids would otherwise give a
bench number and a green test suite."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16
HIDDEN, INTER, HEADS, KV_HEADS, DIM, VOCAB = 2560, 9728, 32, 8, 128, 151936
SM_COUNT = 148


def close(got, want, tol=2e-2, label=""):
    want, got = want.double(), got.double()
    bound = tol * max(1.0, float(want.abs().max()))
    error = float((got - want).abs().max())
    assert torch.isfinite(got).all() and error <= bound, f"{label}: max |diff| {error:.3e} > {bound:.3e}"


def randn(*shape, scale=1.0, seed=0):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=generator) * scale).to(BF16)


def swiglu_reference(x, w):
    inter = w.shape[0] // 2
    gate_up = x.float() @ w.float().t()
    return torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]


def test_many_rows_swiglu_product_runs_many_tiles_per_cta():
    """2,048 x (2 x 9,728) x 2,560: 16 token tiles x 76 column tiles = 1,216 tiles on 148 CTAs, so every CTA takes
    eight tiles: both accumulators, both parities of their barriers, and a ring counter that runs on across tiles."""
    from libmir_b200 import kernels
    x, w = randn(2048, HIDDEN, seed=1), randn(2 * INTER, HIDDEN, scale=0.02, seed=2)
    assert (2048 // 128) * (INTER // 128) > 4 * SM_COUNT
    out = torch.full((2048, INTER), 7.0, device="cuda", dtype=BF16)
    kernels.tensor_core_linear(x, w, out, swiglu=True)
    torch.cuda.synchronize()
    assert kernels.tensor_core_linear_error() == 0
    close(out, swiglu_reference(x, w), label="swiglu 2048 rows")


@pytest.mark.parametrize("mode", ["store", "accumulate", "swiglu"])
def test_many_rows_product_with_narrow_tiles_and_ragged_edges(mode):
    """The same persistent loop made long cheaply: 600 rows (a ragged last token tile) with tiles of 32 accumulator
    columns, several hundred tiles for 148 CTAs, at sizes that are no multiple of the tile."""
    from libmir_b200 import kernels
    lib = kernels.library("bf16")
    m, n, k = 600, 2072, 1000
    x = randn(m, k, seed=3)
    try:
        assert lib.mir_gemm_tc_set_width(32) == 0
        if mode == "swiglu":
            w = randn(2 * n, k, scale=0.05, seed=4)
            out = torch.full((m, n), 7.0, device="cuda", dtype=BF16)
            kernels.tensor_core_linear(x, w, out, swiglu=True)
            expected = swiglu_reference(x, w)
        elif mode == "store":
            w, bias = randn(n, k, scale=0.05, seed=5), randn(n, seed=6)
            out = torch.full((m, n), 7.0, device="cuda", dtype=BF16)
            kernels.tensor_core_linear(x, w, out, bias=bias)
            expected = x.float() @ w.float().t() + bias.float()
        else:
            w = randn(n, k, scale=0.05, seed=7)
            out = torch.randn(m, n, device="cuda")
            expected = out.clone() + x.float() @ w.float().t()
            kernels.tensor_core_linear(x, w, out, accumulate=True)
        torch.cuda.synchronize()
    finally:
        lib.mir_gemm_tc_set_width(0)
    assert kernels.tensor_core_linear_error() == 0
    assert (-(-m // 128)) * (n // 32) > 2 * SM_COUNT
    close(out, expected, label=f"{mode} with 32-column tiles")


@pytest.mark.parametrize("rows", [1, 8, 32])
def test_streaming_product_over_the_whole_vocabulary(rows):
    """The output head of a decode step: 151,936 x 2,560 weights (778 MB) streamed once, 32-bit logits."""
    from libmir_b200 import kernels
    x = randn(rows, HIDDEN, seed=8)
    w = randn(VOCAB, HIDDEN, scale=0.02, seed=9)
    out = torch.full((rows, VOCAB), 7.0, device="cuda")
    kernels.stream_linear(x, w, out)
    torch.cuda.synchronize()
    assert kernels.stream_linear_error() == 0
    close(out, x.float() @ w.float().t(), label=f"head, {rows} rows")


@pytest.mark.parametrize("rows", [1, 8, 32])
def test_streaming_products_of_a_layer(rows):
    """QKV (store, bias), output projection (accumulate into the residual with the sums of squares and weighted
    rows of a folded norm), gate-up (SwiGLU on a folded norm's rows) and down projection at the real widths."""
    from libmir_b200 import kernels
    qkv_width = (HEADS + 2 * KV_HEADS) * DIM
    x = randn(rows, HIDDEN, seed=10)
    w_qkv, bias = randn(qkv_width, HIDDEN, scale=0.02, seed=11), randn(qkv_width, seed=12)
    out = torch.full((rows, qkv_width), 7.0, device="cuda", dtype=BF16)
    kernels.stream_linear(x, w_qkv, out, bias=bias)
    close(out, x.float() @ w_qkv.float().t() + bias.float(), label="qkv")
    # output projection into the residual, leaving what the folded norm needs
    mixed = randn(rows, HEADS * DIM, seed=13)
    w_o = randn(HIDDEN, HEADS * DIM, scale=0.02, seed=14)
    residual = torch.randn(rows, HIDDEN, device="cuda")
    expected_residual = residual + mixed.float() @ w_o.float().t()
    norm_weight = torch.rand(HIDDEN, device="cuda") + 0.5
    tiles = kernels.sumsq_tiles(HIDDEN)
    sumsq = torch.full((tiles, kernels.NORM_STAT_STRIDE), float("nan"), device="cuda")
    weighted = torch.full((rows, HIDDEN), 7.0, device="cuda", dtype=BF16)
    kernels.stream_linear(mixed, w_o, residual, accumulate=True, sumsq_out=sumsq, weighted_out=(weighted, norm_weight))
    close(residual, expected_residual, tol=1e-3, label="output projection")
    close(sumsq[:, :rows].sum(dim=0), (expected_residual ** 2).sum(dim=1), tol=1e-3, label="sums of squares")
    close(weighted, expected_residual * norm_weight, label="weighted rows")
    # gate-up on the folded norm: results scaled by rsqrt(mean of squares + eps)
    eps = 1e-6
    folded = kernels.NormedResidual(residual, norm_weight, eps, sumsq, tiles, BF16, weighted)
    w_gate_up = randn(2 * INTER, HIDDEN, scale=0.02, seed=15)
    hidden = torch.full((rows, INTER), 7.0, device="cuda", dtype=BF16)
    kernels.stream_linear(None, w_gate_up, hidden, swiglu=True, folded=folded)
    scale = torch.rsqrt((expected_residual ** 2).mean(dim=1, keepdim=True) + eps)
    gate_up = (weighted.float() @ w_gate_up.float().t()) * scale
    close(hidden, torch.nn.functional.silu(gate_up[:, :INTER]) * gate_up[:, INTER:], label="gate-up on a folded norm")
    # down projection
    w_down = randn(HIDDEN, INTER, scale=0.02, seed=16)
    before = residual.clone()
    kernels.stream_linear(hidden, w_down, residual, accumulate=True)
    close(residual, before + hidden.float() @ w_down.float().t(), tol=1e-3, label="down projection")
    torch.cuda.synchronize()
    assert kernels.stream_linear_error() == 0


def paged_case(lengths, page, seed):
    """Keys and values of several requests scattered over shuffled pages of one pool, on the device."""
    generator = torch.Generator(device="cuda").manual_seed(seed)
    blocks = [-(-n // page) for n in lengths]
    total = sum(blocks) + 7
    order = torch.randperm(total, device="cuda", generator=generator)
    k_pool = (torch.randn(total * page, KV_HEADS, DIM, device="cuda", generator=generator) * 30).to(BF16)   # garbage
    v_pool = (torch.randn(total * page, KV_HEADS, DIM, device="cuda", generator=generator) * 30).to(BF16)
    table = torch.full((len(lengths), max(blocks)), -1, dtype=torch.int32, device="cuda")
    keys, values, cursor = [], [], 0
    for r, (n, count) in enumerate(zip(lengths, blocks)):
        k = (torch.randn(n, KV_HEADS, DIM, device="cuda", generator=generator) * 1.5).to(BF16)
        v = torch.randn(n, KV_HEADS, DIM, device="cuda", generator=generator).to(BF16)
        pages = order[cursor:cursor + count]
        cursor += count
        table[r, :count] = pages.int()
        slots = (pages[:, None] * page + torch.arange(page, device="cuda")[None, :]).reshape(-1)[:n]
        k_pool[slots], v_pool[slots] = k, v
        keys.append(k)
        values.append(v)
    return k_pool, v_pool, table, keys, values


def plain_attention(q, k, v, scale, first_position):
    """q [n, heads, dim] at positions first_position..; k, v [keys, kv_heads, dim]; 32-bit on the device."""
    group = q.shape[1] // k.shape[1]
    scores = torch.einsum("qhd,khd->hqk", q.float(), k.float().repeat_interleave(group, dim=1)) * scale
    positions = first_position + torch.arange(q.shape[0], device=q.device)
    visible = torch.arange(k.shape[0], device=q.device)[None, :] <= positions[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v.float().repeat_interleave(group, dim=1))


@pytest.mark.parametrize("tensor_cores", [True, False])
def test_decode_attention_at_batch_64(tensor_cores):
    """64 requests of 2,060 to 2,304 cached keys: 4,608 CTAs of 256 keys and the merge of nine partitions."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(3)
    lengths = [int(n) for n in rng.integers(2060, 2305, size=64)]
    lengths[5], lengths[17] = 2304, 2049
    page = 16
    k_pool, v_pool, table, keys, values = paged_case(lengths, page, seed=20)
    rows = len(lengths)
    q = randn(rows, HEADS, DIM, seed=21)
    packed = torch.cat([q.reshape(rows, -1), torch.zeros(rows, 2 * KV_HEADS * DIM, device="cuda", dtype=BF16)], dim=1)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    out = torch.full((rows, HEADS * DIM), 7.0, device="cuda", dtype=BF16)
    scale = 1.0 / math.sqrt(DIM)
    with kernels.option("decode_tensor_cores", int(tensor_cores)):
        partition, count, floats = kernels.decode_attention_plan(rows, HEADS, KV_HEADS, DIM, page, max(lengths))
        scratch = torch.full((floats,), float("nan"), device="cuda")
        kernels.decode_attention(packed, out, k_pool, v_pool, table, positions, page, HEADS, KV_HEADS, DIM, scale, None,
                                 partition, count, scratch)
    assert kernels.decode_attention_error() == 0
    expected = torch.cat([plain_attention(q[r:r + 1], keys[r], values[r], scale, lengths[r] - 1) for r in range(rows)])
    close(out.reshape(rows, HEADS, DIM), expected, label="decode attention, 64 rows")


@pytest.mark.parametrize("tensor_cores", [True, False])
def test_prompt_attention_at_2048_tokens_and_32_heads(tensor_cores):
    """One 2,048-token prompt and a 700-token portion behind 1,300 cached tokens: 32 heads x 22 query tiles of the
    tcgen05 kernel (or 32 x 44 of the mma.sync kernel), more CTAs than one wave."""
    from libmir_b200 import kernels
    page = 16
    lengths = [2048, 2000]
    spans = [(0, 2048), (1300, 2000)]
    k_pool, v_pool, table, keys, values = paged_case(lengths, page, seed=30)
    qs = [randn(end - start, HEADS, DIM, seed=31 + i) for i, (start, end) in enumerate(spans)]
    tokens = sum(q.shape[0] for q in qs)
    packed = torch.cat([torch.cat(qs).reshape(tokens, -1),
                        torch.zeros(tokens, 2 * KV_HEADS * DIM, device="cuda", dtype=BF16)], dim=1)
    starts = torch.tensor([0, qs[0].shape[0], tokens], dtype=torch.int32, device="cuda")
    context = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    out = torch.full((tokens, HEADS * DIM), 7.0, device="cuda", dtype=BF16)
    scale = 1.0 / math.sqrt(DIM)
    kernels.prefill_attention(packed, out, k_pool, v_pool, table, starts, context, page, HEADS, KV_HEADS, DIM, scale,
                              None, tensor_cores=tensor_cores)
    torch.cuda.synchronize()
    assert kernels.prefill_attention_error() == 0
    expected = torch.cat([plain_attention(q, keys[i][:end], values[i][:end], scale, start)
                          for i, (q, (start, end)) in enumerate(zip(qs, spans))])
    close(out.reshape(tokens, HEADS, DIM), expected, label="prompt attention, 2,048 tokens")


def test_one_layer_at_real_widths_against_the_plain_implementation(tmp_path):
    """A one-layer model with the real hidden, head and intermediate sizes and a small vocabulary: a 400-token
    prompt in two portions (library products, tcgen05 gate-up and prompt attention), then decoded tokens in a
    captured graph (streaming products with folded norms, split decode attention)."""
    from helpers import TOL, make_folder, plain_logits, random_ids
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    from libmir_b200.sampling import RequestSampler
    config = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": HIDDEN, "intermediate_size": INTER,
              "num_hidden_layers": 1, "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS, "head_dim": DIM,
              "vocab_size": 1000, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
              "tie_word_embeddings": True}
    folder = make_folder(tmp_path, config, seed=4, dtype="bfloat16", sharpen=3.0)
    ids = random_ids(np.random.default_rng(4), 1000, 420)
    reference = plain_logits(folder, ids)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=16, block_count=64), dtype="bfloat16")).load(folder)
    model.admit("r")

    def check(got, want, label):
        error = float(np.abs(got - want).max())
        bound = TOL["bfloat16"] * max(1.0, float(np.abs(want).max()))
        assert np.isfinite(got).all() and error <= bound, f"{label}: {error:.3e} > {bound:.3e}"

    result = model.step([StepEntry("r", ids[:300], [0, 150, 299])])
    check(result.logits.cpu().numpy(), reference[[0, 150, 299]], "first portion")
    result = model.step([StepEntry("r", ids[300:400], [0, 99])])
    check(result.logits.cpu().numpy(), reference[[300, 399]], "second portion")
    sampler = [RequestSampler()]
    for position in range(400, 420):
        result = model.step([StepEntry("r", [ids[position]], [0])], sampler)
        check(result.logits.cpu().numpy()[0], reference[position], f"decoded token at {position}")
    assert model.runner._graphs is not None and sum(g.replays for g in model.runner._graphs.graphs.values()) == 20
    from libmir_b200 import kernels
    assert (kernels.prefill_attention_error(), kernels.stream_linear_error(), kernels.tensor_core_linear_error()) == (0, 0, 0)
