"""Each kernel alone against its plain reference, at other sizes than the engine's tiny models use."""

import math

import numpy as np
import pytest
import torch

import plain_impl

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 1.6e-2}      # relative to the largest reference value


def cuda(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def close(got, want, dtype, scale=None, factor=1.0):
    want = want.double().cpu()
    got = got.double().cpu()
    bound = TOL[dtype] * factor * max(1.0, float(want.abs().max()) if scale is None else scale)
    error = float((got - want).abs().max())
    assert torch.isfinite(got).all() and error <= bound, f"max |diff| {error:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    from libmir_b200 import kernels
    torch.manual_seed(0)
    table = torch.randn(1000, 200).to(dtype)
    ids = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32)
    out = torch.empty(5, 200, device="cuda")
    kernels.embed(cuda(table), cuda(ids), out, 1.7)
    expected = plain_impl.embedding(table, ids.tolist(), 1.7)
    close(out, expected, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 5000])
def test_rms_norm_with_and_without_row_gather(dtype, hidden):
    from libmir_b200 import kernels
    torch.manual_seed(1)
    x = torch.randn(9, hidden) * 3
    weight = torch.randn(hidden)
    out = torch.empty(9, hidden, device="cuda", dtype=dtype)
    kernels.rms_norm(cuda(x), cuda(weight), 1e-3, out)
    close(out, plain_impl.rms_norm(x.double(), weight, 1e-3), dtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out = torch.empty(3, hidden, device="cuda", dtype=dtype)
    kernels.rms_norm(cuda(x), cuda(weight), 1e-3, out, cuda(rows))
    close(out, plain_impl.rms_norm(x.double()[rows.long()], weight, 1e-3), dtype)


def test_rms_norm_is_exact_to_bf16_rounding():
    """libmir's own kernel test asserts exact bf16 equality with the host formula
    (cuda/src/kernels/decoder/tests/mod.rs:10-33); the same here up to one bf16 ulp of the float64 result."""
    from libmir_b200 import kernels
    torch.manual_seed(2)
    x, weight = torch.randn(4, 256), torch.randn(256)
    out = torch.empty(4, 256, device="cuda", dtype=torch.bfloat16)
    kernels.rms_norm(cuda(x), cuda(weight), 1e-5, out)
    exact = plain_impl.rms_norm(x.double(), weight, 1e-5)
    rounded = exact.to(torch.bfloat16)
    different = (out.cpu() != rounded)
    assert different.float().mean() < 0.01            # only values that sit on a rounding boundary
    assert ((out.cpu().double() - exact).abs() <= exact.abs() * 2 ** -7).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    from libmir_b200 import kernels
    torch.manual_seed(3)
    gate_up = (torch.randn(7, 2 * 333) * 4).to(dtype)
    out = torch.empty(7, 333, device="cuda", dtype=dtype)
    kernels.silu_mul(cuda(gate_up), out)
    g, u = gate_up.double()[:, :333], gate_up.double()[:, 333:]
    close(out, plain_impl.silu(g) * u, dtype)


@pytest.mark.parametrize("m,n,k", [(1, 101, 77), (37, 130, 200), (130, 64, 16), (65, 3, 1000)])
def test_gemm_f32_is_true_32_bit(m, n, k):
    from libmir_b200 import kernels
    torch.manual_seed(4)
    x, w, bias = torch.randn(m, k), torch.randn(n, k), torch.randn(n)
    out = torch.empty(m, n, device="cuda")
    kernels.linear(cuda(x), cuda(w), out, cuda(bias))
    exact = plain_impl.linear(x.double(), w, bias)
    # float32 FMA chain over k terms: error ~ k * 6e-8 * |terms|; TF32 (10-bit mantissa) would be ~1e-3
    assert float((out.double().cpu() - exact).abs().max()) <= 2e-7 * k * float(exact.abs().max() + 1)
    base = torch.randn(m, n)
    out = cuda(base.clone())
    kernels.linear(cuda(x), cuda(w), out, accumulate=True)
    close(out, base.double() + plain_impl.linear(x.double(), w), torch.float32, factor=3)
    # a strided view as input (the q part of packed rows) and as output
    wide = torch.randn(m, k + 24)
    out_wide = torch.zeros(m, n + 8, device="cuda")
    kernels.linear(cuda(wide)[:, 8:8 + k], cuda(w), out_wide[:, :n])
    close(out_wide[:, :n], plain_impl.linear(wide.double()[:, 8:8 + k], w), torch.float32, factor=3)
    assert float(out_wide[:, n:].abs().max()) == 0.0


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    from libmir_b200 import kernels
    torch.manual_seed(5)
    x, w = cuda(torch.randn(150, 333)), cuda(torch.randn(97, 333))
    whole = torch.empty(150, 97, device="cuda")
    kernels.linear(x, w, whole)
    for begin, end in ((0, 1), (63, 66), (149, 150), (10, 140)):
        part = torch.empty(end - begin, 97, device="cuda")
        kernels.linear(x[begin:end], w, part)
        assert torch.equal(part, whole[begin:end])


@pytest.mark.parametrize("m,n,k", [(1, 136, 264), (8, 200, 72), (50, 136, 264), (300, 520, 128)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16(m, n, k, out_dtype):
    from libmir_b200 import kernels
    torch.manual_seed(6)
    x, w = torch.randn(m, k).bfloat16(), torch.randn(n, k).bfloat16()
    bias = torch.randn(n).to(out_dtype)
    out = torch.empty(m, n, device="cuda", dtype=out_dtype)
    kernels.linear(cuda(x), cuda(w), out, cuda(bias))
    exact = plain_impl.linear(x.double(), w, bias)
    close(out, exact, out_dtype if out_dtype == torch.bfloat16 else torch.float32, factor=4)
    if out_dtype == torch.float32:                         # the residual epilogue: out += x w^T
        base = torch.randn(m, n)
        out = cuda(base.clone())
        kernels.linear(cuda(x), cuda(w), out, accumulate=True)
        close(out, base.double() + plain_impl.linear(x.double(), w), torch.float32, factor=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,rotary,norm", [(3, 1, 48, 24, True), (4, 4, 16, 16, False),
                                                           (10, 5, 128, 128, True), (2, 1, 256, 64, False)])
def test_qk_norm_rope_and_cache_write(dtype, heads, kv_heads, dim, rotary, norm):
    from libmir_b200 import kernels
    torch.manual_seed(7)
    tokens, page, pages = 11, 4, 9
    qkv = torch.randn(tokens, (heads + 2 * kv_heads) * dim).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 4, 900, 901, 7, 8, 9, 10], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 7, 20, 21, -1, 0, 1, 2, 3], dtype=torch.int32)
    frequencies = plain_impl.rope_inverse_frequencies(rotary, 50000.0, None)
    q_weight = torch.randn(dim) if norm else None
    k_weight = torch.randn(dim) if norm else None
    k_pages = torch.full((pages * page, kv_heads, dim), 7.0, device="cuda", dtype=dtype)
    v_pages = torch.full((pages * page, kv_heads, dim), 7.0, device="cuda", dtype=dtype)
    device_qkv = cuda(qkv.clone())
    kernels.qk_rope_store(device_qkv, cuda(positions), cuda(slots), cuda(frequencies),
                          None if q_weight is None else cuda(q_weight), None if k_weight is None else cuda(k_weight),
                          k_pages, v_pages, heads, kv_heads, dim, rotary, 1e-4)
    wide = qkv.double()
    q = wide[:, :heads * dim].reshape(tokens, heads, dim)
    k = wide[:, heads * dim:(heads + kv_heads) * dim].reshape(tokens, kv_heads, dim)
    v = wide[:, (heads + kv_heads) * dim:].reshape(tokens, kv_heads, dim)
    if norm:
        q, k = plain_impl.rms_norm(q, q_weight, 1e-4), plain_impl.rms_norm(k, k_weight, 1e-4)
    q, k = plain_impl.rope(q, positions, frequencies), plain_impl.rope(k, positions, frequencies)
    close(device_qkv[:, :heads * dim].reshape(tokens, heads, dim), q, dtype)
    close(device_qkv[:, heads * dim:], wide[:, heads * dim:], dtype)          # k and v columns are not touched
    for token, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        close(k_pages[slot], k[token], dtype)
        close(v_pages[slot], v[token], dtype)
    untouched = sorted(set(range(pages * page)) - set(s for s in slots.tolist() if s >= 0))
    assert torch.all(k_pages[untouched] == 7.0) and torch.all(v_pages[untouched] == 7.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,rotary", [(3, 1, 48, 24), (10, 5, 128, 128), (4, 2, 16, 0)])
def test_qk_norm_rope_with_keys_in_place(dtype, heads, kv_heads, dim, rotary):
    """Keys are normed and rotated in the packed rows like the queries; values and the pages stay as they are."""
    from libmir_b200 import kernels
    torch.manual_seed(8)
    tokens = 7
    qkv = torch.randn(tokens, (heads + 2 * kv_heads) * dim).to(dtype)
    positions = torch.tensor([0, 1, 2, 400, 401, 5, 6], dtype=torch.int32)
    frequencies = plain_impl.rope_inverse_frequencies(rotary, 5000.0, None) if rotary else None
    q_weight, k_weight = torch.randn(dim), torch.randn(dim)
    pages = torch.full((8, kv_heads, dim), 7.0, device="cuda", dtype=dtype)
    device_qkv = cuda(qkv.clone())
    kernels.qk_rope_store(device_qkv, cuda(positions), None, None if frequencies is None else cuda(frequencies),
                          cuda(q_weight), cuda(k_weight), pages, pages, heads, kv_heads, dim, rotary, 1e-4,
                          keys_in_place=True)
    wide = qkv.double()
    q = plain_impl.rms_norm(wide[:, :heads * dim].reshape(tokens, heads, dim), q_weight, 1e-4)
    k = plain_impl.rms_norm(wide[:, heads * dim:(heads + kv_heads) * dim].reshape(tokens, kv_heads, dim), k_weight, 1e-4)
    if rotary:
        q, k = plain_impl.rope(q, positions, frequencies), plain_impl.rope(k, positions, frequencies)
    close(device_qkv[:, :heads * dim].reshape(tokens, heads, dim), q, dtype)
    close(device_qkv[:, heads * dim:(heads + kv_heads) * dim].reshape(tokens, kv_heads, dim), k, dtype)
    close(device_qkv[:, (heads + kv_heads) * dim:], wide[:, (heads + kv_heads) * dim:], dtype)
    assert torch.all(pages == 7.0)


def paged(k, v, page, pages_total, rng):
    """Scatter one request's keys/values [S, H, D] into shuffled pages; returns pages and its table."""
    seq = k.shape[0]
    blocks = -(-seq // page)
    order = rng.permutation(pages_total)[:blocks]
    k_pages = torch.randn(pages_total * page, *k.shape[1:], dtype=k.dtype) * 50     # garbage elsewhere
    v_pages = torch.randn(pages_total * page, *v.shape[1:], dtype=v.dtype) * 50
    for block, physical in enumerate(order):
        chunk = slice(block * page, min(seq, (block + 1) * page))
        n = chunk.stop - chunk.start
        k_pages[physical * page: physical * page + n] = k[chunk]
        v_pages[physical * page: physical * page + n] = v[chunk]
    return k_pages, v_pages, order


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,page,window", [
    (6, 3, 48, 4, None), (4, 1, 16, 16, None), (8, 8, 80, 8, 37), (32, 8, 128, 16, None), (2, 1, 256, 16, 100),
    (5, 5, 64, 1, None), (16, 2, 128, 16, 64)])
def test_paged_attention_prompt_portions_and_decoded_tokens(dtype, heads, kv_heads, dim, page, window):
    """Two requests in one batch: a portion of 40 tokens that starts at position 150 (history in the
    cache), and one decoded token at position 299.  Pages are shuffled and the rest of the pool holds
    large garbage, so a wrong page or slot shows."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(0)
    torch.manual_seed(8)
    lengths = [190, 300]
    starts = [150, 299]
    scale = 0.7 / math.sqrt(dim)
    qs, ks, vs = [], [], []
    for n in lengths:
        qs.append((torch.randn(n, heads, dim) * 2).to(dtype))
        ks.append((torch.randn(n, kv_heads, dim) * 2).to(dtype))
        vs.append(torch.randn(n, kv_heads, dim).to(dtype))
    total_pages = 2 * (300 // page + 2)
    k_pool = torch.randn(total_pages * page, kv_heads, dim).to(dtype) * 50
    v_pool = torch.randn(total_pages * page, kv_heads, dim).to(dtype) * 50
    order = rng.permutation(total_pages)
    width = -(-300 // page)
    table = torch.full((2, width), -1, dtype=torch.int32)
    cursor = 0
    for r, n in enumerate(lengths):
        blocks = -(-n // page)
        for block in range(blocks):
            physical = int(order[cursor]); cursor += 1
            table[r, block] = physical
            chunk = slice(block * page, min(n, (block + 1) * page))
            k_pool[physical * page: physical * page + chunk.stop - chunk.start] = ks[r][chunk]
            v_pool[physical * page: physical * page + chunk.stop - chunk.start] = vs[r][chunk]
    q_rows = torch.cat([qs[0][150:190], qs[1][299:300]]).reshape(41, heads * dim)
    packed = torch.cat([q_rows, torch.randn(41, 2 * kv_heads * dim).to(dtype)], dim=1).contiguous()
    positions = torch.tensor(list(range(150, 190)) + [299], dtype=torch.int32)
    rows = torch.tensor([0] * 40 + [1], dtype=torch.int32)
    out = torch.empty(41, heads * dim, device="cuda", dtype=dtype)
    kernels.paged_attention_generic(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table), cuda(rows),
                                    cuda(positions), page, heads, kv_heads, dim, scale, window)
    expected = torch.cat([
        plain_impl.attention_scores_softmax_values(qs[0].double(), ks[0].double(), vs[0].double(), scale, window)[150:190],
        plain_impl.attention_scores_softmax_values(qs[1].double(), ks[1].double(), vs[1].double(), scale, window)[299:300]])
    close(out.reshape(41, heads, dim), expected, dtype, factor=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_sees_one_far_key_among_hundreds_and_the_windows_edge(dtype):
    """Scores are made so that ONE key dominates: the output must be that key's value.  Placed at the
    first key, at a page's first and last slot, at the first key inside the window and (invisible) at the
    last key outside it."""
    from libmir_b200 import kernels
    heads, kv_heads, dim, page, n = 4, 2, 64, 16, 600
    torch.manual_seed(9)
    direction = torch.randn(dim)
    direction /= direction.norm()

    def run(strong_key, window):
        k = torch.randn(n, kv_heads, dim) * 0.05
        k[strong_key] = direction * 8.0
        v = torch.randn(n, kv_heads, dim)
        q = direction.repeat(1, heads, 1) * 8.0                      # score 64 * scale at the strong key
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        table = torch.arange(-(-n // page), dtype=torch.int32).flip(0).reshape(1, -1).contiguous()
        k_pool = torch.zeros(table.numel() * page, kv_heads, dim, dtype=dtype)
        v_pool = torch.zeros_like(k_pool)
        for block in range(table.numel()):
            physical = int(table[0, block])
            chunk = slice(block * page, min(n, (block + 1) * page))
            k_pool[physical * page: physical * page + chunk.stop - chunk.start] = k[chunk]
            v_pool[physical * page: physical * page + chunk.stop - chunk.start] = v[chunk]
        packed = torch.cat([q.reshape(1, -1), torch.zeros(1, 2 * kv_heads * dim, dtype=dtype)], dim=1)
        out = torch.empty(1, heads * dim, device="cuda", dtype=dtype)
        kernels.paged_attention_generic(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                                        cuda(torch.zeros(1, dtype=torch.int32)),
                                        cuda(torch.tensor([n - 1], dtype=torch.int32)), page, heads, kv_heads, dim,
                                        1.0, window)
        return out.reshape(heads, dim).float().cpu(), v.float()

    for strong in (0, 15, 16, 31, 300, n - 1):
        out, v = run(strong, None)
        for head in range(heads):
            assert torch.allclose(out[head], v[strong, head // 2], atol=2e-2), f"key {strong} was not seen"
    window = 100                                                      # visible keys: n - 100 .. n - 1
    out, v = run(n - window, window)
    assert torch.allclose(out[0], v[n - window, 0], atol=2e-2), "the first key inside the window was not seen"
    out, v = run(n - window - 1, window)
    assert not torch.allclose(out[0], v[n - window - 1, 0], atol=0.3), "a key outside the window was seen"


def test_kernels_refuse_sizes_they_do_not_take():
    from libmir_b200 import KernelError, kernels
    q = torch.zeros(1, 3 * 20, device="cuda")
    with pytest.raises(KernelError, match="head_dim 20"):
        kernels.paged_attention_generic(q, torch.zeros(1, 20, device="cuda"), torch.zeros(4, 1, 20, device="cuda"),
                                        torch.zeros(4, 1, 20, device="cuda"),
                                        torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                                        torch.zeros(1, dtype=torch.int32, device="cuda"),
                                        torch.zeros(1, dtype=torch.int32, device="cuda"), 4, 1, 1, 20, 1.0, None)
    with pytest.raises(KernelError, match="CUDA tensors only"):
        kernels.silu_mul(torch.zeros(1, 4), torch.zeros(1, 2))
    with pytest.raises(KernelError, match="shapes or strides"):
        kernels.linear(torch.zeros(2, 8, device="cuda"), torch.zeros(4, 9, device="cuda"),
                       torch.zeros(2, 4, device="cuda"))


# ------------------------------------------------------------------------------ sampling
def device_sample(logits, options):
    from libmir_b200 import kernels
    rows = logits.shape[0]
    host = np.zeros(rows, dtype=kernels.SAMPLE_OPTIONS)
    for r, (draw, temperature, top_k, top_p) in enumerate(options):
        host[r] = (draw, temperature, top_p, top_k, 0)
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    ranked = any(t > 1.2e-7 and k != 1 and not (k == 0 and p >= 1.0) for _, t, k, p in options)
    keys = torch.empty(kernels.ranked_scratch_keys(rows, logits.shape[1]), dtype=torch.int64, device="cuda")
    kernels.sample(cuda(logits), torch.from_numpy(host.view(np.uint8)).cuda(), tokens, keys if ranked else None,
                   ranked)
    return tokens.cpu().tolist()


@pytest.mark.parametrize("rows,vocab,hidden", [(8, 5003, 256), (1, 640, 64), (19, 33000, 128), (40, 2000, 64)])
def test_the_heads_kernel_leaves_the_candidates_for_each_rows_largest_logit(rows, vocab, hidden):
    """The output head through the weight-streaming kernel also writes, per row, the largest finite logit of every
    32 columns and its column.  The candidates must hold each row's arg max (ties to the lowest id: some vocabulary
    rows are copies of others), and sampling with them must give what sampling from the logits alone gives, greedy
    and drawn.  More than 32 rows go through the library: no candidates, the same tokens."""
    from libmir_b200 import kernels
    torch.manual_seed(vocab)
    x = (torch.randn(rows, hidden) * 0.7).bfloat16().cuda()
    weight = (torch.randn(vocab, hidden) * 0.3).bfloat16()
    copies = torch.randint(0, vocab, (vocab // 7,))
    weight[copies] = weight[(copies * 31 + 5) % vocab]                # equal logits at different ids
    weight = weight.cuda()
    logits = torch.empty(rows, vocab, device="cuda")
    candidates = kernels.HeadCandidates.allocate(lambda shape, dtype: torch.full(shape, -7, dtype=dtype, device="cuda"),
                                                 rows, vocab)
    kernels.head_logits(x, weight, logits, candidates)
    plain = torch.empty_like(logits)
    kernels.linear(x, weight, plain)
    assert torch.equal(logits, plain)
    assert candidates.valid == (rows <= kernels.few_rows_max())
    want = [int(torch.nonzero(row == row.max())[0]) for row in logits.cpu()]
    if candidates.valid:
        values, indices = candidates.values.cpu(), candidates.indices.cpu()
        groups = -(-vocab // 32)
        for r in range(rows):
            for g in range(groups):
                chunk = logits[r, 32 * g: 32 * g + 32].cpu()
                assert float(values[r, g]) == float(chunk.max())
                assert int(indices[r, g]) == 32 * g + int(torch.nonzero(chunk == chunk.max())[0])
            assert (indices[r, groups:] == 0x7fffffff).all()          # columns beyond the vocabulary: no candidate
    host = np.zeros(rows, dtype=kernels.SAMPLE_OPTIONS)
    for name, options in (("greedy", (0.0, 0.0, 1.0, 0, 0)), ("drawn", (0.37, 0.8, 1.0, 0, 0)),
                          ("top-k", (0.61, 0.9, 1.0, 20, 0))):
        host[:] = options
        device_options = torch.from_numpy(host.view(np.uint8)).cuda()
        ranked = name == "top-k"
        keys = torch.empty(kernels.ranked_scratch_keys(rows, vocab), dtype=torch.int64, device="cuda") if ranked else None
        with_candidates = torch.empty(rows, dtype=torch.int32, device="cuda")
        without = torch.empty(rows, dtype=torch.int32, device="cuda")
        kernels.sample(logits, device_options, with_candidates, keys, ranked, candidates)
        kernels.sample(logits, device_options, without, keys, ranked)
        assert with_candidates.tolist() == without.tolist(), name
        if name == "greedy":
            assert without.tolist() == want
    assert kernels.stream_linear_error() == 0


def test_greedy_ties_go_to_the_lowest_id():
    logits = torch.full((3, 5003), -1.0)
    logits[0, [4000, 17, 2500]] = 3.0
    logits[1, 5002] = 0.5
    logits[2, 0] = float("inf")
    logits[2, 9] = 2.0                                            # non-finite logits are not candidates
    assert device_sample(logits, [(0.0, 0.0, 0, 1.0)] * 3) == [17, 5002, 9]
    assert device_sample(logits, [(0.7, 0.9, 1, 1.0)] * 3) == [17, 5002, 9]       # top_k == 1 is greedy


@pytest.mark.parametrize("vocab", [5, 384, 151936])
def test_sampling_picks_what_the_plain_sampler_picks(vocab):
    rng = np.random.default_rng(vocab)
    rows = 12
    logits = torch.from_numpy(rng.normal(0, 2.5, size=(rows, vocab)).astype(np.float32))
    modes = [(0.7, 0, 1.0), (1.0, 0, 1.0), (0.3, 0, 1.0), (0.7, 5, 1.0), (0.7, 0, 0.8), (1.5, 50, 0.9),
             (0.9, 3, 0.5), (2.0, 0, 0.3), (0.7, 1000000, 0.95), (1.0, 2, 1.0), (0.5, 0, 0.999), (1.0, 64, 0.1)]
    for draws in ([0.0] * rows, rng.random(rows).tolist(), rng.random(rows).tolist(), [0.999999] * rows):
        options = [(draw, t, k, p) for draw, (t, k, p) in zip(draws, modes)]
        got = device_sample(logits, options)
        want = [plain_impl.sample(logits[r].numpy(), draw, t, k, p) for r, (draw, t, k, p) in enumerate(options)]
        assert got == want


def test_ranked_sampling_beyond_the_candidates_and_with_many_ties():
    """Ranked sampling decides most draws from the 1,024 best tokens.  Rows made so that it cannot: a flat
    distribution whose nucleus holds tens of thousands of tokens, thousands of tokens tied at the best score (the
    tie goes by lower id), a top_k wider than the candidates, and rows with few or no finite logits; every draw
    must still be the plain sampler's."""
    vocab = 40000
    rng = np.random.default_rng(3)
    flat = rng.normal(0, 0.05, size=vocab).astype(np.float32)
    tied = np.full(vocab, -2.0, dtype=np.float32)
    tied[rng.choice(vocab, size=5000, replace=False)] = 1.5            # 5,000 tokens share the best score
    peaked = rng.normal(0, 3.0, size=vocab).astype(np.float32)
    sparse = np.full(vocab, -np.inf, dtype=np.float32)
    sparse[[7, 39999, 1234]] = [0.5, 0.5, -1.0]                         # three finite logits, two of them tied
    rows = [flat, flat, tied, tied, tied, peaked, peaked, sparse, sparse]
    modes = [(1.0, 0, 0.9), (0.8, 30000, 0.999), (1.0, 0, 0.5), (0.7, 4000, 1.0), (1.0, 3, 0.9), (1.0, 3000, 1.0),
             (5.0, 0, 0.97), (1.0, 0, 0.9), (0.7, 2, 1.0)]
    logits = torch.from_numpy(np.stack(rows))
    for draws in ([0.0] * len(rows), rng.random(len(rows)).tolist(), rng.random(len(rows)).tolist(), [0.999999] * len(rows)):
        options = [(draw, t, k, p) for draw, (t, k, p) in zip(draws, modes)]
        got = device_sample(logits, options)
        want = [plain_impl.sample(logits[r].numpy(), draw, t, k, p) for r, (draw, t, k, p) in enumerate(options)]
        assert got == want, (draws[0], got, want)


def test_repetition_penalty_rewrites_the_rows_logits():
    from libmir_b200 import kernels
    logits = torch.tensor([[2.0, -1.0, 0.5, 3.0], [1.0, 1.0, -2.0, 0.0]])
    device = cuda(logits.clone())
    kernels.repetition_penalty(device, cuda(torch.tensor([3, 1, 2], dtype=torch.int32)),
                               cuda(torch.tensor([0, 0, 1], dtype=torch.int32)), cuda(torch.tensor([2.0, 1.5])))
    assert device.cpu().tolist() == [[2.0, -2.0, 0.5, 1.5], [1.0, 1.0, -3.0, 0.0]]


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16, 17, 32, 33, 64, 65])
@pytest.mark.parametrize("n,k", [(136, 264), (50, 72), (2560, 1024)])
def test_few_rows_products_and_their_epilogues(m, n, k):
    """Up to 32 bf16 rows run the tcgen05 weight-streaming kernel, more run the library: store, accumulate into
    the 32-bit residual, 32-bit output, bias, and a strided view as input."""
    from libmir_b200 import kernels
    torch.manual_seed(m * n + k)
    x, w = torch.randn(m, k).bfloat16(), (torch.randn(n, k) * 0.3).bfloat16()
    exact = plain_impl.linear(x.double(), w)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(n).bfloat16()
    kernels.linear(cuda(x), cuda(w), out, cuda(bias))
    close(out, exact + bias.double(), torch.bfloat16, factor=2)
    base = torch.randn(m, n)
    residual = cuda(base.clone())
    kernels.linear(cuda(x), cuda(w), residual, accumulate=True)
    close(residual, base.double() + exact, torch.float32, factor=40)       # bf16 products, 32-bit sums
    logits = torch.empty(m, n, device="cuda")
    kernels.linear(cuda(x), cuda(w), logits)
    close(logits, exact, torch.float32, factor=40)
    wide = cuda(torch.randn(m, k + 40).bfloat16())
    kernels.linear(wide[:, 16:16 + k], cuda(w), logits)
    close(logits, plain_impl.linear(wide[:, 16:16 + k].double().cpu(), w), torch.float32, factor=40)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,inter,k", [(1, 333, 72), (8, 9728 // 8, 320), (40, 200, 136), (64, 176, 264), (70, 96, 64),
                                       (130, 200, 136), (256, 333, 72), (300, 1216, 320)])
def test_gate_up_silu(dtype, m, inter, k):
    from libmir_b200 import kernels
    torch.manual_seed(m + inter)
    x = torch.randn(m, k).to(dtype)
    w = (torch.randn(2 * inter, k) * 0.2).to(dtype)
    out = torch.empty(m, inter, device="cuda", dtype=dtype)
    kernels.gate_up_silu(cuda(x), cuda(w), out, lambda shape, dt: torch.empty(shape, device="cuda", dtype=dt))
    gate = plain_impl.linear(x.double(), w[:inter])
    up = plain_impl.linear(x.double(), w[inter:])
    close(out, plain_impl.silu(gate) * up, dtype, factor=2)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 328, 520), (77, 100, 72), (300, 272, 1032), (129, 48, 8),
                                   (640, 1000, 264)])
def test_tensor_core_product_and_its_epilogues(m, n, k):
    """The tcgen05 products for many rows (TMA ring, accumulator in tensor memory): store with bias, accumulate into the 32-bit residual, 32-bit output, a
    strided view as input, and the SwiGLU epilogue, at sizes that are no multiples of the tiles; none of the
    bounded waits may have run out."""
    from libmir_b200 import kernels
    kernels_tensor_core_linear = kernels.tensor_core_linear
    torch.manual_seed(m + n + k)
    x, w = torch.randn(m, k).bfloat16(), (torch.randn(n, k) * 0.3).bfloat16()
    exact = plain_impl.linear(x.double(), w)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(n).bfloat16()
    kernels_tensor_core_linear(cuda(x), cuda(w), out, cuda(bias))
    close(out, exact + bias.double(), torch.bfloat16, factor=2)
    base = torch.randn(m, n)
    residual = cuda(base.clone())
    kernels_tensor_core_linear(cuda(x), cuda(w), residual, accumulate=True)
    close(residual, base.double() + exact, torch.float32, factor=40)       # bf16 products, 32-bit sums
    logits = torch.empty(m, n, device="cuda")
    float_bias = torch.randn(n)
    kernels_tensor_core_linear(cuda(x), cuda(w), logits, cuda(float_bias))
    close(logits, exact + float_bias.double(), torch.float32, factor=40)
    wide = cuda(torch.randn(m, k + 40).bfloat16())
    kernels_tensor_core_linear(wide[:, 16:16 + k], cuda(w), logits)
    close(logits, plain_impl.linear(wide[:, 16:16 + k].double().cpu(), w), torch.float32, factor=40)
    if n % 2 == 0:
        inter = n // 2
        gated = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16)
        kernels_tensor_core_linear(cuda(x), cuda(w), gated, swiglu=True)
        close(gated, plain_impl.silu(exact[:, :inter]) * exact[:, inter:], torch.bfloat16, factor=2)
    assert kernels.tensor_core_linear_error() == 0


def test_tensor_core_product_refuses_what_it_cannot_take():
    from libmir_b200 import kernels
    from libmir_b200.errors import KernelError
    x, w = cuda(torch.randn(128, 20).bfloat16()), cuda(torch.randn(64, 20).bfloat16())
    with pytest.raises(KernelError, match="multiples of 8"):
        kernels.tensor_core_linear(x, w, torch.empty(128, 64, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("m", [1, 8, 13, 24, 32])
def test_norm_folded_into_the_few_rows_products_around_it(m):
    """The accumulating product leaves the sums of squares of the new residual and its rows times the next
    norm's weight; the product after the norm scales its results: together they equal norm then product."""
    from libmir_b200 import kernels
    torch.manual_seed(m)
    hidden, inner, wide, eps = 264, 136, 200, 1e-5
    x = torch.randn(m, inner).bfloat16()
    w_in = (torch.randn(hidden, inner) * 0.3).bfloat16()
    gain = torch.rand(hidden) + 0.5
    base = torch.randn(m, hidden) * 3.0
    residual = cuda(base.clone())
    tiles = kernels.sumsq_tiles(hidden)
    sumsq = torch.zeros(tiles, kernels.NORM_STAT_STRIDE, device="cuda")
    weighted = torch.zeros(m, hidden, device="cuda", dtype=torch.bfloat16)
    wrote = kernels.linear(cuda(x), cuda(w_in), residual, accumulate=True, sumsq_out=sumsq,
                           weighted_out=(weighted, cuda(gain)))
    assert wrote
    new_residual = base.double() + plain_impl.linear(x.double(), w_in)
    close(residual, new_residual, torch.float32, factor=40)
    normed = plain_impl.rms_norm(new_residual, gain, eps)
    lazy = kernels.NormedResidual(residual, cuda(gain), eps, sumsq, tiles, torch.bfloat16, weighted)
    w_out = (torch.randn(wide, hidden) * 0.2).bfloat16()
    out = torch.empty(m, wide, device="cuda", dtype=torch.bfloat16)
    kernels.linear(lazy, cuda(w_out), out, alloc=lambda shape, dt: torch.empty(shape, device="cuda", dtype=dt))
    close(out, plain_impl.linear(normed, w_out), torch.bfloat16, factor=2)
    w_gate_up = (torch.randn(2 * wide, hidden) * 0.2).bfloat16()
    gated = torch.empty(m, wide, device="cuda", dtype=torch.bfloat16)
    kernels.gate_up_silu(lazy, cuda(w_gate_up), gated, lambda shape, dt: torch.empty(shape, device="cuda", dtype=dt))
    both = plain_impl.linear(normed, w_gate_up)
    close(gated, plain_impl.silu(both[:, :wide]) * both[:, wide:], torch.bfloat16, factor=2)
    # what cannot be folded falls back to the norm kernel
    assert torch.equal(lazy.materialize(lambda shape, dt: torch.empty(shape, device="cuda", dtype=dt)).cpu(),
                       _rms_norm_kernel(residual, gain, eps).cpu())


def _rms_norm_kernel(residual, gain, eps):
    from libmir_b200 import kernels
    out = torch.empty(residual.shape, device="cuda", dtype=torch.bfloat16)
    kernels.rms_norm(residual, cuda(gain), eps, out)
    return out


@pytest.mark.parametrize("m", [1, 8, 16, 17, 77, 128])
@pytest.mark.parametrize("n,k", [(136, 264), (50, 72), (2560, 1024), (1000, 4104)])
def test_weight_streaming_product_and_its_epilogues(m, n, k):
    """The tcgen05 product for 1 to 128 rows (weights as the A operand, K cut over a cluster): store with bias,
    accumulate into the 32-bit residual, 32-bit output, a strided view as input, the SwiGLU epilogue; sizes that
    are no multiples of its tiles; none of its bounded waits may have run out."""
    from libmir_b200 import kernels
    torch.manual_seed(m * n + k)
    x, w = torch.randn(m, k).bfloat16(), (torch.randn(n, k) * 0.3).bfloat16()
    exact = plain_impl.linear(x.double(), w)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(n).bfloat16()
    kernels.stream_linear(cuda(x), cuda(w), out, cuda(bias))
    close(out, exact + bias.double(), torch.bfloat16, factor=2)
    base = torch.randn(m, n)
    residual = cuda(base.clone())
    kernels.stream_linear(cuda(x), cuda(w), residual, accumulate=True)
    close(residual, base.double() + exact, torch.float32, factor=40)       # bf16 products, 32-bit sums
    logits = torch.empty(m, n, device="cuda")
    float_bias = torch.randn(n)
    kernels.stream_linear(cuda(x), cuda(w), logits, cuda(float_bias))
    close(logits, exact + float_bias.double(), torch.float32, factor=40)
    wide = cuda(torch.randn(m, k + 40).bfloat16())
    kernels.stream_linear(wide[:, 16:16 + k], cuda(w), logits)
    close(logits, plain_impl.linear(wide[:, 16:16 + k].double().cpu(), w), torch.float32, factor=40)
    inter = n // 2
    gated = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16)
    kernels.stream_linear(cuda(x), cuda(w[:2 * inter]), gated, swiglu=True)
    close(gated, plain_impl.silu(exact[:, :inter]) * exact[:, inter:2 * inter], torch.bfloat16, factor=2)
    assert kernels.stream_linear_error() == 0


# ------------------------------------------------------------------------------ load-time kernels
@pytest.mark.parametrize("source,target", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                           (torch.float16, torch.bfloat16), (torch.float16, torch.float32)])
def test_load_time_casts_round_as_a_conversion_does(source, target):
    from libmir_b200 import kernels
    torch.manual_seed(3)
    values = (torch.randn(3, 1001) * 5).to(source).cuda()
    values[0, :4] = torch.tensor([0.0, -0.0, 65504.0 if source == torch.float16 else 3.0e38, -1e-7]).to(source)
    out = torch.empty(values.shape, dtype=target, device="cuda")
    kernels.cast(values, out)
    assert torch.equal(out, values.to(target))


def test_random_weights_from_the_device_generator():
    """Normal deviates that depend on the seed and the element's index only: the same again for the same seed, others
    for another seed, the asked deviation, no correlation between neighbours."""
    from libmir_b200 import kernels
    a = torch.empty(1 << 20, device="cuda")
    b = torch.empty(1 << 20, device="cuda")
    kernels.random_normal(a, 12345, 0.02)
    kernels.random_normal(b, 12345, 0.02)
    assert torch.equal(a, b) and torch.isfinite(a).all()
    head = torch.empty(1000, device="cuda")
    kernels.random_normal(head, 12345, 0.02)
    assert torch.equal(head, a[:1000])                           # (no dependence on the launch's size)
    kernels.random_normal(b, 12346, 0.02)
    assert not torch.equal(a, b)
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    assert abs(float((a[1:] * a[:-1]).mean())) < 2e-6 and abs(float((a * b).mean())) < 2e-6
    assert 0.66 < float((a.abs() < 0.02).float().mean()) < 0.70   # one deviation holds 68 % of a normal
    half = torch.empty(4096, device="cuda", dtype=torch.bfloat16)
    kernels.random_normal(half, 12345, 0.02)
    assert torch.equal(half, a[:4096].bfloat16())
