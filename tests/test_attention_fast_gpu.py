"""The tensor-core attention kernels (bf16, head_dim 64/128) alone against plain attention: decode split
over partitions of the keys, and portions of prompts; shuffled pages, garbage elsewhere in the pool,
windows, groups of 1 to 20 query heads per kv head, one dominant far key, the window's edge."""

import math

import numpy as np
import pytest
import torch

import plain_impl

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def cuda(t):
    return t.to("cuda")


def build_pool(ks, vs, page, rng, garbage=50.0, runs=False):
    """Scatter each request's keys/values into shuffled pages of one pool; returns pools and the tables.  With `runs`
    the pages lie one behind the other in stretches of 1 to 40 pages (a pool that is partly fragmented): the tcgen05
    prompt kernel then fetches whole tiles where it can and single pages where it cannot."""
    kv_heads, dim = ks[0].shape[1:]
    blocks = [-(-k.shape[0] // page) for k in ks]
    total = sum(blocks) + 5
    order = rng.permutation(total)
    if runs:
        starts, cursor = [], 0
        while cursor < total:
            length = int(rng.integers(1, 41))
            starts.append((cursor, min(total, cursor + length)))
            cursor += length
        order = np.concatenate([np.arange(a, b) for a, b in (starts[i] for i in rng.permutation(len(starts)))])
    k_pool = (torch.randn(total * page, kv_heads, dim) * garbage).to(BF16)
    v_pool = (torch.randn(total * page, kv_heads, dim) * garbage).to(BF16)
    table = torch.full((len(ks), max(blocks)), -1, dtype=torch.int32)
    cursor = 0
    for r, (k, v) in enumerate(zip(ks, vs)):
        for block in range(blocks[r]):
            physical = int(order[cursor]); cursor += 1
            table[r, block] = physical
            chunk = slice(block * page, min(k.shape[0], (block + 1) * page))
            n = chunk.stop - chunk.start
            k_pool[physical * page: physical * page + n] = k[chunk]
            v_pool[physical * page: physical * page + n] = v[chunk]
    return k_pool, v_pool, table


def expect(q, k, v, scale, window, rows):
    full = plain_impl.attention_scores_softmax_values(q.double(), k.double(), v.double(), scale, window)
    return full[rows]


def close(got, want, tol=2e-2):
    want, got = want.double().cpu(), got.double().cpu()
    bound = tol * max(1.0, float(want.abs().max()))
    error = float((got - want).abs().max())
    assert torch.isfinite(got).all() and error <= bound, f"max |diff| {error:.3e} > {bound:.3e}"


def decode_kernel_counts(kernels):
    counts = kernels.launch_counts()
    return counts.get("decode_attention_tc", 0), counts.get("decode_attention", 0)


@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window,partition", [
    (32, 8, 128, 16, None, 512), (32, 8, 128, 16, None, 64), (8, 8, 64, 8, None, 128), (16, 1, 128, 16, 300, 256),
    (40, 2, 64, 4, None, 64), (6, 3, 128, 32, 70, 64), (4, 4, 128, 1, None, 192), (64, 8, 128, 16, None, 128),
    (8, 2, 128, 12, None, 256), (6, 2, 64, 2, 45, 128), (40, 2, 128, 32, None, 128), (12, 4, 128, 128, 100, 256),
    (8, 2, 128, 8, None, 384), (6, 3, 128, 64, 70, 128)])
def test_decode_attention(heads, kv_heads, dim, page, window, partition, tensor_cores):
    """Both decode kernels: the tcgen05 kernel takes head_dim 128 with pages of 8..128 keys that divide 128 and
    partitions that are multiples of 128 keys (groups of 1, 3, 4, 8, 16 and 20 query heads here), the mma.sync kernel
    everything else, and everything when the option decode_tensor_cores is off."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(heads + dim)
    torch.manual_seed(heads * dim)
    lengths = [700, 1, 64, 65, 513, 16]
    scale = 0.8 / math.sqrt(dim)
    qs = [(torch.randn(n, heads, dim) * 2).to(BF16) for n in lengths]
    ks = [(torch.randn(n, kv_heads, dim) * 2).to(BF16) for n in lengths]
    vs = [torch.randn(n, kv_heads, dim).to(BF16) for n in lengths]
    # (pages in runs where the partition is 256 keys or more: the tcgen05 kernel then fetches whole tiles where it can)
    k_pool, v_pool, table = build_pool(ks, vs, page, rng, runs=partition >= 256)
    rows = len(lengths) + 2                                      # two padding rows, as in a captured batch
    q_rows = torch.cat([q[-1:] for q in qs] + [torch.zeros(2, heads, dim, dtype=BF16)]).reshape(rows, heads * dim)
    packed = torch.cat([q_rows, torch.randn(rows, 2 * kv_heads * dim).to(BF16)], dim=1).contiguous()
    positions = torch.tensor([n - 1 for n in lengths] + [-1, -1], dtype=torch.int32)
    table = torch.cat([table, torch.zeros(2, table.shape[1], dtype=torch.int32)])
    count = -(-max(lengths) // partition)
    floats = kernels.decode_attention_scratch_floats(rows, heads, dim, count)
    scratch = torch.full((max(floats, 1),), float("nan"), device="cuda")
    out = torch.full((rows, heads * dim), 9.0, device="cuda", dtype=BF16)
    takes = dim == 128 and page in (8, 16, 32, 64, 128) and partition % 128 == 0
    with kernels.option("decode_tensor_cores", int(tensor_cores)):
        assert kernels.decode_attention_takes_tensor_cores(dim, page, partition) == (takes and tensor_cores)
        before = decode_kernel_counts(kernels)
        kernels.decode_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table), cuda(positions), page, heads,
                                 kv_heads, dim, scale, window, partition, count, scratch if floats else None)
        after = decode_kernel_counts(kernels)
    assert (after[0] - before[0], after[1] - before[1]) == ((1, 0) if takes and tensor_cores else (0, 1))
    expected = torch.cat([expect(q, k, v, scale, window, slice(n - 1, n)) for q, k, v, n in zip(qs, ks, vs, lengths)])
    close(out[:len(lengths)].reshape(len(lengths), heads, dim), expected)
    if count > 1:
        assert float(out[len(lengths):].abs().max()) == 0.0     # padding rows give zeros
    assert kernels.decode_attention_error() == 0


@pytest.mark.parametrize("heads,kv_heads,dim,page,window", [
    (8, 2, 128, 16, None), (4, 4, 64, 8, None), (6, 1, 128, 16, 100), (3, 3, 64, 4, 17), (32, 8, 128, 16, None)])
def test_prefill_attention_mixed_portions(heads, kv_heads, dim, page, window):
    """Four rows in one batch: a whole 200-token prompt, a 70-token portion that starts at 333, a single
    decoded token at 129, and a 2-token portion at 64 (a page's and a tile's edge)."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(dim + heads)
    torch.manual_seed(dim + heads)
    spans = [(0, 200), (333, 403), (129, 130), (64, 66)]
    scale = 0.8 / math.sqrt(dim)
    qs = [(torch.randn(end, heads, dim) * 2).to(BF16) for _, end in spans]
    ks = [(torch.randn(end, kv_heads, dim) * 2).to(BF16) for _, end in spans]
    vs = [torch.randn(end, kv_heads, dim).to(BF16) for _, end in spans]
    k_pool, v_pool, table = build_pool(ks, vs, page, rng)
    q_rows = torch.cat([q[start:end] for q, (start, end) in zip(qs, spans)])
    tokens = q_rows.shape[0]
    packed = torch.cat([q_rows.reshape(tokens, -1), torch.randn(tokens, 2 * kv_heads * dim).to(BF16)], dim=1).contiguous()
    starts = np.cumsum([0] + [end - start for start, end in spans])
    out = torch.full((tokens, heads * dim), 9.0, device="cuda", dtype=BF16)
    kernels.prefill_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                              cuda(torch.tensor(starts, dtype=torch.int32)),
                              cuda(torch.tensor([end for _, end in spans], dtype=torch.int32)), page, heads, kv_heads,
                              dim, scale, window)
    expected = torch.cat([expect(q, k, v, scale, window, slice(start, end))
                          for q, k, v, (start, end) in zip(qs, ks, vs, spans)])
    close(out.reshape(tokens, heads, dim), expected)


@pytest.mark.parametrize("heads,kv_heads,page,window", [
    (8, 2, 16, None), (4, 4, 8, None), (6, 1, 32, 100), (3, 3, 128, 300), (32, 8, 16, None), (2, 1, 64, 129)])
@pytest.mark.parametrize("runs", [False, True])
@pytest.mark.parametrize("shared", [True, False])
def test_prefill_attention_on_tcgen05(heads, kv_heads, page, window, shared, runs):
    """The tcgen05 kernel (head_dim 128; its two softmax streams sharing a row's reference and one output accumulator,
    or each with a softmax of its own): a whole 700-token prompt, a 300-token portion that starts at 333, a single
    decoded token at 129, a 2-token portion at 64, and a 130-token portion that ends on a tile's edge."""
    from libmir_b200 import kernels
    kernels.set_prefill_shared_reference(shared)
    dim = 128
    rng = np.random.default_rng(page + heads)
    torch.manual_seed(page + heads)
    spans = [(0, 700), (333, 633), (129, 130), (64, 66), (126, 256)]
    scale = 0.8 / math.sqrt(dim)
    qs = [(torch.randn(end, heads, dim) * 2).to(BF16) for _, end in spans]
    ks = [(torch.randn(end, kv_heads, dim) * 2).to(BF16) for _, end in spans]
    vs = [torch.randn(end, kv_heads, dim).to(BF16) for _, end in spans]
    k_pool, v_pool, table = build_pool(ks, vs, page, rng, runs=runs)
    q_rows = torch.cat([q[start:end] for q, (start, end) in zip(qs, spans)])
    tokens = q_rows.shape[0]
    packed = torch.cat([q_rows.reshape(tokens, -1), torch.randn(tokens, 2 * kv_heads * dim).to(BF16)], dim=1).contiguous()
    starts = np.cumsum([0] + [end - start for start, end in spans])
    out = torch.full((tokens, heads * dim), 9.0, device="cuda", dtype=BF16)
    kernels.prefill_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                              cuda(torch.tensor(starts, dtype=torch.int32)),
                              cuda(torch.tensor([end for _, end in spans], dtype=torch.int32)), page, heads, kv_heads,
                              dim, scale, window, tensor_cores=True)
    torch.cuda.synchronize()
    kernels.set_prefill_shared_reference(True)
    assert kernels.prefill_attention_error() == 0
    expected = torch.cat([expect(q, k, v, scale, window, slice(start, end))
                          for q, k, v, (start, end) in zip(qs, ks, vs, spans)])
    close(out.reshape(tokens, heads, dim), expected)


@pytest.mark.parametrize("kind", ["decode", "decode_tcgen05", "prefill", "prefill_tcgen05"])
def test_one_far_key_among_hundreds_and_the_windows_edge(kind):
    from libmir_b200 import kernels
    heads, kv_heads, dim, page, n = 8, 2, 128, 16, 1100
    torch.manual_seed(11)
    direction = torch.randn(dim)
    direction /= direction.norm()

    def run(strong_key, window):
        k = torch.randn(n, kv_heads, dim) * 0.05
        k[strong_key] = direction * 8.0
        v = torch.randn(n, kv_heads, dim)
        q = (direction.repeat(1, heads, 1) * 8.0).to(BF16)
        k, v = k.to(BF16), v.to(BF16)
        k_pool, v_pool, table = build_pool([k], [v], page, np.random.default_rng(strong_key), garbage=0.0)
        packed = torch.cat([q.reshape(1, -1), torch.zeros(1, 2 * kv_heads * dim, dtype=BF16)], dim=1)
        out = torch.empty(1, heads * dim, device="cuda", dtype=BF16)
        if kind.startswith("decode"):
            count = -(-n // 128)
            scratch = torch.empty(kernels.decode_attention_scratch_floats(1, heads, dim, count), device="cuda")
            with kernels.option("decode_tensor_cores", int(kind == "decode_tcgen05")):
                kernels.decode_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                                         cuda(torch.tensor([n - 1], dtype=torch.int32)), page, heads, kv_heads, dim,
                                         1.0, window, 128, count, scratch)
        else:
            kernels.prefill_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                                      cuda(torch.tensor([0, 1], dtype=torch.int32)),
                                      cuda(torch.tensor([n], dtype=torch.int32)), page, heads, kv_heads, dim, 1.0,
                                      window, tensor_cores=(kind == "prefill_tcgen05"))
        return out.reshape(heads, dim).float().cpu(), v.float()

    for strong in (0, 15, 16, 63, 64, 127, 128, 600, n - 1):
        out, v = run(strong, None)
        for head in range(heads):
            assert torch.allclose(out[head], v[strong, head // 4], atol=3e-2), f"{kind}: key {strong} was not seen"
    window = 333                                                       # visible keys: n - 333 .. n - 1
    out, v = run(n - window, window)
    assert torch.allclose(out[0], v[n - window, 0], atol=3e-2), "the first key inside the window was not seen"
    out, v = run(n - window - 1, window)
    assert not torch.allclose(out[0], v[n - window - 1, 0], atol=0.3), "a key outside the window was seen"


def pool_after_poison(k_pool, v_pool, page):
    """The pools as views that start one page into larger allocations whose first page holds NaN: a kernel that
    formed an address from a block-table entry of -1 would read that page, and NaN times a zero weight is NaN."""
    def shifted(pool):
        whole = torch.full((pool.shape[0] + page,) + tuple(pool.shape[1:]), float("nan"), dtype=BF16, device="cuda")
        whole[page:] = pool.to("cuda")
        return whole[page:]
    return shifted(k_pool), shifted(v_pool)


@pytest.mark.parametrize("kind,dim,page,window,length,portion", [
    ("decode", 128, 8, 1024, 2100, 1), ("decode", 64, 4, 200, 700, 1), ("decode", 128, 4, 70, 333, 1),
    ("decode", 64, 16, 100, 1000, 1), ("decode", 128, 1, 40, 300, 1), ("decode_tcgen05", 128, 8, 1024, 2100, 1),
    ("decode_tcgen05", 128, 16, 300, 900, 1), ("decode_tcgen05", 128, 128, 200, 1000, 1),
    ("prefill", 128, 16, 1024, 2106, 10), ("prefill", 64, 16, 1024, 2106, 10),
    ("prefill", 64, 8, 100, 700, 70), ("prefill", 128, 4, 130, 450, 3), ("prefill_tcgen05", 128, 16, 1024, 2106, 40)])
def test_pages_that_a_window_has_released_are_never_read(kind, dim, page, window, length, portion):
    """The block table holds -1 for every page that lies wholly behind the window of the first query (what the cache
    manager writes when it gives such pages back), and the memory one page before the pool is NaN."""
    from libmir_b200 import kernels
    heads, kv_heads = 4, 2
    rng = np.random.default_rng(dim + page + length)
    torch.manual_seed(dim + page + length)
    scale = 0.8 / math.sqrt(dim)
    q = (torch.randn(length, heads, dim) * 2).to(BF16)
    k = (torch.randn(length, kv_heads, dim) * 2).to(BF16)
    v = torch.randn(length, kv_heads, dim).to(BF16)
    k_pool, v_pool, table = build_pool([k], [v], page, rng)
    first_query = length - portion
    first_visible = max(0, first_query + 1 - window)
    released = first_visible // page
    assert released > 2
    for block in range(released):
        physical = int(table[0, block])
        k_pool[physical * page:(physical + 1) * page] = float("nan")          # given back: someone else's now
        v_pool[physical * page:(physical + 1) * page] = float("nan")
        table[0, block] = -1
    k_dev, v_dev = pool_after_poison(k_pool, v_pool, page)
    packed = torch.cat([q[first_query:].reshape(portion, -1), torch.zeros(portion, 2 * kv_heads * dim, dtype=BF16)],
                       dim=1).contiguous()
    out = torch.full((portion, heads * dim), 9.0, device="cuda", dtype=BF16)
    if kind.startswith("decode"):
        partition = 128
        count = -(-length // partition)
        scratch = torch.full((kernels.decode_attention_scratch_floats(1, heads, dim, count),), float("nan"), device="cuda")
        with kernels.option("decode_tensor_cores", int(kind == "decode_tcgen05")):
            kernels.decode_attention(cuda(packed), out, k_dev, v_dev, cuda(table),
                                     cuda(torch.tensor([length - 1], dtype=torch.int32)), page, heads, kv_heads, dim,
                                     scale, window, partition, count, scratch)
        assert kernels.decode_attention_error() == 0
    else:
        kernels.prefill_attention(cuda(packed), out, k_dev, v_dev, cuda(table), cuda(torch.tensor([0, portion], dtype=torch.int32)),
                                  cuda(torch.tensor([length], dtype=torch.int32)), page, heads, kv_heads, dim, scale, window,
                                  tensor_cores=(kind == "prefill_tcgen05"))
        torch.cuda.synchronize()
        assert kernels.prefill_attention_error() == 0
    close(out.reshape(portion, heads, dim), expect(q, k, v, scale, window, slice(first_query, length)))


def test_fast_kernels_refuse_other_head_sizes():
    from libmir_b200 import KernelError, kernels
    z = lambda *shape: torch.zeros(*shape, device="cuda", dtype=BF16)
    meta = lambda *shape: torch.zeros(*shape, device="cuda", dtype=torch.int32)
    with pytest.raises(KernelError, match="head_dim 48 is not one of 64, 128"):
        kernels.decode_attention(z(1, 3 * 48), z(1, 48), z(16, 1, 48), z(16, 1, 48), meta(1, 1), meta(1), 16, 1, 1, 48,
                                 1.0, None, 64, 1, None)
    with pytest.raises(KernelError, match="head_dim 80 is not one of 64, 128"):
        kernels.prefill_attention(z(1, 3 * 80), z(1, 80), z(16, 1, 80), z(16, 1, 80), meta(1, 1), meta(2), meta(1), 16,
                                  1, 1, 80, 1.0, None)


@pytest.mark.parametrize("fuse_norm", [False, True])
def test_engine_uses_the_fast_kernels_and_matches_the_plain_model(tmp_path, fuse_norm, monkeypatch):
    """A model with head_dim 64 in bfloat16: prompt portions, mixed steps and graph-captured decode steps
    all run the tensor-core kernels; logits against the plain implementation."""
    from helpers import TOL, make_folder, plain_logits, random_ids
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry, kernels
    from libmir_b200.sampling import RequestSampler
    # with fuse_norm the decode steps leave each RMSNorm to the product after it (kernels.NormedResidual)
    monkeypatch.setattr(kernels, "FUSE_NORM_INTO_PRODUCT", fuse_norm)
    config = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "intermediate_size": 320,
              "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
              "vocab_size": 500, "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
              "tie_word_embeddings": True}
    folder = make_folder(tmp_path, config, seed=5, dtype="bfloat16", sharpen=4.0)
    rng = np.random.default_rng(0)
    first, second = random_ids(rng, 500, 900), random_ids(rng, 500, 300)
    ref_first, ref_second = plain_logits(folder, first), plain_logits(folder, second)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=16, block_count=128), dtype="bfloat16")).load(folder)
    model.admit("a"); model.admit("b")

    def check(got, want, label):
        error = float(np.abs(got - want).max())
        assert error <= TOL["bfloat16"] * max(1.0, float(np.abs(want).max())), f"{label}: {error:.3e}"

    result = model.step([StepEntry("a", first[:700], [0, 350, 699])])
    check(result.logits.cpu().numpy(), ref_first[[0, 350, 699]], "whole portion")
    result = model.step([StepEntry("a", first[700:701], [0]), StepEntry("b", second[:250], [249])])
    check(result.logits.cpu().numpy(), np.stack([ref_first[700], ref_second[249]]), "mixed step")
    samplers = [RequestSampler(), RequestSampler()]
    for offset in range(40):                                           # captured decode steps, two requests
        result = model.step([StepEntry("a", [first[701 + offset]], [0]), StepEntry("b", [second[250 + offset]], [0])],
                            samplers)
        check(result.logits.cpu().numpy(), np.stack([ref_first[701 + offset], ref_second[250 + offset]]),
              f"decode step {offset}")
        assert result.tokens.cpu().tolist() == [int(np.argmax(l)) for l in result.logits.cpu().numpy()]
    assert model.runner._graphs is not None and len(model.runner._graphs.graphs) >= 1
    # a portion given before a single token: the step packs the single token first, the logits keep the given order
    result = model.step([StepEntry("b", second[290:300], [9, 0]), StepEntry("a", [first[741]], [0])])
    assert result.rows == [("b", 9), ("b", 0), ("a", 0)]
    check(result.logits.cpu().numpy(), np.stack([ref_second[299], ref_second[290], ref_first[741]]), "portion, then single")
    # 24 and 31 tokens: more than 16 rows still run the few-rows products (with the norm folded into them if it is on)
    result = model.step([StepEntry("a", first[742:766], [0, 23])])
    check(result.logits.cpu().numpy(), ref_first[[742, 765]], "a portion of 24 tokens")
    model.admit("c")
    result = model.step([StepEntry("a", first[766:767], [0]), StepEntry("c", second[:30], [29])])
    check(result.logits.cpu().numpy(), np.stack([ref_first[766], ref_second[29]]), "31 tokens in a mixed step")


@pytest.mark.parametrize("tensor_cores", [True, False])
def test_decode_attention_over_a_long_context(tensor_cores):
    """20,000 cached keys for one request beside a 3-key request: 79 partitions of 256 keys and their merge; one
    far key dominates the long request's scores for some heads."""
    from libmir_b200 import kernels
    heads, kv_heads, dim, page = 8, 2, 128, 16
    lengths = [20000, 3]
    rng = np.random.default_rng(5)
    torch.manual_seed(5)
    scale = 1.0 / math.sqrt(dim)
    qs = [torch.randn(n, heads, dim).to(BF16) for n in lengths]
    ks = [torch.randn(n, kv_heads, dim).to(BF16) for n in lengths]
    vs = [torch.randn(n, kv_heads, dim).to(BF16) for n in lengths]
    ks[0][777, 0] = (qs[0][-1, 0].float() * 3.0).to(BF16)       # head 0's query meets its own direction far back
    k_pool, v_pool, table = build_pool(ks, vs, page, rng)
    rows = len(lengths)
    q_rows = torch.cat([q[-1:] for q in qs]).reshape(rows, heads * dim)
    packed = torch.cat([q_rows, torch.zeros(rows, 2 * kv_heads * dim, dtype=BF16)], dim=1).contiguous()
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    with kernels.option("decode_tensor_cores", int(tensor_cores)):
        # (the tcgen05 kernel walks over several tiles per partition here: the far key raises its running maximum
        # after it has accumulated hundreds of keys, so what it holds in tensor memory is rescaled)
        partition, count, floats = kernels.decode_attention_plan(rows, heads, kv_heads, dim, page, max(lengths))
        assert count >= (16 if tensor_cores else 40) and (partition > 128 or not tensor_cores)
        scratch = torch.empty(floats, device="cuda")
        out = torch.empty(rows, heads * dim, device="cuda", dtype=BF16)
        kernels.decode_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table), cuda(positions), page,
                                 heads, kv_heads, dim, scale, None, partition, count, scratch)
    assert kernels.decode_attention_error() == 0
    expected = torch.cat([expect(q, k, v, scale, None, slice(n - 1, n)) for q, k, v, n in zip(qs, ks, vs, lengths)])
    close(out.reshape(rows, heads, dim), expected)
    assert torch.allclose(out.reshape(rows, heads, dim)[0, 0].float().cpu(), vs[0][777, 0].float(), atol=5e-2)


@pytest.mark.parametrize("shared", [True, False])
@pytest.mark.parametrize("window", [None, 1000])
def test_prefill_attention_on_tcgen05_over_a_long_prompt(window, shared):
    """9,000 tokens in one portion: 71 key tiles for the last queries, shared out over both softmax streams; keys
    late in the prompt that dominate (one in an even tile, one in an odd one) raise each stream's running maximum
    after thousands of keys, which rescales what it has accumulated.  Checked on a sample of query rows."""
    from libmir_b200 import kernels
    heads, kv_heads, dim, page, n = 4, 2, 128, 16, 9000
    rng = np.random.default_rng(17)
    torch.manual_seed(17)
    scale = 1.0 / math.sqrt(dim)
    q = torch.randn(n, heads, dim).to(BF16)
    k = torch.randn(n, kv_heads, dim).to(BF16)
    v = torch.randn(n, kv_heads, dim).to(BF16)
    for key in (7000, 7000 + 128 + 5):                         # tile 54 (even) and tile 55 (odd)
        k[key, 0] = (q[8500, 0].float() * 2.0).to(BF16)        # head 0 of query 8500 looks straight at them
        k[key, 1] = (q[8990, 3].float() * 2.0).to(BF16)
    k_pool, v_pool, table = build_pool([k], [v], page, rng, runs=shared)
    packed = torch.cat([q.reshape(n, -1), torch.zeros(n, 2 * kv_heads * dim, dtype=BF16)], dim=1).contiguous()
    out = torch.full((n, heads * dim), 9.0, device="cuda", dtype=BF16)
    kernels.set_prefill_shared_reference(shared)
    kernels.prefill_attention(cuda(packed), out, cuda(k_pool), cuda(v_pool), cuda(table),
                              cuda(torch.tensor([0, n], dtype=torch.int32)), cuda(torch.tensor([n], dtype=torch.int32)),
                              page, heads, kv_heads, dim, scale, window, tensor_cores=True)
    torch.cuda.synchronize()
    kernels.set_prefill_shared_reference(True)
    assert kernels.prefill_attention_error() == 0
    rows = sorted(set([0, 1, 127, 128, 129, 999, 1000, 1001, 4095, 4096, 7133, 7134, 8500, 8990, n - 1]
                      + rng.integers(0, n, 150).tolist()))
    qd, kd, vd = cuda(q).double(), cuda(k).double(), cuda(v).double()
    group = heads // kv_heads
    index = torch.tensor(rows, device="cuda")
    scores = torch.einsum("rhd,shd->rhs", qd[index], kd.repeat_interleave(group, dim=1)) * scale
    keys = torch.arange(n, device="cuda")
    visible = keys[None, :] <= index[:, None]
    if window is not None:
        visible &= keys[None, :] > index[:, None] - window
    scores = scores.masked_fill(~visible[:, None, :], float("-inf"))
    expected = torch.einsum("rhs,shd->rhd", torch.softmax(scores, dim=-1), vd.repeat_interleave(group, dim=1))
    close(out.reshape(n, heads, dim)[index], expected)
    if window is None:                                         # the two planted keys carry nearly all the weight
        planted = (v[7000, 0].float() + v[7133, 0].float()) / 2
        assert torch.allclose(out.reshape(n, heads, dim)[8500, 0].float().cpu(), planted, atol=6e-2)


def test_engine_with_a_window_on_the_fast_kernels(tmp_path):
    """head_dim 128 in bfloat16 with one sliding-window layer and one full layer: a whole portion longer than
    the window (tcgen05 kernel, pages behind the window given back), mixed steps whose single tokens run the
    split decode kernel beside a portion, and captured decode steps; logits against the plain implementation."""
    from helpers import TOL, make_folder, plain_logits, random_ids
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    from libmir_b200.sampling import RequestSampler
    config = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "intermediate_size": 192,
              "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128,
              "vocab_size": 300, "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1e5,
              "layer_types": ["sliding_attention", "full_attention"], "sliding_window": 200,
              "tie_word_embeddings": False}
    folder = make_folder(tmp_path, config, seed=9, dtype="bfloat16", sharpen=4.0)
    rng = np.random.default_rng(9)
    first, second, third = random_ids(rng, 300, 700), random_ids(rng, 300, 400), random_ids(rng, 300, 260)
    refs = {"a": plain_logits(folder, first), "b": plain_logits(folder, second), "c": plain_logits(folder, third)}
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=16, block_count=96), dtype="bfloat16")).load(folder)
    for name in ("a", "b", "c"):
        model.admit(name)

    def check(got, want, label):
        error = float(np.abs(got - want).max())
        bound = TOL["bfloat16"] * max(1.0, float(np.abs(want).max()))
        assert np.isfinite(got).all() and error <= bound, f"{label}: {error:.3e}"

    result = model.step([StepEntry("a", first[:600], [0, 199, 200, 599])])
    check(result.logits.cpu().numpy(), refs["a"][[0, 199, 200, 599]], "a portion longer than the window")
    windowed = [g for g in model.cache.groups if g.window is not None][0]
    assert windowed.pool.held < 600 // 16                       # pages behind the window were given back
    result = model.step([StepEntry("b", second[:330], [329]), StepEntry("a", first[600:601], [0])])
    check(result.logits.cpu().numpy(), np.stack([refs["b"][329], refs["a"][600]]), "portion beside a single token")
    samplers = [RequestSampler(), RequestSampler()]
    for offset in range(24):                                    # captured decode steps across a window's edge
        result = model.step([StepEntry("a", [first[601 + offset]], [0]), StepEntry("b", [second[330 + offset]], [0])],
                            samplers)
        check(result.logits.cpu().numpy(), np.stack([refs["a"][601 + offset], refs["b"][330 + offset]]),
              f"decode step {offset}")
    result = model.step([StepEntry("a", [first[625]], [0]), StepEntry("c", third[:250], [0, 249]),
                         StepEntry("b", [second[354]], [0])])
    check(result.logits.cpu().numpy(), np.stack([refs["a"][625], refs["c"][0], refs["c"][249], refs["b"][354]]),
          "two single tokens around a portion")
    assert kernels_error_flags() == (0, 0)


def kernels_error_flags():
    from libmir_b200 import kernels
    return kernels.prefill_attention_error(), kernels.stream_linear_error()
