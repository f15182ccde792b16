"""The plain implementation checked against fixed points that libmir's own tests give, and against
itself computed another way (no GPU)."""

import math

import numpy as np
import torch

import plain_impl
from libmir_b200.parts.rope import inverse_frequencies
from libmir_b200.config import DecoderConfig
from libmir_b200.weights import write_model_folder
from tiny_configs import ALL, TINY_A, TINY_C


def test_llama3_frequency_table_fixed_point():
    """metal/src/engine/tests/rope.rs:4-18: dims 8, base 1e4, factor 8, low 1, high 4, original 8192
    gives periods [1, 10, 100, between 4000 and 5000]."""
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    periods = 1.0 / plain_impl.rope_inverse_frequencies(8, 10000.0, scaling).double()
    assert abs(periods[0] - 1.0) < 1e-6 and abs(periods[1] - 10.0) < 1e-5 and abs(periods[2] - 100.0) < 1e-4
    assert 4000.0 < periods[3] < 5000.0
    plain = 1.0 / plain_impl.rope_inverse_frequencies(8, 10000.0, None).double()
    assert torch.allclose(plain, torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float64), rtol=1e-6)


def test_engine_frequency_table_equals_the_plain_one():
    for config in ALL.values():
        parsed = DecoderConfig.from_dict(config)
        s = plain_impl.sizes(config)
        assert s["rotary_dim"] == parsed.rotary_dim
        ours = inverse_frequencies(parsed.rotary_dim, parsed.rope_theta, parsed.rope_scaling)
        assert torch.equal(ours, plain_impl.rope_inverse_frequencies(s["rotary_dim"], s["theta"], s["scaling"]))


def test_rms_norm_matches_the_reference_formula():
    """cuda/src/kernels/decoder/tests/mod.rs:10-33 restates x * rsqrt(sum(x^2)/n + eps) * w on the host."""
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=torch.float64)
    w = torch.tensor([1.0, 0.5, 2.0, 1.0])
    inverse = 1.0 / math.sqrt((1 + 4 + 9 + 0.25) / 4 + 1e-5)
    expected = torch.tensor([[1.0 * inverse, -2.0 * inverse * 0.5, 3.0 * inverse * 2.0, 0.5 * inverse]], dtype=torch.float64)
    assert torch.allclose(plain_impl.rms_norm(x, w, 1e-5), expected, rtol=1e-12)


def test_rope_rotates_pairs_and_keeps_the_rest():
    x = torch.zeros(2, 1, 8, dtype=torch.float64)
    x[:, 0, 0] = 1.0          # pairs with dim 2 when rotary_dim is 4
    x[:, 0, 5] = 7.0          # outside the rotary dims
    frequencies = torch.tensor([1.0, 0.5])
    y = plain_impl.rope(x, torch.tensor([0, 3]), frequencies)
    assert torch.allclose(y[0], x[0])                                    # position 0 rotates by 0
    assert abs(y[1, 0, 0] - math.cos(3.0)) < 1e-6 and abs(y[1, 0, 2] - math.sin(3.0)) < 1e-6
    assert y[1, 0, 5] == 7.0 and y[1, 0, 1] == 0.0 and y[1, 0, 3] == 0.0


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    seq, heads, kv_heads, dim = 9, 4, 2, 8
    q, k, v = (torch.randn(seq, h, dim, dtype=torch.float64) for h in (heads, kv_heads, kv_heads))
    out = plain_impl.attention_scores_softmax_values(q, k, v, 0.3, None)
    again = out.clone()
    k2, v2 = k.clone(), v.clone()
    k2[6:], v2[6:] = 0.0, 0.0                                           # the future never matters
    assert torch.allclose(plain_impl.attention_scores_softmax_values(q, k2, v2, 0.3, None)[:6], again[:6])
    # query head 3 reads kv head 1: by hand for the last position
    scores = (q[8, 3] @ k[:, 1].T) * 0.3
    assert torch.allclose(out[8, 3], torch.softmax(scores, -1) @ v[:, 1])
    windowed = plain_impl.attention_scores_softmax_values(q, k, v, 0.3, 3)
    scores = (q[8, 0] @ k[6:9, 0].T) * 0.3                              # window 3: keys 6, 7, 8
    assert torch.allclose(windowed[8, 0], torch.softmax(scores, -1) @ v[6:9, 0])
    assert torch.allclose(windowed[1], out[1])                          # shorter than the window: the same


def test_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    folder = write_model_folder(tmp_path, TINY_C, seed=5, dtype="float32")
    config, weights = plain_impl.read_model(folder)
    ids = np.random.default_rng(1).integers(0, 515, size=70).tolist()
    whole = plain_impl.forward(config, weights, ids)
    prefix = plain_impl.forward(config, weights, ids[:50])
    assert whole.shape == (70, 515) and torch.allclose(whole[:50], prefix, atol=1e-12)
    assert not torch.allclose(whole[60], plain_impl.forward(config, weights, ids[20:61])[-1], atol=1e-3)


def test_splitmix64_and_sampling_rules():
    rng = plain_impl.SplitMix64(0)
    assert rng.next_u64() == 0xE220A8397B1DCDAF and rng.next_u64() == 0x6E789E6AA1B965F4   # published vectors
    from libmir_b200.sampling import SplitMix64
    ours, theirs = SplitMix64(0x4D49524D4952), plain_impl.SplitMix64(0x4D49524D4952)
    assert [ours.next_unit() for _ in range(5)] == [theirs.next_unit() for _ in range(5)]
    logits = np.array([0.5, 2.0, 2.0, -1.0, 1.5], dtype=np.float32)
    assert plain_impl.greedy(logits) == 1                                   # lowest id on ties
    assert plain_impl.sample(logits, 0.3, 0.0) == 1 and plain_impl.sample(logits, 0.9, 1.0, top_k=1) == 1
    weights = np.exp((logits - 2.0).astype(np.float64) / 0.7)
    cumulative = np.cumsum(weights) / weights.sum()
    for draw in (0.0, 0.1, 0.35, 0.6, 0.85, 0.999):
        assert plain_impl.sample(logits, draw, 0.7) == int(np.searchsorted(cumulative, draw, side="left"))
    # ranked: order 1, 2, 4, 0, 3; top_k 2 keeps tokens 1 and 2 with equal weights
    assert plain_impl.sample(logits, 0.49, 0.7, top_k=2) == 1 and plain_impl.sample(logits, 0.51, 0.7, top_k=2) == 2
    assert plain_impl.sample(logits, 0.99, 0.7, top_p=0.3) == 1               # the first rank alone reaches 0.3
    # repetition penalty: positive scores divided, negative multiplied
    assert plain_impl.sample(logits, 0.0, 0.0, repetition_penalty=2.0, history=[1, 2, 3]) == 4
