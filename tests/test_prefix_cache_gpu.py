"""The prefix cache on the device: a request that takes over another's pages gets the logits the plain
implementation gives for its whole sequence; shared pages are not written again; evicted pages are computed
again; generation gives the same tokens with and without it."""

import numpy as np
import pytest
import torch

import plain_impl
from helpers import TOL, make_folder, plain_logits, random_ids
from tiny_configs import TINY_A, TINY_B, TINY_E

pytestmark = pytest.mark.gpu

# head_dim 128 without a window: in bfloat16 the tcgen05 prompt and decode kernels read the shared pages
TINY_E_FULL = {key: value for key, value in TINY_E.items() if key not in ("layer_types", "sliding_window")}
CONFIGS = {"A": TINY_A, "B": TINY_B, "E": TINY_E_FULL}


def load(folder, dtype, pages, page_size, prefix_cache=True, **scheduler):
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, SchedulerConfig
    cache = CacheConfig(block_size=page_size, block_count=pages, prefix_cache=prefix_cache)
    return Library(RuntimeConfig(kv_cache=cache, scheduler=SchedulerConfig(**scheduler), dtype=dtype)).load(folder)


def check(got, want, tol, label):
    error = float(np.abs(got - want).max())
    scale = max(1.0, float(np.abs(want).max()))
    assert np.isfinite(got).all() and error <= tol * scale, f"{label}: max |diff| {error:.3e} > {tol * scale:.3e}"


def feed(model, name, ids, portion, reference, tol, label):
    """Admit `name` with all its tokens, feed what is not cached in portions, compare every logit it computes;
    returns how many tokens were found cached."""
    from libmir_b200 import StepEntry
    cached = model.admit(name, ids)
    position = cached
    while position < len(ids):
        tokens = ids[position:position + portion]
        result = model.step([StepEntry(name, tokens, list(range(len(tokens))))])
        check(result.logits.float().cpu().numpy(), reference[position:position + len(tokens)], tol,
              f"{label} positions {position}..{position + len(tokens) - 1} ({cached} cached)")
        position += len(tokens)
    return cached


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_requests_that_start_alike_share_pages_and_get_the_plain_logits(tmp_path, name, dtype):
    from libmir_b200 import StepEntry
    config, page = CONFIGS[name], 8
    folder = make_folder(tmp_path, config, seed=5, dtype=dtype, sharpen=6.0)
    rng = np.random.default_rng(11)
    first = random_ids(rng, config["vocab_size"], 53)
    second = first[:37] + random_ids(rng, config["vocab_size"], 20)          # shares four full pages and five tokens
    third = first[:16] + random_ids(rng, config["vocab_size"], 9)            # shares two pages exactly
    other = random_ids(rng, config["vocab_size"], 70)
    tol = TOL[dtype]
    model = load(folder, dtype, pages=16, page_size=page)
    pool = model.cache.groups[0].pool

    assert feed(model, "first", first, 19, plain_logits(folder, first), tol, "first") == 0
    assert len(model.cache.prefix) == 6
    # while the first is live: the second takes four of its pages, the third two; all three decode side by side
    assert feed(model, "second", second, 7, plain_logits(folder, second), tol, "second") == 32
    assert feed(model, "third", third, 64, plain_logits(folder, third), tol, "third") == 16
    shared = model.cache.live["first"].tables[0][:4]
    assert model.cache.live["second"].tables[0][:4] == shared and model.cache.live["third"].tables[0][:2] == shared[:2]
    assert [pool.holders(p) for p in shared] == [4, 4, 3, 3]
    sequences = {"first": list(first), "second": list(second), "third": list(third)}
    for _ in range(6):
        for ids in sequences.values():
            ids.append(int(rng.integers(config["vocab_size"])))
        result = model.step([StepEntry(n, [ids[-1]], [0]) for n, ids in sequences.items()])
        got = result.logits.float().cpu().numpy()
        for row, (n, ids) in enumerate(sequences.items()):
            check(got[row], plain_logits(folder, ids)[-1], tol, f"{n} decoding at {len(ids) - 1}")
    model.cache.check()
    for n in sequences:
        model.release(n)
    # a request that needs most of the pool pushes the oldest cached pages out; what is left is still right
    evictions = model.cache.prefix_evictions
    assert feed(model, "other", other, 33, plain_logits(folder, other), tol, "other") == 0
    assert model.cache.prefix_evictions > evictions
    model.release("other")
    again = first[:50]
    cached = feed(model, "again", again, 64, plain_logits(folder, again), tol, "first again")
    assert cached % page == 0 and cached <= 48
    model.release("again")
    assert feed(model, "other again", other, 64, plain_logits(folder, other), tol, "other again") == 64
    model.release("other again")
    model.cache.check()
    assert pool.available == 16 and pool.reused > 0
    model.unload()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_gives_the_same_tokens_with_and_without_the_prefix_cache(tmp_path, dtype):
    from libmir_b200 import GenerationOverrides, GenerationRequest
    config = TINY_E_FULL
    folder = make_folder(tmp_path, config, seed=9, dtype=dtype, sharpen=6.0)
    rng = np.random.default_rng(3)
    system = random_ids(rng, config["vocab_size"], 70)
    prompts = [system + random_ids(rng, config["vocab_size"], n) for n in (5, 23, 1, 40)]
    requests = [GenerationRequest(p, GenerationOverrides(max_tokens=12)) for p in prompts]
    plain = load(folder, dtype, pages=64, page_size=16, prefix_cache=False, prefill_chunk_tokens=48)
    want = [output.token_ids for output in plain.generate_batch(requests)]
    plain.unload()
    model = load(folder, dtype, pages=64, page_size=16, prefill_chunk_tokens=48)
    one = model.generate_batch(requests[:1])
    assert one[0].metrics["cached_prompt_tokens"] == 0
    rest = model.generate_batch(requests)                          # the system prompt's four pages are there already
    assert [output.metrics["cached_prompt_tokens"] for output in rest] == [64, 64, 64, 64]
    got = [output.token_ids for output in rest]
    if dtype == "float32":                                         # (in bfloat16 another cut may flip a near-tie)
        assert got == want and one[0].token_ids == got[0]
    plain_config, weights = plain_impl.read_model(folder)
    for prompt, output in zip(prompts, got):                       # and what the plain implementation decodes
        tokens = list(prompt)
        for step, token in enumerate(output):
            logits = plain_impl.forward(plain_config, weights, tokens)[-1].numpy()
            best = plain_impl.greedy(logits)
            if token != best:                                      # allowed only on a near-tie in bfloat16
                margin = logits[best] - logits[token]
                assert dtype == "bfloat16" and margin <= 2 * TOL[dtype] * max(1.0, np.abs(logits).max()), (
                    f"{dtype}: token {step} is {token}, plain says {best} (margin {margin:.3e})")
            tokens.append(token)
    stats = model.cache_stats()
    assert stats["groups"][0]["free"] == 64 and stats["cached_prefix_pages"] > 0 and stats["live_requests"] == 0
    model.cache.check()
    model.unload()


def test_a_session_takes_over_cached_pages_at_its_first_prefill(tmp_path):
    from libmir_b200 import SamplingLogits
    folder = make_folder(tmp_path, TINY_A, seed=4, dtype="float32", sharpen=6.0)
    ids = random_ids(np.random.default_rng(8), TINY_A["vocab_size"], 45)
    reference = plain_logits(folder, ids)
    model = load(folder, "float32", pages=16, page_size=8)
    with model.session() as session:
        out = session.prefill(ids[:40], SamplingLogits.FULL)
        assert out.reused_tokens == 0 and out.cached_tokens == 40
        check(out.logits, reference[39], TOL["float32"], "first session")
    with model.session() as session:                         # five full pages of the same tokens are there
        out = session.prefill(ids[:44], SamplingLogits.FULL)
        assert out.reused_tokens == 40 and out.cached_tokens == 44
        check(out.logits, reference[43], TOL["float32"], "second session, 40 tokens taken over")
        out = session.decode(ids[44], SamplingLogits.FULL)
        assert out.reused_tokens == 0 and out.cached_tokens == 45
        check(out.logits, reference[44], TOL["float32"], "second session decoding")
    assert model.clear_prefix_cache() == 5 and model.cache_stats()["cached_prefix_pages"] == 0
    with model.session() as session:
        assert session.prefill(ids[:44], SamplingLogits.FULL).reused_tokens == 0
    model.cache.check()
    model.unload()
