"""The engine in-process against the plain implementation: the first tokens of a sequence, long
decoding, a page's edge, greedy and sampled generation through the entry point."""

import numpy as np
import pytest
import torch

import plain_impl
from helpers import TOL, make_folder, plain_logits, random_ids
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu


def load(folder, dtype, pages=64, page_size=16, **scheduler):
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, SchedulerConfig
    return Library(RuntimeConfig(kv_cache=CacheConfig(block_size=page_size, block_count=pages),
                                 scheduler=SchedulerConfig(**scheduler), dtype=dtype)).load(folder)


def check(got, want, tol, label):
    error = float(np.abs(got - want).max())
    scale = max(1.0, float(np.abs(want).max()))
    assert np.isfinite(got).all() and error <= tol * scale, f"{label}: max |diff| {error:.3e} > {tol * scale:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence_one_by_one(tmp_path, name, dtype):
    from libmir_b200 import StepEntry
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=3, dtype=dtype, sharpen=6.0)
    ids = random_ids(np.random.default_rng(0), config["vocab_size"], 20)
    reference = plain_logits(folder, ids)
    model = load(folder, dtype, page_size=4)
    model.admit("r")
    for position, token in enumerate(ids):
        result = model.step([StepEntry("r", [token], [0])])
        check(result.logits.cpu().numpy()[0], reference[position], TOL[dtype], f"{name}/{dtype} position {position}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_windows_and_small_pages(tmp_path, dtype):
    """700 tokens decoded one by one after a 60-token prompt on the model with sliding-window layers:
    the window (40) passes many pages (8 tokens each), which go back to the pool and are used again."""
    from libmir_b200 import StepEntry
    folder = make_folder(tmp_path, TINY_C, seed=4, dtype=dtype, sharpen=6.0)
    ids = random_ids(np.random.default_rng(1), TINY_C["vocab_size"], 760)
    reference = plain_logits(folder, ids)
    model = load(folder, dtype, pages=100, page_size=8)
    model.admit("r")
    result = model.step([StepEntry("r", ids[:60], [59])])
    check(result.logits.cpu().numpy()[0], reference[59], TOL[dtype], "prompt")
    for position in range(60, 760):
        result = model.step([StepEntry("r", [ids[position]], [0])])
        if position % 7 == 0 or position > 740:
            check(result.logits.cpu().numpy()[0], reference[position], TOL[dtype], f"{dtype} position {position}")
    full, windowed = model.cache_stats()["groups"]
    assert full["high_water"] == 95 and windowed["high_water"] <= 8
    model.release("r")
    model.admit("again")                                    # the next request runs on pages used before
    result = model.step([StepEntry("again", ids[:100], [99])])
    check(result.logits.cpu().numpy()[0], reference[99], TOL[dtype], "reused pages")
    assert model.cache_stats()["groups"][0]["reused"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_portion_that_ends_and_starts_at_a_pages_edge(tmp_path, dtype):
    from libmir_b200 import StepEntry
    folder = make_folder(tmp_path, TINY_B, seed=6, dtype=dtype, sharpen=6.0)
    ids = random_ids(np.random.default_rng(2), TINY_B["vocab_size"], 50)
    reference = plain_logits(folder, ids)
    model = load(folder, dtype, page_size=8)
    model.admit("r")
    cursor = 0
    for size in (8, 8, 1, 7, 16, 2, 8):                     # edges at 8, 16, 24, 40, 48
        result = model.step([StepEntry("r", ids[cursor:cursor + size], range(size))])
        check(result.logits.cpu().numpy(), reference[cursor:cursor + size], TOL[dtype], f"portion at {cursor}")
        cursor += size


def test_float32_logits_do_not_depend_on_the_cut_or_the_batch_at_all(tmp_path):
    """In 32-bit every reduction's order is fixed by the token's own position, so the same position
    gives bit-identical logits whole, decoded, in portions and beside other requests."""
    from libmir_b200 import StepEntry
    folder = make_folder(tmp_path, TINY_C, seed=8, dtype="float32", sharpen=6.0)
    rng = np.random.default_rng(3)
    ids, other = (random_ids(rng, TINY_C["vocab_size"], n) for n in (90, 70))
    model = load(folder, "float32", page_size=8)
    model.admit("whole")
    whole = model.step([StepEntry("whole", ids, range(90))]).logits.cpu().numpy()
    model.admit("cut"); model.admit("other")
    rows = []
    cursor = 0
    for size in (13, 2, 30, 1, 1, 20, 23):
        entries = [StepEntry("cut", ids[cursor:cursor + size], range(size))]
        if cursor < 60:
            entries.insert(0, StepEntry("other", other[cursor:cursor + 9], [0]))
        result = model.step(entries)
        rows.append(result.logits.cpu().numpy()[-size:])
        cursor += size
    assert np.array_equal(np.concatenate(rows), whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """Prompts of 5/11/17 (A) and 1/9/33/64 (B) tokens, greedy, against the plain
    implementation decoding the same way (whole sequence recomputed for every token)."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=0 if name == "A" else 1, dtype=dtype, sharpen=6.0)
    rng = np.random.default_rng(7)
    lengths = [5, 11, 17] if name == "A" else [1, 9, 33, 64]
    prompts = [random_ids(rng, config["vocab_size"], n) for n in lengths]
    model = load(folder, dtype, page_size=16 if name == "A" else 8, prefill_chunk_tokens=16)
    outputs = model.generate_batch([GenerationRequest(p, GenerationOverrides(max_tokens=8)) for p in prompts])
    plain_config, weights = plain_impl.read_model(folder)
    for prompt, output in zip(prompts, outputs):
        assert output.finish_reason == "length" and len(output.token_ids) == 8
        tokens = list(prompt)
        for step, token in enumerate(output.token_ids):
            logits = plain_impl.forward(plain_config, weights, tokens)[-1].numpy()
            best = plain_impl.greedy(logits)
            if token != best:                                  # allowed only on a near-tie in bfloat16
                margin = logits[best] - logits[token]
                assert dtype == "bfloat16" and margin <= 2 * TOL[dtype] * max(1.0, np.abs(logits).max()), (
                    f"{name}/{dtype}: token {step} is {token}, plain says {best} (margin {margin:.3e})")
            tokens.append(token)
    assert model.cache_stats()["groups"][0]["free"] == 64


def test_sampled_generation_follows_the_plain_sampler(tmp_path):
    """Temperature 0.7, top-k/top-p and a repetition penalty: with the same seed the engine must pick the
    token the plain sampler picks from the plain logits, draw by draw (32-bit)."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    folder = make_folder(tmp_path, TINY_B, seed=1, dtype="float32", sharpen=6.0)
    rng = np.random.default_rng(9)
    prompts = [random_ids(rng, TINY_B["vocab_size"], n) for n in (1, 9, 33, 64)]
    options = [GenerationOverrides(max_tokens=12, temperature=0.7),
               GenerationOverrides(max_tokens=12, temperature=0.7, top_k=5),
               GenerationOverrides(max_tokens=12, temperature=1.3, top_p=0.8),
               GenerationOverrides(max_tokens=12, temperature=0.9, top_k=40, top_p=0.9, repetition_penalty=1.3)]
    model = load(folder, "float32", page_size=8, prefill_chunk_tokens=16)
    outputs = model.generate_batch([GenerationRequest(p, o, seed=100 + i)
                                    for i, (p, o) in enumerate(zip(prompts, options))])
    plain_config, weights = plain_impl.read_model(folder)
    for index, (prompt, option, output) in enumerate(zip(prompts, options, outputs)):
        generator = plain_impl.SplitMix64(100 + index)
        tokens = list(prompt)
        for step, token in enumerate(output.token_ids):
            logits = plain_impl.forward(plain_config, weights, tokens)[-1].numpy()
            expected = plain_impl.sample(logits, generator.next_unit(), option.temperature, option.top_k or 0,
                                         option.top_p or 1.0, option.repetition_penalty or 1.0, tokens)
            assert token == expected, f"request {index} token {step}: engine {token}, plain sampler {expected}"
            tokens.append(token)


def follow_plain_sampler(folder, prompts, options, seeds, outputs, dtype="float32"):
    """Every generated token against the plain sampler on the plain logits, draw by draw."""
    plain_config, weights = plain_impl.read_model(folder)
    for index, (prompt, option, seed, output) in enumerate(zip(prompts, options, seeds, outputs)):
        generator = plain_impl.SplitMix64(seed)
        tokens = list(prompt)
        assert len(output.token_ids) == option.max_tokens
        for step, token in enumerate(output.token_ids):
            logits = plain_impl.forward(plain_config, weights, tokens)[-1].numpy()
            greedy = (option.temperature or 0.0) <= 1e-7 or option.top_k == 1
            draw = 0.0 if greedy else generator.next_unit()
            expected = plain_impl.sample(logits, draw, option.temperature or 0.0, option.top_k or 0,
                                         option.top_p or 1.0, option.repetition_penalty or 1.0, tokens)
            if token != expected and dtype == "bfloat16" and greedy:      # allowed only on a near-tie in bfloat16
                margin = logits[expected] - logits[token]
                assert margin <= 2 * TOL[dtype] * max(1.0, np.abs(logits).max()), (
                    f"request {index} token {step}: {token}, plain says {expected} (margin {margin:.3e})")
            else:
                assert token == expected, f"request {index} token {step}: engine {token}, plain sampler {expected}"
            tokens.append(token)


def test_sampled_generation_on_captured_decode_steps_follows_the_plain_sampler(tmp_path):
    """No request has a repetition penalty, so every decode-only step replays a captured graph, whose sampling
    options (draw, temperature, top-p, top-k per row) the host writes into the graph's own block.  The requests
    produce different numbers of tokens, so rows of the captured batch pass from one request to another while
    others go on.  Every token must be the one the plain sampler picks with the same seed, draw by draw."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    folder = make_folder(tmp_path, TINY_B, seed=1, dtype="float32", sharpen=6.0)
    rng = np.random.default_rng(19)
    prompts = [random_ids(rng, TINY_B["vocab_size"], n) for n in (3, 9, 33, 20, 6)]
    options = [GenerationOverrides(max_tokens=20, temperature=0.7),
               GenerationOverrides(max_tokens=7, temperature=0.8, top_k=5),
               GenerationOverrides(max_tokens=13, temperature=1.3, top_p=0.8),
               GenerationOverrides(max_tokens=16, temperature=0.0),
               GenerationOverrides(max_tokens=18, temperature=0.9, top_k=30, top_p=0.9)]
    seeds = [200 + i for i in range(len(prompts))]
    model = load(folder, "float32", page_size=8, prefill_chunk_tokens=16, max_batch_requests=4)
    outputs = model.generate_batch([GenerationRequest(p, o, seed=s) for p, o, s in zip(prompts, options, seeds)])
    graphs = model.runner._graphs
    assert graphs is not None and sum(g.replays for g in graphs.graphs.values()) >= 15
    assert any(g.ranked for g in graphs.graphs.values()) and len({g.rows for g in graphs.graphs.values()}) >= 2
    assert model.runner.steps_again >= 5         # steps that only wrote tokens, positions and draws (_step_again)
    follow_plain_sampler(folder, prompts, options, seeds, outputs)


def test_greedy_generation_in_bfloat16_on_the_tensor_core_kernels(tmp_path):
    """Configuration E (head_dim 128) through the entry point: prompts in portions of 128 tokens, then captured
    decode steps; greedy tokens against the plain implementation, a differing token only at a near-tie."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    from tiny_configs import TINY_E
    folder = make_folder(tmp_path, TINY_E, seed=3, dtype="bfloat16", sharpen=6.0)
    rng = np.random.default_rng(23)
    prompts = [random_ids(rng, TINY_E["vocab_size"], n) for n in (300, 5, 150)]
    options = [GenerationOverrides(max_tokens=n, temperature=0.0) for n in (10, 6, 8)]
    model = load(folder, "bfloat16", prefill_chunk_tokens=128)
    outputs = model.generate_batch([GenerationRequest(p, o) for p, o in zip(prompts, options)])
    graphs = model.runner._graphs
    assert graphs is not None and sum(g.replays for g in graphs.graphs.values()) >= 5
    follow_plain_sampler(folder, prompts, options, [0, 0, 0], outputs, dtype="bfloat16")


def test_session_prefill_and_decode(tmp_path):
    from libmir_b200 import SamplingLogits
    folder = make_folder(tmp_path, TINY_A, seed=2, dtype="float32")
    ids = random_ids(np.random.default_rng(4), 256, 12)
    reference = plain_logits(folder, ids)
    model = load(folder, "float32")
    with model.session() as session:
        out = session.prefill(ids[:8], SamplingLogits.FULL)
        check(out.logits, reference[7], TOL["float32"], "session prefill")
        assert out.cached_tokens == 8
        out = session.decode(ids[8], SamplingLogits.TOKEN)
        assert out.next_token == plain_impl.greedy(reference[8]) and session.cache_stats()["cached_tokens"] == 9
    assert model.cache_stats()["live_requests"] == 0
    model.unload()


def test_decode_profiling_attaches_timings_to_decode_steps_only(tmp_path):
    """Model.set_profile_decode, as libmir's: while it is on, steps of one token per request carry how long they took
    on the host and on the device and how many rows they had; portions of prompts and steps after it was switched off
    carry nothing, and the tokens are what they are without it."""
    from libmir_b200 import GenerationOverrides, GenerationRequest, StepEntry
    from libmir_b200.sampling import RequestSampler
    folder = make_folder(tmp_path, TINY_B, seed=5, dtype="bfloat16")
    rng = np.random.default_rng(9)
    prompts = [random_ids(rng, TINY_B["vocab_size"], n) for n in (12, 7)]
    model = load(folder, "bfloat16")
    request = [GenerationRequest(prompt_ids=p, options=GenerationOverrides(max_tokens=6, ignore_eos=True)) for p in prompts]
    plain = [o.token_ids for o in model.generate_batch(request)]
    model.set_profile_decode(True)
    outputs = model.generate_batch(request)
    assert [o.token_ids for o in outputs] == plain
    metrics = outputs[0].metrics
    assert metrics["decode_steps_profiled"] == 5                  # six tokens: one from the prompts' step, five decoded
    assert 0.0 < metrics["decode_device_seconds"] < 1.0 and 0.0 < metrics["decode_backend_seconds"] < 5.0
    for name in ("a", "b"):
        model.admit(name)
    first = model.step([StepEntry("a", prompts[0], [len(prompts[0]) - 1]), StepEntry("b", prompts[1], [6])],
                       [RequestSampler(), RequestSampler()])
    assert first.timings is None                                  # a step of prompt portions
    tokens = first.tokens.cpu().tolist()
    second = model.step([StepEntry("a", [tokens[0]], [0]), StepEntry("b", [tokens[1]], [0])],
                        [RequestSampler(), RequestSampler()])
    assert second.timings is not None and second.timings.batch_rows == 2
    assert second.timings.device_execution > 0.0 and second.timings.backend_execution > 0.0
    assert set(second.timings.as_dict()) == {"backend_execution", "device_execution", "batch_rows"}
    model.set_profile_decode(False)
    tokens = second.tokens.cpu().tolist()
    third = model.step([StepEntry("a", [tokens[0]], [0]), StepEntry("b", [tokens[1]], [0])],
                       [RequestSampler(), RequestSampler()])
    assert third.timings is None
    for name in ("a", "b"):
        model.release(name)
    assert "decode_steps_profiled" not in model.generate_batch(request)[0].metrics
    model.unload()


def test_generate_command_line(tmp_path):
    """bin/generate as a user runs it: a folder written by --write-random-model, then greedy tokens that match
    the plain implementation, the `finish_reason=` line, and the batch form."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    config_path = tmp_path / "tiny.json"
    config_path.write_text(json.dumps(TINY_A))
    folder = tmp_path / "model"
    run = lambda *args: subprocess.run([sys.executable, str(ROOT / "bin" / "generate"), *args], capture_output=True,
                                       text=True, timeout=300)
    done = run("--random-weights", str(config_path), "--write-random-model", str(folder), "--dtype", "float32",
               "--weights-seed", "5")
    assert done.returncode == 0 and (folder / "model.safetensors").is_file(), done.stderr[-2000:]
    done = run(str(folder), "--prompt-ids", "5,17,3,200,9", "--max-tokens", "6", "--dtype", "float32",
               "--block-count", "32")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = done.stdout.strip().splitlines()
    assert lines[-1] == "finish_reason=length"
    tokens = [int(t) for t in lines[0].split()]
    plain_config, weights = plain_impl.read_model(folder)
    sequence = [5, 17, 3, 200, 9]
    for token in tokens:
        assert token == plain_impl.greedy(plain_impl.forward(plain_config, weights, sequence)[-1].numpy())
        sequence.append(token)
    assert len(tokens) == 6
    done = run(str(folder), "--prompt-ids", "5,17,3;9,9", "--max-tokens", "3", "--dtype", "float32", "--temperature",
               "0.8", "--seed", "7", "--block-count", "32")
    assert done.returncode == 0, done.stderr[-2000:]
    records = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert [r["request"] for r in records] == [0, 1] and all(len(r["token_ids"]) == 3 for r in records)
    for record, prompt in zip(records, ([5, 17, 3], [9, 9])):               # every request draws from seed 7
        generator = plain_impl.SplitMix64(7)
        sequence = list(prompt)
        for token in record["token_ids"]:
            logits = plain_impl.forward(plain_config, weights, sequence)[-1].numpy()
            assert token == plain_impl.sample(logits, generator.next_unit(), 0.8)
            sequence.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_tokens_between_portions_keep_the_order_of_what_is_wanted(tmp_path, dtype):
    """The step packs single-token rows first (they run as decoded tokens, the portions as tiles of queries);
    the logits still come in the order of the entries and of their wanted places."""
    from libmir_b200 import StepEntry
    folder = make_folder(tmp_path, TINY_B, seed=21, dtype=dtype)
    rng = np.random.default_rng(21)
    vocab = TINY_B["vocab_size"]
    prompts = {name: random_ids(rng, vocab, n) for name, n in (("a", 70), ("b", 41), ("c", 55), ("d", 33))}
    want = {name: plain_logits(folder, ids) for name, ids in prompts.items()}
    model = load(folder, dtype, page_size=8, pages=64)
    for name in prompts:
        model.admit(name)
    # b and d are 40 and 32 tokens in already, so that their next token is a single decoded one
    model.step([StepEntry("b", prompts["b"][:40], []), StepEntry("d", prompts["d"][:32], [])])
    result = model.step([StepEntry("a", prompts["a"][:37], [36, 0, 5]), StepEntry("b", prompts["b"][40:41], [0]),
                         StepEntry("c", prompts["c"][:2], [1]), StepEntry("d", prompts["d"][32:33], [0])])
    assert result.rows == [("a", 36), ("a", 0), ("a", 5), ("b", 0), ("c", 1), ("d", 0)]
    got = result.logits.cpu().numpy()
    expected = np.stack([want["a"][36], want["a"][0], want["a"][5], want["b"][40], want["c"][1], want["d"][32]])
    check(got, expected, TOL[dtype], "mixed step")
    # and the cache is right afterwards: everyone's next tokens
    result = model.step([StepEntry("c", prompts["c"][2:55], [52]), StepEntry("a", prompts["a"][37:70], [32])])
    assert result.rows == [("c", 52), ("a", 32)]
    check(result.logits.cpu().numpy(), np.stack([want["c"][54], want["a"][69]]), TOL[dtype], "after the mixed step")


def test_a_folder_with_fused_and_transposed_tensors_gives_the_same_logits(tmp_path):
    """The same weights stored as libmir also accepts them: query, key and value as one `qkv_proj` tensor, the
    down projection as [in, out], an auxiliary buffer nobody asks for.  32-bit logits must be the same bits."""
    from libmir_b200 import StepEntry
    from libmir_b200.weights import load_tensor, read_catalog, write_file
    plain_folder = make_folder(tmp_path / "plain", TINY_C, seed=12, dtype="float32", sharpen=6.0)
    other = make_folder(tmp_path / "fused", TINY_C, seed=12, dtype="float32", sharpen=6.0)
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(other).items()}
    for layer in range(TINY_C["num_hidden_layers"]):
        stem = f"model.layers.{layer}."
        for kind in ("weight", "bias"):
            tensors[f"{stem}self_attn.qkv_proj.{kind}"] = torch.cat(
                [tensors.pop(f"{stem}self_attn.{p}_proj.{kind}") for p in "qkv"], dim=0)
        tensors[f"{stem}mlp.down_proj.weight"] = tensors[f"{stem}mlp.down_proj.weight"].t().contiguous()
        tensors[f"{stem}self_attn.rotary_emb.inv_freq"] = torch.zeros(12)
    write_file(other / "model.safetensors", tensors)
    ids = random_ids(np.random.default_rng(12), TINY_C["vocab_size"], 75)
    logits = []
    for folder in (plain_folder, other):
        model = load(folder, "float32", page_size=8)
        model.admit("r")
        logits.append(model.step([StepEntry("r", ids, range(len(ids)))]).logits.cpu().numpy())
        model.unload()
    assert np.array_equal(logits[0], logits[1])
    check(logits[0], plain_logits(plain_folder, ids), TOL["float32"], "against the plain implementation")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E", "F"])
def test_native_executor_and_python_parts_launch_the_same_work(tmp_path, name, dtype, monkeypatch):
    """The layer executor issues the launches that the parts issue when they run one by one from Python: the same
    kernels on the same data in the same order, so the logits must be the same bits, for whole prompts, portions,
    mixed steps and decoded tokens (folded norms included)."""
    from libmir_b200 import StepEntry, kernels
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=31, dtype=dtype, sharpen=4.0)
    rng = np.random.default_rng(31)
    first, second = random_ids(rng, config["vocab_size"], 330), random_ids(rng, config["vocab_size"], 200)
    results = []
    for native in (True, False):
        monkeypatch.setattr(kernels, "NATIVE_LAYERS", native)
        counts_before = kernels.launch_counts()
        model = load(folder, dtype, page_size=8, pages=128)
        model.admit("a"); model.admit("b")
        logits = [model.step([StepEntry("a", first[:150], [0, 149])]).logits.clone()]
        logits.append(model.step([StepEntry("a", first[150:151], [0]), StepEntry("b", second[:140], [139])]).logits.clone())
        logits.append(model.step([StepEntry("b", second[140:160], [19]), StepEntry("a", first[151:152], [0])]).logits.clone())
        for offset in range(3):
            logits.append(model.step([StepEntry("a", [first[152 + offset]], [0]),
                                      StepEntry("b", [second[160 + offset]], [0])]).logits.clone())
        logits.append(model.step([StepEntry("a", first[155:330], [174])]).logits.clone())
        results.append(torch.cat(logits).cpu())
        assert any(isinstance(run.layers, list) for run in model.decoder._runs_list) == native
        model.unload()
    assert torch.equal(results[0], results[1])
    reference = plain_logits(folder, first)
    check(results[0][-1].numpy(), reference[329], TOL[dtype], "against the plain implementation")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_greedy_decode_steps_take_the_short_path_and_stay_right(tmp_path, dtype):
    """Captured greedy decode steps of the same requests skip what cannot have changed (StepRunner._step_again) until
    one of them needs a page, another request joins, one leaves, or a sampler draws: the logits of every step, short
    path or not, are the plain implementation's."""
    from libmir_b200 import StepEntry
    from libmir_b200.sampling import RequestSampler
    config = TINY_A
    folder = make_folder(tmp_path, config, seed=6, dtype=dtype, sharpen=6.0)
    rng = np.random.default_rng(21)
    model = load(folder, dtype, pages=32, page_size=4)
    runner = model.runner
    sequences = {name: random_ids(rng, config["vocab_size"], n) for name, n in (("a", 5), ("b", 11))}
    samplers = {name: RequestSampler() for name in ("a", "b", "c")}
    for name, ids in sequences.items():
        model.admit(name)
        model.step([StepEntry(name, ids, [])])

    last = {"names": None}

    def decode(names):
        """One greedy decode step; the short path must be taken exactly when the step before was a captured greedy
        decode step of the same requests in the same order and every one of them has room in its last page."""
        cached = {name: len(sequences[name]) for name in names}
        expect_short = last["names"] == names and all(cached[name] % 4 != 0 for name in names)
        before = runner.steps_again
        for name in names:
            sequences[name].append(int(rng.integers(config["vocab_size"])))
        result = model.step([StepEntry(name, [sequences[name][-1]], [0]) for name in names], [samplers[n] for n in names])
        assert (runner.steps_again - before == 1) == expect_short, (names, cached, last)
        last["names"] = list(names)
        got = result.logits.float().cpu().numpy()
        for row, name in enumerate(names):
            check(got[row], plain_logits(folder, sequences[name])[-1], TOL[dtype], f"{name} at {len(sequences[name]) - 1}")
        assert result.tokens.cpu().tolist() == [int(np.argmax(got[row])) for row in range(len(names))]
        return expect_short

    taken = [decode(["a", "b"]) for _ in range(7)]             # pages of 4: a and b reach page edges at different steps
    assert taken.count(True) >= 3 and taken.count(False) >= 3, taken
    taken = [decode(["b", "a"]) for _ in range(4)]             # another order is another batch
    assert taken[0] is False and True in taken
    sequences["c"] = random_ids(rng, config["vocab_size"], 6)
    model.admit("c")
    model.step([StepEntry("c", sequences["c"], [])])          # a prompt in between
    last["names"] = None
    assert decode(["b", "a"]) is False
    assert decode(["b", "a", "c"]) is False
    taken = [decode(["b", "a", "c"]) for _ in range(5)]
    assert True in taken
    model.release("a")
    model.admit("a")                                           # the same name, another request
    sequences["a"] = random_ids(rng, config["vocab_size"], 3)
    model.step([StepEntry("a", sequences["a"], [])])
    last["names"] = None
    assert decode(["b", "a", "c"]) is False
    decode(["b", "a", "c"])
    samplers["c"] = RequestSampler(temperature=0.7, seed=3)    # a sampler that draws ends it, too
    before = runner.steps_again
    for name in ("b", "a", "c"):
        sequences[name].append(int(rng.integers(config["vocab_size"])))
    model.step([StepEntry(n, [sequences[n][-1]], [0]) for n in ("b", "a", "c")], [samplers[n] for n in ("b", "a", "c")])
    assert runner.steps_again == before
    with pytest.raises(Exception, match="token id outside"):
        model.step([StepEntry("b", [config["vocab_size"]], [0])], [samplers["b"]])
    model.cache.check()
    model.unload()
