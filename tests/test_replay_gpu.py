"""Trace replay through bin/trace_run, as a user runs it, against the plain implementation:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size down to two tokens; and mixed, up to four live requests, portions of some beside decoded
tokens of others, in a pool so small that pages are used again.  In 32-bit and in bfloat16."""

import numpy as np
import pytest

from helpers import TOL, Trace, compare_trace, make_folder, plain_logits, random_ids, run_trace
from tiny_configs import ALL, PAGE_SIZES

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [100, 70, 45, 120, 33, 64], "B": [200, 64, 33, 129, 97, 48], "C": [300, 130, 41, 520, 64, 90],
           "D": [150, 90, 260, 48, 35, 201],
           # E and F run the tensor-core attention kernels in bfloat16: prompts of several 128-query tiles, contexts
           # of more than one 256-key partition, longer than the window
           "E": [700, 420, 300, 530, 160, 280], "F": [600, 330, 290, 450, 130, 200]}
PORTIONS = [7, 2, 16, 3, 2, 33, 5, 2, 64, 9, 2, 17]
LONG_PORTIONS = [130, 2, 257, 16, 3, 128, 40, 2, 64, 9, 2, 300]      # whole query tiles beside ragged ones
FAST = ("E", "F")                                                  # configurations the tensor-core attention takes


def build_trace(requests, rng, portions=PORTIONS, mixed_portion=24):
    trace = Trace()
    names = {}
    # 1. each request alone and whole
    for index, ids in enumerate(requests[:4]):
        name = f"w{index}"
        names[name] = index
        trace.step([(name, ids, range(len(ids)))], end=[name])
    # 2. most of it in one step, the last 32 tokens one by one
    for index, ids in enumerate(requests[:3]):
        name = f"t{index}"
        names[name] = index
        head = len(ids) - 32
        trace.step([(name, ids[:head], [head - 1])])
        for position in range(head, len(ids)):
            trace.step([(name, ids[position:position + 1], [0])], end=[name] if position == len(ids) - 1 else [])
    # 3. portions of changing size, down to two tokens
    for index, ids in enumerate(requests[:3]):
        name = f"p{index}"
        names[name] = index
        cursor, turn = 0, index
        while cursor < len(ids):
            size = min(portions[turn % len(portions)], len(ids) - cursor)
            turn += 1
            last = cursor + size == len(ids)
            trace.step([(name, ids[cursor:cursor + size], range(size))], end=[name] if last else [])
            cursor += size
    # 4. mixed: up to four live; prompts in portions, the last 32 tokens decoded one by one; some requests
    #    sit a step out; finished ones make room for the next, whose pages are the ones just freed
    queue = list(range(len(requests)))
    live = {}
    while queue or live:
        while queue and len(live) < 4:
            index = queue.pop(0)
            name = f"m{index}"
            names[name] = index
            live[name] = 0
        entries, ended = [], []
        for name in list(live):
            ids = requests[names[name]]
            cursor = live[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step, goes on later
            decode_from = max(2, len(ids) - 32)
            if cursor >= decode_from:
                size = 1
            else:
                size = min(int(rng.integers(2, mixed_portion)), decode_from - cursor)
                if decode_from - cursor - size == 1:
                    size += 1
            want = [size - 1] if size > 1 else [0]
            if size > 2 and rng.random() < 0.5:
                want = sorted({0, size // 2, size - 1})
            entries.append((name, ids[cursor:cursor + size], want))
            live[name] = cursor + size
            if live[name] == len(ids):
                ended.append(name)
        if entries:
            trace.step(entries, end=ended)
        for name in ended:
            del live[name]
    return trace, names


def replay_case(tmp_path, name, dtype, graphs):
    import json
    config = ALL[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    folder = make_folder(tmp_path / "model", config, seed=11, dtype=dtype, sharpen=6.0)
    requests = [random_ids(rng, config["vocab_size"], n) for n in LENGTHS[name]]
    fast = name in FAST
    trace, names = build_trace(requests, rng, LONG_PORTIONS if fast else PORTIONS, 150 if fast else 24)
    logits = [plain_logits(folder, ids) for ids in requests]
    reference = {label: logits[index] for label, index in names.items()}
    report_path = tmp_path / "report.json"
    extra = ["--page-size", str(PAGE_SIZES[name]), "--report", str(report_path)] + (["--decode-graphs"] if graphs else [])
    results = run_trace(folder, dtype, trace, tmp_path / "out", extra_args=extra)
    label = f"{name}/{dtype}" + ("/graphs" if graphs else "")
    worst = compare_trace(results, trace, reference, TOL[dtype], label)
    print(f"{label}: {len(trace.lines)} steps, pool for {trace.peak} tokens, worst relative error {worst:.2e}")
    report = json.loads(report_path.read_text())
    for group in report["cache"]["groups"]:
        assert group["free"] == group["pages"], "every page came back"
    assert any(group["reused"] > group["pages"] for group in report["cache"]["groups"]), "pages were used again"
    assert all(flag == 0 for flag in report["errors"].values()), report["errors"]
    if graphs:
        assert report["graphs_captured"] > 0
    return report


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_replay_matches_the_plain_implementation(tmp_path, name, dtype):
    report = replay_case(tmp_path, name, dtype, graphs=False)
    launches = report["launches"]
    if dtype == "bfloat16" and name in FAST:
        # these configurations are here so that the four scripts run the tensor-core attention kernels
        assert launches.get("paged_attention_generic", 0) == 0, launches
        assert launches.get("prefill_attention", 0) > 0, launches
        if name == "E":                                     # head_dim 128: the tcgen05 kernels for prompts and decoding
            assert launches.get("prefill_attention_tc", 0) > 0 and launches.get("decode_attention_tc", 0) > 0, launches
        else:
            assert launches.get("decode_attention", 0) > 0, launches
        assert launches.get("tc_stream", 0) > 0 and launches.get("gemm_bf16_lt", 0) > 0, launches


@pytest.mark.parametrize("name, dtype", [("E", "bfloat16"), ("F", "bfloat16"), ("E", "float32"), ("B", "bfloat16"),
                                         ("C", "float32")])
def test_replay_with_captured_decode_steps(tmp_path, name, dtype):
    """The same four scripts with every step of single tokens run as generation runs it: as a replay of a CUDA
    graph captured for its bucket of rows and table widths."""
    report = replay_case(tmp_path, name, dtype, graphs=True)
    if dtype == "bfloat16" and name in FAST:
        assert report["launches"].get("paged_attention_generic", 0) == 0, report["launches"]


def test_pool_is_small_enough_that_pages_are_used_again(tmp_path):
    """The same mixed trace in-process, reading the cache manager's counters."""
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    import json
    config = ALL["B"]
    rng = np.random.default_rng(5)
    folder = make_folder(tmp_path / "model", config, seed=2, dtype="float32")
    requests = [random_ids(rng, config["vocab_size"], n) for n in LENGTHS["B"]]
    trace, names = build_trace(requests, rng)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=16, block_count=trace.peak // 16),
                                  dtype="float32")).load(folder)
    for line in trace.lines:
        record = json.loads(line)
        for item in record["entries"]:
            if item["id"] not in model.cache.live:
                model.admit(item["id"])
        model.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in record["entries"]])
        for request_id in record["end"]:
            model.release(request_id)
        model.cache.check()
    stats = model.cache_stats()["groups"][0]
    assert stats["reused"] > stats["pages"] and stats["free"] == stats["pages"]
