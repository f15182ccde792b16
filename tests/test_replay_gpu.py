"""Trace replay through bin/trace_run, as a user runs it, against the plain implementation:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size down to two tokens; and mixed, up to four live requests, portions of some beside decoded
tokens of others, in a pool so small that pages are used again.  In 32-bit and in bfloat16."""

import numpy as np
import pytest

from helpers import TOL, Trace, compare_trace, make_folder, plain_logits, random_ids, run_trace
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [100, 70, 45, 120, 33, 64], "B": [200, 64, 33, 129, 97, 48], "C": [300, 130, 41, 520, 64, 90],
           "D": [150, 90, 260, 48, 35, 201]}
PORTIONS = [7, 2, 16, 3, 2, 33, 5, 2, 64, 9, 2, 17]


def build_trace(requests, rng):
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
            size = min(PORTIONS[turn % len(PORTIONS)], len(ids) - cursor)
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
                size = min(int(rng.integers(2, 24)), decode_from - cursor)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_replay_matches_the_plain_implementation(tmp_path, name, dtype):
    config = ALL[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    folder = make_folder(tmp_path / "model", config, seed=11, dtype=dtype, sharpen=6.0)
    requests = [random_ids(rng, config["vocab_size"], n) for n in LENGTHS[name]]
    trace, names = build_trace(requests, rng)
    logits = [plain_logits(folder, ids) for ids in requests]
    reference = {label: logits[index] for label, index in names.items()}
    results = run_trace(folder, dtype, trace, tmp_path / "out")
    worst = compare_trace(results, trace, reference, TOL[dtype], f"{name}/{dtype}")
    print(f"{name}/{dtype}: {len(trace.lines)} steps, pool for {trace.peak} tokens, worst relative error {worst:.2e}")


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
