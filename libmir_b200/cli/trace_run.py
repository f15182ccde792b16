"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
All entries of a step run as one batch through the engine's own step function, cache and kernels (the
ones generation uses); nothing is sampled.  For a step in which something is wanted the logits at the
wanted places are written to OUT/<step>.f32 as little-endian float32 [wanted, vocab], in the order of
the entries and of `want`.  After every step a line `done <step>` is printed and flushed.  Requests
named in `end` give back what they hold after the step.  The cache pool holds --max-tokens tokens
(rounded up to whole pages), so pages are used again.

Two more options, for tests: --decode-graphs runs every step in which each request brings one token and wants
its logits the way generation runs such steps, as a replay of a captured CUDA graph (the logits written are the
ones the graph computed; the greedy token it also samples is dropped); --report FILE writes, when the input
ends, a JSON object with the number of launches of each kernel, the error flags of the kernels with bounded
waits, and the cache manager's counters.

Modelled on libmir's examples/teacher-forcing.rs:68-109 and examples/batch-parity.rs:114-165, which
can only see last-position logits through Session::prefill/decode.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-requests", type=int, default=8)
    parser.add_argument("--decode-graphs", action="store_true",
                        help="run steps of single tokens as replays of captured CUDA graphs, as generation does")
    parser.add_argument("--report", help="write launch counts, kernel error flags and cache counters to this file")
    args = parser.parse_args(argv)

    from ..config.runtime import CacheConfig, CudaConfig, RuntimeConfig, SchedulerConfig
    from ..engine.api import Library
    from ..engine.step import StepEntry
    from ..sampling.sampler import RequestSampler

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    page = args.page_size
    # the caller rounds each request's count up to a multiple of 64; pages of 16 tokens divide that
    unit = max(page, 64) if 64 % page == 0 or page % 64 == 0 else page * 64
    pages = -(-(-(-args.max_tokens // unit) * unit) // page)
    runtime = RuntimeConfig(
        kv_cache=CacheConfig(block_size=page, block_count=pages),
        scheduler=SchedulerConfig(max_batch_requests=args.max_requests),
        cuda=CudaConfig(decode_graphs=args.decode_graphs),
        dtype=args.dtype)
    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = Library(runtime).load(args.model, progress=lambda m: print(f"[trace_run] {m}", file=sys.stderr, flush=True))
    print(f"[trace_run] ready: {pages} pages of {page} tokens per cache group", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = item["id"]
            if request_id not in model.cache.live:
                model.admit(request_id)
            entries.append(StepEntry(request_id, item["tokens"], item.get("want", [])))
        samplers = None
        if args.decode_graphs and entries and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            samplers = [RequestSampler() for _ in entries]       # greedy: what makes a step eligible for a graph
        result = model.step(entries, samplers)
        if result.logits is not None and result.logits.shape[0] > 0:
            values = result.logits.float().cpu().numpy().astype("<f4", copy=False)
            values.tofile(out / f"{step}.f32")
        for request_id in record.get("end", []):
            if request_id in model.cache.live:
                model.release(request_id)
        print(f"done {step}", flush=True)
    if args.report:
        from .. import kernels
        import torch
        torch.cuda.synchronize()
        graphs = model.runner._graphs
        report = {"launches": kernels.launch_counts(), "cache": model.cache_stats(),
                  "graphs_captured": len(graphs.graphs) if graphs is not None else 0,
                  "errors": {"stream_linear": kernels.stream_linear_error(),
                             "tensor_core_linear": kernels.tensor_core_linear_error(),
                             "prefill_attention": kernels.prefill_attention_error(),
                             "decode_attention": kernels.decode_attention_error()}
                  if args.dtype == "bfloat16" else {}}
        Path(args.report).write_text(json.dumps(report, indent=1, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
