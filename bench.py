#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-4B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with 2,048 tokens of context
per request, timed on the device over exactly K decode steps that run back to back (each step's
sampled token is the next step's input on the device).  `e2e` is the same through the Python entry
point with host token ids in and out every step.  `prefill` is one 2,048-token prompt in one step.
`points` has decode at batch 1 and 64 and the time of a mixed step (32 decoded tokens beside a 512-token portion).  Weights are random (N(0, 0.02), seeded), token ids are seeded
uniform random, and the cache of the decode runs is filled with random keys and values of the stated
context length (a decode step's cost does not depend on the values).

The engine runs on one GPU: for --gpus N > 1 a line says so and the exit code is 2.
The reference (mirmir-tech/libmir) is a Rust workspace with crates.io-only dependencies; it cannot be
installed offline with pip, so `--impl reference` prints an `unavailable` line and exits 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "hidden_size": 2560, "intermediate_size": 9728, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936,
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "hidden_act": "silu",
}
LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "hidden_act": "silu",
}
QWEN3_32B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64,
    "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936,
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "hidden_act": "silu",
}
SIZES = {"qwen3-4b": ("Qwen3-4B sizes (BASELINE.json configs[2])", QWEN3_4B),
         "llama-3.1-8b": ("Llama-3.1-8B sizes (BASELINE.json configs[3])", LLAMA31_8B),
         "qwen3-32b": ("Qwen3-32B sizes (BASELINE.json configs[4])", QWEN3_32B)}
PROMPT_TOKENS = 2048
GENERATED_TOKENS = 256
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            data = json.load(open(path))
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key in FALLBACK_PEAKS:
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {**FALLBACK_PEAKS, **flat}, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.samples = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self):
        clocks, reasons, maximum = [], set(), None
        for sm, sm_max, hw, hw_thermal, sw_thermal, power in self.samples:
            try:
                clocks.append(float(sm))
                maximum = float(sm_max)
            except ValueError:
                continue
            for name, value in (("hw_slowdown", hw), ("hw_thermal_slowdown", hw_thermal),
                                ("sw_thermal_slowdown", sw_thermal), ("sw_power_cap", power)):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": maximum,
                "reasons": sorted(reasons), "samples": len(clocks)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--sizes", default="qwen3-4b", choices=sorted(SIZES),
                        help="layer sizes of the model (default: the headline configuration)")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--repeats", type=int, default=5,
                        help="how often the timed region of K steps is run; the median region is reported")
    parser.add_argument("--context", type=int, default=PROMPT_TOKENS,
                        help="tokens every request holds when decoding starts, and the length of the timed prompt "
                             "(default: the headline configuration's 2,048; up to 8,192 in one prefill step)")
    parser.add_argument("--skip-points", action="store_true", help="only the batch-8 decode and the prefill")
    parser.add_argument("--deep-ring-ctas", type=int, default=None,
                        help="up to how many CTAs decode attention keeps three tiles in flight per warp")
    parser.add_argument("--set", action="append", default=[], metavar="NAME=VALUE",
                        help="set a tuning constant of libmir_b200.kernels or an option of the native product dispatch (an "
                             "integer), e.g. PREFILL_TENSOR_CORES=0, few_rows_max=16 or decode_tensor_cores=0")
    parser.add_argument("--stream-shape", default=None, metavar="SPLITS,RING_KB,TILE_ROWS",
                        help="fix the shape of the weight-streaming product (0 = chosen by the launcher), e.g. 0,56,0")
    parser.add_argument("--no-fold-norm", action="store_true",
                        help="run every RMSNorm as a kernel of its own instead of folding it into the few-rows "
                             "products around it")
    parser.add_argument("--phase", default="all", choices=["all", "decode", "prefill", "serve", "kernels", "trace"],
                        help="decode / prefill: run only that phase, bracketed by cudaProfilerStart/Stop (for ncu "
                             "--profile-from-start off); the JSON line then holds only that phase")
    parser.add_argument("--no-graphs", action="store_true", help="decode steps as plain launches, not as CUDA graphs")
    parser.add_argument("--library-modes", default="", help="few-rows epilogues (store,accum,f32,swiglu) to run "
                        "through the library product instead (an experiment switch)")
    parser.add_argument("--pdl", type=int, default=None, choices=[0, 1, 2],
                        help="launch kernels with (1) or without (0) programmatic stream serialization")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "mirmir-tech/libmir is a Rust workspace (no setup.py/pyproject; cargo, rustc and its "
                          "crates.io dependencies mircuda/mirtal/mircup are absent offline): pip cannot install it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch

    from libmir_b200 import CacheConfig, CudaConfig, Library, RuntimeConfig, SchedulerConfig, StepEntry, kernels
    from libmir_b200.sampling import RequestSampler

    if args.phase == "trace":
        kernels.use_traced_kernels()                          # before anything loads the plain bfloat16 library
    if args.library_modes:
        modes = kernels.get_option("few_rows_modes")
        for name in args.library_modes.split(","):
            modes &= ~(1 << ["store", "accum", "f32", "swiglu"].index(name))
        kernels.set_option("few_rows_modes", modes)
    if args.pdl is not None:
        kernels.set_programmatic_launch(args.pdl)
    if args.no_fold_norm:
        kernels.FUSE_NORM_INTO_PRODUCT = False
    for item in args.set:
        name, _, value = item.partition("=")
        if isinstance(getattr(kernels, name, None), (int, bool)):
            setattr(kernels, name, int(value))
        elif kernels.get_option(name) >= 0:
            kernels.set_option(name, int(value))
        else:
            parser.error(f"libmir_b200.kernels has no constant or option {name}")
    if args.stream_shape:
        splits, ring_kb, tile_rows = (int(v) for v in args.stream_shape.split(","))
        lib = kernels.library("bf16")
        if lib.mir_gemm_tc_stream_set_splits(splits, ring_kb, tile_rows) != 0:
            parser.error(lib.mir_last_error().decode())
    if args.deep_ring_ctas is not None:
        import ctypes
        lib = kernels.library("bf16")
        lib.mir_decode_attention_set_deep_ring_ctas.argtypes = [ctypes.c_longlong]
        lib.mir_decode_attention_set_deep_ring_ctas.restype = None
        lib.mir_decode_attention_set_deep_ring_ctas(args.deep_ring_ctas)
    peaks, peaks_kind = read_peaks()
    sizes_name, sizes_config = SIZES[args.sizes]
    config = dict(sizes_config)
    layers_full = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    layers = config["num_hidden_layers"]
    prompt_tokens = args.context
    if not 1 <= prompt_tokens <= 8192 and args.phase != "decode":
        parser.error("--context above 8,192 only with --phase decode (one prefill step holds up to 8,192 tokens)")
    max_batch = args.batch if (args.skip_points or args.phase != "all") else max(64, args.batch)
    context_limit = prompt_tokens + GENERATED_TOKENS + args.steps + args.warmup + 64
    if args.phase == "serve":                                 # 64 requests of up to 4,096 + 128 tokens
        max_batch, context_limit = 64, 4096 + 128 + 64
    pages = max_batch * (-(-context_limit // PAGE_SIZE)) + 64
    runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=PAGE_SIZE, block_count=pages),
                            scheduler=SchedulerConfig(max_batch_requests=max_batch, max_batch_tokens=8192,
                                                      prefill_chunk_tokens=4096),
                            cuda=CudaConfig(decode_graphs=not args.no_graphs), dtype="bfloat16")
    torch.cuda.set_device(0)
    model = Library(runtime).load_random(config, seed=0)
    rng = np.random.default_rng(0)
    vocab = config["vocab_size"]
    for buffer in model.storage.buffers:                      # synthetic cache content
        buffer.normal_(0.0, 0.5)
    kv_bytes_per_token = sum(len(g.entries) * g.requirement.elements_per_token * 2 for g in model.cache.groups)
    weight_bytes = model.decoder.weight_bytes_per_step()

    def fill(batch):
        ids = []
        for index in range(batch):
            request_id = f"d{batch}-{index}"
            seq = model.cache.admit(request_id)
            model.cache.grow(seq, prompt_tokens)
            model.cache.commit(seq, prompt_tokens)
            ids.append(request_id)
        return ids

    def release(ids):
        for request_id in ids:
            model.release(request_id)

    def event_pair():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def decode_device(batch, steps, warmup, repeats=1):
        """`repeats` regions of K back-to-back decode steps on the device, each after W warm-up steps from the same
        context; returns (tokens/s, ms per step, launches, clocks, context, ms per step of every region) with the
        median region's time."""
        regions, launches = [], 0
        with ClockSampler() as clocks:
            for _ in range(repeats):
                ids = fill(batch)
                samplers = [RequestSampler() for _ in ids]
                tokens = rng.integers(0, vocab, size=batch).tolist()
                entries = [StepEntry(i, [t], [0]) for i, t in zip(ids, tokens)]
                out = model.decode_many(entries, samplers, warmup)
                entries = [StepEntry(i, [int(t)], [0]) for i, t in zip(ids, out[-1].tolist())]
                torch.cuda.synchronize()
                launches = kernels.launches()
                start, stop = event_pair()
                start.record()
                model.decode_many(entries, samplers, steps)
                stop.record()
                torch.cuda.synchronize()
                regions.append(start.elapsed_time(stop) / steps)
                launches = kernels.launches() - launches
                release(ids)
        ms_per_step = statistics.median(regions)
        context = prompt_tokens + warmup + steps / 2.0
        return batch * 1e3 / ms_per_step, ms_per_step, launches, clocks.summary(), context, regions

    def decode_e2e(batch, steps, warmup, profile=False):
        """The same through Model.step: host ids in, sampled ids out, every step."""
        ids = fill(batch)
        samplers = [RequestSampler() for _ in ids]
        tokens = rng.integers(0, vocab, size=batch).tolist()
        h2d = d2h = 0
        started = None
        for step in range(warmup + steps):
            if step == warmup:
                torch.cuda.synchronize()
                if profile:
                    torch.cuda.profiler.start()
                started = time.perf_counter()
            result = model.step([StepEntry(i, [t], [0]) for i, t in zip(ids, tokens)], samplers)
            tokens = result.tokens.cpu().tolist()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        if profile:
            torch.cuda.profiler.stop()
        graphs = model.runner._graphs.graphs if model.runner._graphs else {}
        for graph in graphs.values():
            if graph.rows >= batch:
                h2d = max(h2d, graph.staging.numel() * 4)
        d2h = batch * 4
        release(ids)
        return batch * steps / seconds, h2d, d2h

    def prefill(repeats=5, profile=False):
        tokens = rng.integers(0, vocab, size=prompt_tokens).tolist()
        times = []
        for index in range(repeats + 2):
            request_id = f"p{index}"
            model.admit(request_id)
            start, stop = event_pair()
            torch.cuda.synchronize()
            if profile and index == 2:
                torch.cuda.profiler.start()
            start.record()
            result = model.step([StepEntry(request_id, tokens, [prompt_tokens - 1])], [RequestSampler()])
            stop.record()
            torch.cuda.synchronize()
            result.tokens.cpu()
            model.release(request_id)
            if index >= 2:
                times.append(start.elapsed_time(stop))
        if profile:
            torch.cuda.profiler.stop()
        return statistics.median(times)

    def mixed_step(decodes=32, portion=512, repeats=5):
        """One step of `decodes` single decoded tokens beside one prompt portion of `portion` tokens (ms, host
        clock around Model.step and the read of the logits)."""
        ids = fill(decodes)
        tokens = rng.integers(0, vocab, size=portion).tolist()
        times = []
        for index in range(repeats + 1):
            model.admit("mixed")
            entries = [StepEntry("mixed", tokens, [portion - 1])] + [StepEntry(i, [5], [0]) for i in ids]
            torch.cuda.synchronize()
            started = time.perf_counter()
            model.step(entries).logits[:, :8].cpu()
            times.append((time.perf_counter() - started) * 1e3)
            model.release("mixed")
        release(ids)
        return statistics.median(times[1:])

    def kernel_points(batch, repeats=5):
        """Each dominant kernel of the step alone at this model's layer sizes: (microseconds, fraction of its
        roofline).  A kernel runs 24 times inside one CUDA graph, each time on another copy of its weights (or
        another layer of the cache), together more than the L2 holds, so every launch reads from HBM; the graph is
        replayed `repeats` times and the median per-launch time is taken (CUDA events).  Decode kernels (few rows)
        are measured against the copy bandwidth over the bytes they must read, the prompt kernels (2,048 rows)
        against the matrix-product peak over their flops."""
        import math
        bf16, f32 = torch.bfloat16, torch.float32
        results = {}
        launches_per_graph = 24

        def timed(build, work, peak):
            calls = build()
            for call in calls[:2]:
                call()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for index in range(launches_per_graph):
                    calls[index % len(calls)]()
            graph.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(repeats):
                start, stop = event_pair()
                start.record()
                graph.replay()
                stop.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(stop) * 1e3 / launches_per_graph)
            us = statistics.median(times)
            return [round(us, 2), round(work / (us * 1e-6) / peak, 4)]

        def copies_of(rows, cols, scale=0.02):
            count = max(2, min(launches_per_graph, -(-(400 << 20) // (rows * cols * 2))))
            return [torch.randn(rows, cols, device="cuda", dtype=bf16) * scale for _ in range(count)]

        hbm, flops_peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
        qkv_width = (heads + 2 * kv_heads) * dim
        shapes = {"qkv": (qkv_width, hidden), "output": (hidden, heads * dim), "gate_up": (2 * inter, hidden),
                  "down": (hidden, inter)}
        for rows, label in ((batch, f"decode_b{batch}"), (prompt_tokens, f"prefill_{prompt_tokens}")):
            for name, (n, k) in shapes.items():
                def build(n=n, k=k, name=name, rows=rows):
                    weights = copies_of(n, k)
                    x = torch.randn(rows, k, device="cuda", dtype=bf16)
                    if name == "gate_up":
                        out = torch.empty(rows, n // 2, device="cuda", dtype=bf16)
                        scratch = lambda shape, dtype: torch.empty(shape, device="cuda", dtype=dtype)
                        return [lambda w=w: kernels.gate_up_silu(x, w, out, scratch) for w in weights]
                    if name == "qkv":
                        out = torch.empty(rows, n, device="cuda", dtype=bf16)
                        return [lambda w=w: kernels.linear(x, w, out) for w in weights]
                    out = torch.zeros(rows, n, device="cuda", dtype=f32)
                    return [lambda w=w: kernels.linear(x, w, out, accumulate=True) for w in weights]
                if rows == batch:
                    results[f"{label}_{name}"] = timed(build, n * k * 2, hbm)
                else:
                    results[f"{label}_{name}"] = timed(build, 2.0 * rows * n * k, flops_peak)
        # the output head of a decode step
        def build_head():
            x = torch.randn(batch, hidden, device="cuda", dtype=bf16)
            out = torch.empty(batch, vocab, device="cuda", dtype=f32)
            return [lambda: kernels.linear(x, model.decoder.head, out)]
        results[f"decode_b{batch}_head"] = timed(build_head, vocab * hidden * 2, hbm)
        # attention over distinct layers of the cache: decoded tokens, and one prompt
        group = model.cache.groups[0]
        views = [model.storage.views[entry] for entry in group.entries]
        ids = fill(batch)
        sequences = [model.cache.live[i] for i in ids]
        width = max(len(seq.tables[0]) for seq in sequences)
        table = torch.tensor([seq.tables[0] + [-1] * (width - len(seq.tables[0])) for seq in sequences],
                             dtype=torch.int32, device="cuda")
        positions = torch.full((batch,), prompt_tokens - 1, dtype=torch.int32, device="cuda")
        qkv = torch.randn(batch, qkv_width, device="cuda", dtype=bf16)
        mixed = torch.empty(batch, heads * dim, device="cuda", dtype=bf16)
        partition, count, floats = kernels.decode_attention_plan(batch, heads, kv_heads, dim, PAGE_SIZE, prompt_tokens)
        scratch = torch.empty(max(1, floats), device="cuda")
        scale = 1.0 / math.sqrt(dim)
        def build_decode_attention():
            return [lambda v=v: kernels.decode_attention(qkv, mixed, v.k_pages, v.v_pages, table, positions, PAGE_SIZE,
                                                         heads, kv_heads, dim, scale, None, partition, count, scratch)
                    for v in views]
        results[f"decode_b{batch}_attention"] = timed(build_decode_attention,
                                                      batch * prompt_tokens * kv_heads * dim * 2 * 2, hbm)
        release(ids)
        ids = fill(1)
        table = torch.tensor([model.cache.live[ids[0]].tables[0]], dtype=torch.int32, device="cuda")
        qkv = torch.randn(prompt_tokens, qkv_width, device="cuda", dtype=bf16)
        mixed = torch.empty(prompt_tokens, heads * dim, device="cuda", dtype=bf16)
        starts = torch.tensor([0, prompt_tokens], dtype=torch.int32, device="cuda")
        lens = torch.tensor([prompt_tokens], dtype=torch.int32, device="cuda")
        def build_prompt_attention():
            return [lambda v=v: kernels.prefill_attention(qkv, mixed, v.k_pages, v.v_pages, table, starts, lens,
                                                          PAGE_SIZE, heads, kv_heads, dim, scale, None) for v in views]
        results[f"prefill_{prompt_tokens}_attention"] = timed(
            build_prompt_attention, 4.0 * heads * dim * prompt_tokens * (prompt_tokens + 1) / 2.0, flops_peak)
        release(ids)
        return results

    hidden, inter, heads, kv_heads, dim = (config[k] for k in ("hidden_size", "intermediate_size",
                                                               "num_attention_heads", "num_key_value_heads",
                                                               "head_dim"))
    per_layer = hidden * (heads + 2 * kv_heads) * dim + heads * dim * hidden + 3 * hidden * inter
    gemm_flops = 2.0 * prompt_tokens * per_layer * layers + 2.0 * hidden * vocab
    attention_flops = 4.0 * heads * dim * (prompt_tokens * (prompt_tokens + 1) / 2.0) * layers
    prefill_flops = gemm_flops + attention_flops

    if args.phase == "decode":
        device_value = device_ms = launches = hbm_frac = 0.0
        if not args.no_graphs:
            device_value, device_ms, launches, _, context, _ = decode_device(args.batch, args.steps, args.warmup,
                                                                            args.repeats)
            step_bytes = weight_bytes + args.batch * context * kv_bytes_per_token
            hbm_frac = step_bytes / (device_ms / 1e3) / 1e9 / peaks["hbm_gbs"]
        tokens_per_second, _, _ = decode_e2e(args.batch, args.steps, args.warmup, profile=True)
        print(json.dumps({"phase": "decode", "batch": args.batch, "steps": args.steps, "layers": layers,
                          "graphs": not args.no_graphs, "tokens_per_second": round(tokens_per_second, 1),
                          "device_tokens_per_second": round(device_value, 1), "device_ms_per_step": round(device_ms, 4),
                          "context": prompt_tokens, "hbm_frac": round(hbm_frac, 4),
                          "launches_per_step": launches / max(1, args.steps)}))
        return 0
    if args.phase == "serve":
        # BASELINE.json configs[3]'s workload: 64 requests through the scheduler (Model.generate_batch), prompt
        # lengths uniform in 16..4,096, 128 generated tokens each; the second of two runs is timed.
        from libmir_b200.config.generation import GenerationOverrides
        from libmir_b200.engine.api import GenerationRequest
        lengths = rng.integers(16, 4097, size=64).tolist()
        options = GenerationOverrides(max_tokens=128, ignore_eos=True)

        def run():
            requests = [GenerationRequest(prompt_ids=rng.integers(0, vocab, size=n).tolist(), options=options)
                        for n in lengths]
            torch.cuda.synchronize()
            started = time.perf_counter()
            outputs = model.generate_batch(requests)
            torch.cuda.synchronize()
            return sum(len(o.token_ids) for o in outputs), time.perf_counter() - started, outputs[0].metrics["steps"]

        run()
        generated, seconds, steps = run()
        print(json.dumps({"phase": "serve", "requests": 64, "prompt_tokens": int(sum(lengths)),
                          "generated_tokens": generated, "seconds": round(seconds, 3), "steps": steps,
                          "generated_tokens_per_second": round(generated / seconds, 1),
                          "all_tokens_per_second": round((generated + sum(lengths)) / seconds, 1), "layers": layers}))
        return 0
    if args.phase == "trace":
        # A few captured decode steps with the traced kernels (csrc/trace.cuh), then the last step's records on one
        # time line: microseconds since the step's first record, per launch the first CTA and the last one.
        decode_device(args.batch, 3, 2, 1)
        records = kernels.read_trace()
        names = {
            "stream": ["start", "weights_asked", "dependency", "activations_asked", "first_stage", "last_stage",
                       "products_done", "cluster_barrier", "written", "second_barrier"],
            "decode": ["start", "set_up", "loads_may_go", "dependency", "queries_in", "scores_issued", "first_scores",
                       "first_p", "last_scores", "last_p", "last_product", "written", "end"],
            "merge": ["start", "dependency", "end"], "rope": ["start", "dependency", "end"]}
        stream_kinds = {0: "store (QKV)", 1: "accumulate (output / down)", 2: "float32 (head)", 3: "SwiGLU (gate-up)"}
        rows = []
        for group, table in records.items():
            for record in table:
                tag = int(record[15])
                what = f"stream {stream_kinds[tag // 2]}" if group == "stream" else group
                if group == "decode":
                    what += f" ({int(record[14])} tiles)"
                rows.append((int(record[0]), what, "first CTA" if tag % 2 == 0 else "last CTA", group, record))
        rows.sort(key=lambda row: row[0])
        per_step = (layers * 7 + 1) * 2                       # launches with records in a step, two CTAs each
        rows = rows[-per_step:]
        origin = rows[0][0] if rows else 0
        for _, what, which, group, record in rows:
            stamps = " ".join(f"{name}={(int(record[i]) - origin) / 1e3:.2f}" for i, name in enumerate(names[group])
                              if record[i] > 0)
            print(f"{what:36s} {which:9s} {stamps}")
        print(json.dumps({"phase": "trace", "batch": args.batch, "layers": layers, "records": len(rows),
                          "unit": "us since the step's first record"}))
        return 0
    if args.phase == "kernels":
        print(json.dumps({"phase": "kernels", "batch": args.batch, "context": prompt_tokens,
                          "kernels": kernel_points(args.batch)}))
        return 0
    if args.phase == "prefill":
        ms = prefill(repeats=max(1, min(args.steps, 5)), profile=True)
        print(json.dumps({"phase": "prefill", "tokens": prompt_tokens, "layers": layers, "ms": round(ms, 3),
                          "frac_of_peak": round(prefill_flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}))
        return 0

    value, ms_per_step, launches, clocks, context, regions = decode_device(args.batch, args.steps, args.warmup,
                                                                           args.repeats)
    step_bytes = weight_bytes + args.batch * context * kv_bytes_per_token
    achieved_gbs = step_bytes / (ms_per_step / 1e3) / 1e9
    e2e_value, h2d, d2h = decode_e2e(args.batch, args.steps, args.warmup)
    prefill_ms = prefill()
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            points[f"decode_b{batch}"] = round(decode_device(batch, args.steps, args.warmup, args.repeats)[0], 1)
        points["mixed_32_decodes_512_prompt_tokens_ms"] = round(mixed_step(32, 512), 3)

    line = {
        "metric": f"decode tok/s at batch {args.batch} ({sizes_name.split(' (')[0]}, 2,048-token context, 1 B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random token ids, random N(0,0.02) weights, random cache",
        "config": {
            "model": sizes_name, "layers": layers, "layers_of_config": layers_full,
            "hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": dim, "intermediate": inter,
            "vocab": vocab, "global_batch": args.batch, "seq_len": prompt_tokens + GENERATED_TOKENS,
            "context_at_decode": round(context, 1), "page_size": PAGE_SIZE, "tied_embeddings": bool(config.get("tie_word_embeddings", False)),
            "parallelism": "1 GPU", "l2": "inputs larger than L2 (a step reads every weight and the cache)",
            "peaks": peaks_kind, "timed_regions": args.repeats,
        },
        "ms_per_step_regions": [round(r, 4) for r in regions],
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "prefill": {"value": round(prompt_tokens / (prefill_ms / 1e3), 1), "tokens": prompt_tokens,
                    "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernel_points(args.batch) if not args.skip_points else {},
        "native_libraries": sorted(os.path.basename(p) for p in kernels.loaded_libraries().values()),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
