"""Shared helpers of the tests: model folders made in temporary places, traces, tolerances."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import plain_impl

ROOT = Path(__file__).resolve().parent.parent

# Tolerances, chosen once from the arithmetic and never widened to make a test pass:
#   float32: every reduction is 32-bit (eps 6e-8); logits of magnitude ~1 after a few hundred-term
#            dot products through <= 4 layers differ from the float64 oracle by a few 1e-7.
#   bfloat16: weights are the same bf16 values in both; activations are rounded to bf16 (eps 3.9e-3)
#            between kernels, which through a few layers gives errors of a few 1e-3 on logits ~1.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def make_folder(tmp_path, config: dict, seed: int, dtype: str, sharpen: float = 1.0) -> Path:
    """Write config.json + model.safetensors with random weights.  `sharpen` scales the query and key
    projections (or the q/k-norm weights) so that attention is far from uniform and one missed or
    extra key changes the logits well beyond the tolerance."""
    from libmir_b200.weights import read_catalog, load_tensor, write_file, write_model_folder
    folder = write_model_folder(Path(tmp_path), config, seed=seed, dtype=dtype)
    if sharpen != 1.0:
        entries = read_catalog(folder)
        tensors = {name: load_tensor(entry) for name, entry in entries.items()}
        has_norm = any(name.endswith("q_norm.weight") for name in tensors)
        for name in tensors:
            if has_norm and (name.endswith("q_norm.weight") or name.endswith("k_norm.weight")):
                tensors[name] = tensors[name] * (sharpen ** 0.5)
            elif not has_norm and (name.endswith("q_proj.weight") or name.endswith("k_proj.weight")):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
            elif name.endswith("embed_tokens.weight"):
                tensors[name] = (tensors[name].float() * 8.0).to(tensors[name].dtype)
        write_file(folder / "model.safetensors", tensors)
    return folder


def plain_logits(folder, ids) -> np.ndarray:
    config, weights = plain_impl.read_model(folder)
    return plain_impl.forward(config, weights, list(ids)).numpy()


def random_ids(rng, vocab: int, n: int) -> list:
    return rng.integers(0, vocab, size=n).tolist()


def round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


# ------------------------------------------------------------------------------ traces
class Trace:
    """Builds the JSON lines that bin/trace_run reads and remembers what each output row is."""

    def __init__(self):
        self.lines = []
        self.expect = []         # per step: list of (request name, absolute position)
        self.live = {}           # request name -> tokens fed so far
        self.peak = 0

    def step(self, entries, end=()):
        """entries: list of (name, tokens, want local indices)."""
        record = {"step": len(self.lines), "entries": [], "end": list(end)}
        rows = []
        for name, tokens, want in entries:
            start = self.live.get(name, 0)
            record["entries"].append({"id": name, "tokens": [int(t) for t in tokens], "want": [int(w) for w in want]})
            rows += [(name, start + w) for w in want]
            self.live[name] = start + len(tokens)
        self.peak = max(self.peak, sum(round_up(n, 64) for n in self.live.values()))
        for name in end:
            self.live.pop(name, None)
        self.lines.append(json.dumps(record))
        self.expect.append(rows)
        return self

    def text(self) -> str:
        return "\n".join(self.lines) + "\n"


def run_trace(folder, dtype: str, trace: Trace, out_dir, max_tokens=None, extra_args=()):
    """Run bin/trace_run as a user would; returns {step: array [wanted, vocab]}."""
    out_dir = Path(out_dir)
    command = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
               "--out", str(out_dir), "--max-tokens", str(max_tokens or trace.peak), *extra_args]
    done = subprocess.run(command, input=trace.text(), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, f"trace_run failed:\n{done.stdout[-2000:]}\n{done.stderr[-4000:]}"
    acknowledged = [line for line in done.stdout.splitlines() if line.startswith("done ")]
    assert acknowledged == [f"done {i}" for i in range(len(trace.lines))], done.stdout[-2000:]
    vocab = json.loads((Path(folder) / "config.json").read_text())["vocab_size"]
    results = {}
    for index, rows in enumerate(trace.expect):
        path = out_dir / f"{index}.f32"
        if not rows:
            assert not path.exists()
            continue
        values = np.fromfile(path, dtype="<f4")
        assert values.size == len(rows) * vocab, f"step {index}: {values.size} floats for {len(rows)} rows"
        results[index] = values.reshape(len(rows), vocab)
    return results


def compare_trace(results, trace: Trace, reference: dict, tol: float, label: str):
    """Every wanted row against the plain implementation's logits; reports the first wrong row."""
    worst = 0.0
    for index, rows in enumerate(trace.expect):
        for row, (name, position) in enumerate(rows):
            want = reference[name][position]
            got = results[index][row]
            error = float(np.abs(got - want).max())
            scale = max(1.0, float(np.abs(want).max()))
            assert np.isfinite(got).all(), f"{label}: step {index} request {name} position {position}: not finite"
            assert error <= tol * scale, (
                f"{label}: first wrong logits at step {index}, request {name}, position {position}: "
                f"max |diff| {error:.3e} > {tol * scale:.3e}")
            worst = max(worst, error / scale)
    return worst
