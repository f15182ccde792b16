"""Plain, slow, whole-sequence implementation of the dense SwiGLU decoder.

This file is the oracle of the test-suite.  It rests on the FORMULAS of
mirmir-tech/libmir (the reference is a Rust workspace that cannot be compiled
or imported here: no cargo, no network, three crates that are not in the
tree), so there is no golden output of the reference's own code beside it.
Every function cites the reference file and lines whose arithmetic it restates.

Rules it keeps:
  * whole sequences, no cache, no paging, no batching: one request at a time;
  * one function for each part;
  * float64 arithmetic on the weights as stored (the caller rounds the weights
    to bfloat16 first when it wants the bfloat16 model);
  * it shares no code with the `libmir_b200` package: it reads config.json
    and model.safetensors by itself with `json` and `struct`.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
_ST_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """u64 little-endian header length, JSON header, payload.

    models/src/weights/catalog.rs:125-168 (header), :28-39 (payload offset).
    """
    raw = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + header_len])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dtype, _ = _ST_DTYPES[meta["dtype"]]
        begin, end = meta["data_offsets"]
        buf = bytearray(raw[8 + header_len + begin: 8 + header_len + end])
        tensor = torch.frombuffer(buf, dtype=dtype).reshape(meta["shape"]).clone()
        out[name] = tensor
    return out


def read_model(folder) -> tuple[dict, dict[str, torch.Tensor]]:
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return config, weights


# --------------------------------------------------------------------------- config
def _first(config: dict, keys, default=None):
    """Alias lists as in models/src/layout/decoder/parse/value.rs:9-27 (null = absent)."""
    for key in keys:
        if key in config:
            return default if config[key] is None else config[key]
    return default


def sizes(config: dict) -> dict:
    """The numbers of models/src/layout/decoder/parse/mod.rs:46-131 that this architecture uses."""
    hidden = _first(config, ["hidden_size", "n_embd"])
    heads = _first(config, ["num_attention_heads", "n_head"])
    layers = _first(config, ["num_hidden_layers", "num_layers", "n_layer"])
    rope_parameters = config.get("rope_parameters") or {}
    theta = _first(config, ["rope_theta", "rotary_emb_base"])
    if theta is None:
        theta = rope_parameters.get("rope_theta", 10000.0)
    head_dim = _first(config, ["head_dim", "attention_head_dim", "kv_channels"], hidden // heads)
    partial = _first(config, ["partial_rotary_factor"], rope_parameters.get("partial_rotary_factor", 1.0))
    layer_types = config.get("layer_types") or ["full_attention"] * layers
    window = config.get("sliding_window")
    scaling = config.get("rope_scaling")
    if scaling is None:
        scaling = rope_parameters if rope_parameters.get("rope_type") == "llama3" else None
    return dict(
        hidden=hidden, heads=heads, layers=layers, head_dim=head_dim,
        kv_heads=_first(config, ["num_key_value_heads", "multi_query_group_num", "n_kv_heads"], heads),
        intermediate=_first(config, ["intermediate_size", "ffn_hidden_size", "n_inner"]),
        vocab=config["vocab_size"],
        eps=_first(config, ["rms_norm_eps", "layer_norm_epsilon", "layernorm_epsilon", "norm_epsilon"], 1e-5),
        theta=float(theta), rotary_dim=int(head_dim * partial) // 2 * 2,
        scaling=scaling,
        scale=_first(config, ["attention_scale", "attention_multiplier"], 1.0 / math.sqrt(head_dim)),
        embedding_multiplier=_first(config, ["embedding_multiplier"], 1.0),
        tied=bool(config.get("tie_word_embeddings") or False),
        windows=[window if kind == "sliding_attention" else None for kind in layer_types],
    )


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, ids, multiplier: float) -> torch.Tensor:
    """x0[t] = E[id_t] * m.  cuda/kernels/embedding_bf16.cu:3-19."""
    return table.to(F64)[torch.as_tensor(ids, dtype=torch.long)] * multiplier


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis.  cuda/kernels/rms_norm_bf16.cu:3-36."""
    inverse = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inverse * weight.to(F64)


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """f_i = theta^(-2i/rotary_dim), then the llama3 piecewise rule, held as float32.

    Plain: cuda/kernels/qkv_postprocess_bf16.cu:56.  llama3:
    metal/src/engine/attention/rope.rs:58-96 with the keys of
    models/src/layout/decoder/rope.rs:61-95.  The table is 32-bit in the
    reference (powf / MLX float32 graph), so it is rounded to float32 here.
    """
    index = torch.arange(0, rotary_dim, 2, dtype=F64)
    inverse = theta ** (-index / rotary_dim)
    if scaling is not None:
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position_embeddings"])
        wavelength = 2.0 * math.pi / inverse
        smooth = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
        inverse = (inverse / factor) * (1.0 - smooth) + inverse * smooth
    return inverse.to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, inverse_frequencies: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of the first rotary_dim dims of every head; x is [S, heads, D].

    angle = float32(pos) * float32(f_i) as a 32-bit product; y_i = x_i cos - x_{i+r/2} sin,
    y_{i+r/2} = x_i sin + x_{i+r/2} cos.  cuda/kernels/qkv_postprocess_bf16.cu:37-69.
    """
    half = inverse_frequencies.numel()
    angle32 = positions.to(torch.float32)[:, None] * inverse_frequencies[None, :]
    angle = angle32.to(F64)
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    first, second, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([first * cos - second * sin, first * sin + second * cos, rest], dim=-1)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ b), W is [out, in].  cuda/src/backend/linear/mod.rs:141-194."""
    y = x @ weight.to(F64).T
    return y if bias is None else y + bias.to(F64)


def attention_scores_softmax_values(q, k, v, scale: float, window: int | None) -> torch.Tensor:
    """Causal grouped-query softmax attention of one whole sequence.

    q [S, Hq, D], k and v [S, Hkv, D]; query head h reads kv head h // (Hq / Hkv);
    key j is visible to query p iff j <= p and (no window or j > p - window).
    cuda/kernels/paged_attention_bf16.cu:26-31,43-92 (scale, window, group, online softmax),
    cuda/kernels/paged_prefill_attention_batch_bf16.cu:30-35 (causal limit = position + 1).
    """
    seq, heads, dim = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(seq, heads, v.shape[2], dtype=F64)
    position = torch.arange(seq)
    visible = position[None, :] <= position[:, None]
    if window is not None:
        visible &= position[None, :] > position[:, None] - window
    for head in range(heads):
        scores = (q[:, head, :] @ k[:, head // group, :].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, head, :] = torch.softmax(scores, dim=-1) @ v[:, head // group, :]
    return out


def attention(x, weights: dict, prefix: str, s: dict, positions, window) -> torch.Tensor:
    """q/k/v projections, optional per-head q/k RMSNorm before RoPE, attention, o projection.

    metal/src/engine/dense/swiglu/attention.rs:14-112; q/k-norm is on iff both weights exist
    (models/src/semantic/compile/tensors.rs:7-18).
    """
    seq = x.shape[0]
    w = lambda name: weights.get(prefix + name)
    q = linear(x, w("q_proj.weight"), w("q_proj.bias")).reshape(seq, s["heads"], s["head_dim"])
    k = linear(x, w("k_proj.weight"), w("k_proj.bias")).reshape(seq, s["kv_heads"], s["head_dim"])
    v = linear(x, w("v_proj.weight"), w("v_proj.bias")).reshape(seq, s["kv_heads"], s["head_dim"])
    if w("q_norm.weight") is not None and w("k_norm.weight") is not None:
        q = rms_norm(q, w("q_norm.weight"), s["eps"])
        k = rms_norm(k, w("k_norm.weight"), s["eps"])
    frequencies = rope_inverse_frequencies(s["rotary_dim"], s["theta"], s["scaling"])
    q, k = rope(q, positions, frequencies), rope(k, positions, frequencies)
    mixed = attention_scores_softmax_values(q, k, v, s["scale"], window)
    return linear(mixed.reshape(seq, -1), w("o_proj.weight"), w("o_proj.bias"))


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + e^-z).  cuda/kernels/elementwise_bf16.cu:30-31."""
    return z / (1.0 + torch.exp(-z))


def swiglu(x, weights: dict, prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)).  cuda/src/backend/dense/feed_forward.rs:108-150."""
    gate = linear(x, weights[prefix + "gate_proj.weight"])
    up = linear(x, weights[prefix + "up_proj.weight"])
    return linear(silu(gate) * up, weights[prefix + "down_proj.weight"])


def block(x, weights: dict, layer: int, s: dict, positions) -> torch.Tensor:
    """x + attention(norm(x)), then x + swiglu(norm(x)).  metal/src/engine/dense/swiglu/layer.rs:123-166."""
    prefix = f"model.layers.{layer}."
    normed = rms_norm(x, weights[prefix + "input_layernorm.weight"], s["eps"])
    x = x + attention(normed, weights, prefix + "self_attn.", s, positions, s["windows"][layer])
    normed = rms_norm(x, weights[prefix + "post_attention_layernorm.weight"], s["eps"])
    return x + swiglu(normed, weights, prefix + "mlp.")


def output_head(x, weights: dict, s: dict) -> torch.Tensor:
    """Final RMSNorm (eps = rms_norm_eps, models/src/semantic/compile/mod.rs:23-26,39) and
    the tied or untied projection (models/src/weights/binding/view.rs:97-111)."""
    normed = rms_norm(x, weights["model.norm.weight"], s["eps"])
    table = weights["model.embed_tokens.weight"] if s["tied"] else weights["lm_head.weight"]
    return linear(normed, table)


def forward(config: dict, weights: dict, ids) -> torch.Tensor:
    """Logits [S, V] (float64) of one whole sequence.  metal/src/engine/dense/swiglu/model.rs:117-131."""
    s = sizes(config)
    positions = torch.arange(len(ids))
    x = embedding(weights["model.embed_tokens.weight"], ids, s["embedding_multiplier"])
    for layer in range(s["layers"]):
        x = block(x, weights, layer, s, positions)
    return output_head(x, weights, s)


# --------------------------------------------------------------------------- sampling
class SplitMix64:
    """runtime/src/sampling/mod.rs:180-203."""

    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = seed & self.MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        value = self.state
        value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & self.MASK
        return value ^ (value >> 31)

    def next_unit(self) -> float:
        return (self.next_u64() >> 32) / 4294967296.0


def greedy(logits) -> int:
    """Highest logit, lowest id on ties.  cuda/kernels/sampling_bf16.cu:18-27."""
    values = np.asarray(logits, dtype=np.float64)
    return int(np.flatnonzero(values == values.max())[0])


def sample(logits, draw: float, temperature: float, top_k: int = 0, top_p: float = 1.0,
           repetition_penalty: float = 1.0, history=()) -> int:
    """One token from one row of logits with a given uniform draw in [0, 1).

    Full-vocabulary temperature sampling walks the vocabulary in id order
    (runtime/src/sampling/mod.rs:82-116); with top-k or top-p the candidates are
    ranked by score first, weights exp((l - max) / T), top-p truncation then top-k,
    and the walk is in rank order (:72-80,118-135, candidate.rs:69-107).
    """
    values = np.asarray(logits, dtype=np.float32).copy()
    if repetition_penalty > 1.0:
        for token in set(int(t) for t in history):
            values[token] = values[token] / repetition_penalty if values[token] >= 0 else values[token] * repetition_penalty
    if temperature <= np.finfo(np.float32).eps or top_k == 1:
        return greedy(values)
    if top_p >= 1.0 and top_k == 0:
        finite = np.isfinite(values)
        weights = np.where(finite, np.exp((values - values[finite].max()).astype(np.float64) / temperature), 0.0)
        return _first_reaching(weights, draw * weights.sum())
    candidates = np.flatnonzero(np.isfinite(values))
    order = candidates[np.argsort(-values[candidates].astype(np.float64), kind="stable")]
    weights = np.exp((values[order] - values[order[0]]).astype(np.float64) / temperature)
    keep = len(order)
    if top_p < 1.0:
        keep = _first_reaching(weights / weights.sum(), top_p) + 1
    if top_k > 0:
        keep = min(keep, top_k)
    weights, order = weights[:keep], order[:keep]
    return int(order[_first_reaching(weights, draw * weights.sum())])


def _first_reaching(weights, threshold: float) -> int:
    """The walk `threshold -= w; stop when threshold <= 0` of runtime/src/sampling/mod.rs:104-113,226-238:
    the first index whose running sum (accumulated in order, in float64) reaches the threshold; the last
    index if rounding leaves none."""
    if threshold <= 0.0:
        return 0
    reached = np.flatnonzero(np.cumsum(weights) >= threshold)
    return int(reached[0]) if reached.size else len(weights) - 1
