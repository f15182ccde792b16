"""Typed reading of a decoder's config.json.

Keys, aliases, defaults and error texts follow libmir's
models/src/layout/decoder/parse/mod.rs:40-166 and parse/value.rs:5-108:
an alias list is tried in order, `null` means absent, and a value of the wrong
JSON type is an error that names the key.  Nothing here knows which model will
be built from the numbers; `libmir_b200.models` turns a DecoderConfig into a
ModelSpec.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional, Sequence

from ..errors import ConfigError

_NESTED_SECTIONS = ("text_config", "language_config", "llm_config")
LAYER_TYPES = ("full_attention", "sliding_attention")


def _present(value: Mapping[str, Any], key: str) -> bool:
    return key in value


def optional_usize(value: Mapping[str, Any], keys: Sequence[str]) -> Optional[int]:
    for key in keys:
        if not _present(value, key):
            continue
        raw = value[key]
        if raw is None:
            return None
        if isinstance(raw, bool) or not isinstance(raw, int) or raw < 0:
            raise ConfigError(f"{key} must be an unsigned integer")
        return raw
    return None


def require_usize(value: Mapping[str, Any], keys: Sequence[str]) -> int:
    found = optional_usize(value, keys)
    if found is None:
        raise ConfigError("missing " + " or ".join(keys))
    return found


def optional_f64(value: Mapping[str, Any], keys: Sequence[str]) -> Optional[float]:
    for key in keys:
        if not _present(value, key):
            continue
        raw = value[key]
        if raw is None:
            return None
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise ConfigError(f"{key} must be a number")
        return float(raw)
    return None


def optional_bool(value: Mapping[str, Any], key: str) -> Optional[bool]:
    raw = value.get(key)
    if raw is None:
        return None
    if not isinstance(raw, bool):
        raise ConfigError(f"{key} must be a boolean")
    return raw


def optional_string(value: Mapping[str, Any], key: str) -> Optional[str]:
    raw = value.get(key)
    if raw is None:
        return None
    if not isinstance(raw, str):
        raise ConfigError(f"{key} must be a string")
    return raw


@dataclass(frozen=True)
class RopeScaling:
    """llama3 piecewise frequency interpolation (models/src/layout/decoder/rope.rs:61-95)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


def _rope_scaling(decoder: Mapping[str, Any]) -> Optional[RopeScaling]:
    raw = decoder.get("rope_scaling")
    if raw is None:
        parameters = decoder.get("rope_parameters")
        if isinstance(parameters, Mapping) and parameters.get("rope_type") not in (None, "default"):
            raw = parameters
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError("rope_scaling must be an object")
    rope_type = raw.get("rope_type", raw.get("type"))
    if not isinstance(rope_type, str):
        raise ConfigError("rope_scaling.rope_type must be a string")
    if rope_type == "default":
        return None
    if rope_type != "llama3":
        raise ConfigError(f"unsupported rope_scaling type {rope_type}")
    numbers = {}
    for key in ("factor", "low_freq_factor", "high_freq_factor"):
        number = raw.get(key)
        if isinstance(number, bool) or not isinstance(number, (int, float)):
            raise ConfigError(f"rope_scaling.{key} must be a number")
        numbers[key] = float(number)
    original = raw.get("original_max_position_embeddings")
    if isinstance(original, bool) or not isinstance(original, int):
        raise ConfigError("rope_scaling.original_max_position_embeddings must be an unsigned integer")
    if (not all(math.isfinite(v) for v in numbers.values()) or numbers["factor"] <= 0.0
            or numbers["low_freq_factor"] <= 0.0
            or numbers["high_freq_factor"] <= numbers["low_freq_factor"] or original <= 0):
        raise ConfigError("invalid piecewise rope_scaling parameters")
    return RopeScaling(original_max_position_embeddings=original, **numbers)


def _rope_theta(decoder: Mapping[str, Any]) -> Optional[float]:
    theta = optional_f64(decoder, ["rope_theta", "rotary_emb_base"])
    if theta is not None:
        return theta
    parameters = decoder.get("rope_parameters")
    if isinstance(parameters, Mapping):
        inner = parameters.get("rope_theta")
        if isinstance(inner, (int, float)) and not isinstance(inner, bool):
            return float(inner)
    return None


def _partial_rotary_factor(decoder: Mapping[str, Any]) -> Optional[float]:
    factor = optional_f64(decoder, ["partial_rotary_factor"])
    if factor is not None:
        return factor
    parameters = decoder.get("rope_parameters")
    if isinstance(parameters, Mapping) and parameters.get("partial_rotary_factor") is not None:
        raw = parameters["partial_rotary_factor"]
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise ConfigError("rope partial_rotary_factor must be a number")
        return float(raw)
    return None


def _layer_types(decoder: Mapping[str, Any], count: int) -> tuple[str, ...]:
    raw = decoder.get("layer_types")
    if raw is None:
        return ("full_attention",) * count
    if not isinstance(raw, list):
        raise ConfigError("layer_types must be an array")
    if len(raw) != count:
        raise ConfigError(f"layer_types has {len(raw)} entries, expected {count}")
    for item in raw:
        if not isinstance(item, str):
            raise ConfigError("layer_types entries must be strings")
        if item not in LAYER_TYPES:
            raise ConfigError(f"unsupported layer_type {item}")
    return tuple(raw)


@dataclass(frozen=True)
class DecoderConfig:
    """Every number of config.json that a dense decoder is built from."""

    architectures: tuple[str, ...]
    model_type: Optional[str]
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    partial_rotary_factor: float
    layer_types: tuple[str, ...]
    sliding_window: Optional[int]
    tie_word_embeddings: bool
    attention_scale: Optional[float]
    embedding_multiplier: float
    attention_bias: Optional[bool]
    qk_normalization: Optional[bool]
    hidden_activation: Optional[str]
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # -- derived -------------------------------------------------------------
    def layer_sliding_window(self, index: int) -> Optional[int]:
        """models/src/layout/decoder/attention.rs:77-80: the window binds sliding layers only."""
        return self.sliding_window if self.layer_types[index] == "sliding_attention" else None

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    @property
    def softmax_scale(self) -> float:
        return self.attention_scale if self.attention_scale is not None else 1.0 / math.sqrt(self.head_dim)

    # -- construction --------------------------------------------------------
    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> "DecoderConfig":
        if not isinstance(value, Mapping):
            raise ConfigError("config.json must hold a JSON object")
        decoder = value
        for key in _NESTED_SECTIONS:
            if isinstance(value.get(key), Mapping):
                decoder = value[key]
                break
        shared = optional_usize(decoder, ["num_kv_shared_layers"])
        if shared:
            raise ConfigError("shared K/V layers are not supported")
        heads = require_usize(decoder, ["num_attention_heads", "n_head"])
        if heads == 0:
            raise ConfigError("num_attention_heads must be greater than zero")
        hidden = require_usize(decoder, ["hidden_size", "n_embd"])
        layers = require_usize(decoder, ["num_hidden_layers", "num_layers", "n_layer"])
        head_dim = optional_usize(decoder, ["head_dim", "attention_head_dim", "kv_channels"])
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("hidden_size must be divisible by num_attention_heads")
            head_dim = hidden // heads
        kv_heads = optional_usize(decoder, ["num_key_value_heads", "multi_query_group_num", "n_kv_heads"])
        kv_heads = heads if kv_heads is None else kv_heads
        intermediate = optional_usize(decoder, ["intermediate_size", "ffn_hidden_size", "n_inner"])
        if intermediate is None:
            raise ConfigError("missing intermediate_size or ffn_hidden_size or n_inner")
        for key in ("num_experts", "num_local_experts", "n_routed_experts"):
            if optional_usize(decoder, [key]):
                raise ConfigError(f"{key} is set: routed experts are not part of the dense SwiGLU decoder")
        if optional_f64(decoder, ["final_logit_softcapping"]):
            raise ConfigError("final_logit_softcapping is not part of the dense SwiGLU decoder")
        if optional_bool(decoder, "attention_sinks"):
            raise ConfigError("attention_sinks are not part of the dense SwiGLU decoder")
        activation = optional_string(decoder, "hidden_activation") or optional_string(decoder, "hidden_act")
        if activation is not None and activation != "silu":
            raise ConfigError(f"hidden_act {activation} is not supported: the feed-forward is SwiGLU (silu)")
        partial = _partial_rotary_factor(decoder)
        tie = optional_bool(decoder, "tie_word_embeddings")
        if tie is None:
            tie = optional_bool(value, "tie_word_embeddings")
        architectures = value.get("architectures") or decoder.get("architectures") or []
        if not isinstance(architectures, list) or not all(isinstance(a, str) for a in architectures):
            raise ConfigError("architectures must be an array of strings")
        scale = optional_f64(decoder, ["attention_scale", "attention_multiplier"])
        qk = decoder.get("qk_normalization")
        if qk is not None and not isinstance(qk, bool):
            raise ConfigError("qk_normalization must be a boolean")
        config = cls(
            architectures=tuple(architectures),
            model_type=optional_string(decoder, "model_type") or optional_string(value, "model_type"),
            hidden_size=hidden,
            intermediate_size=intermediate,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=require_usize(decoder, ["vocab_size"]),
            max_position_embeddings=optional_usize(
                decoder, ["max_position_embeddings", "max_sequence_length", "seq_length", "n_positions"]) or 4096,
            rms_norm_eps=_or(optional_f64(
                decoder, ["rms_norm_eps", "layer_norm_epsilon", "layernorm_epsilon", "norm_epsilon"]), 1e-5),
            rope_theta=_or(_rope_theta(decoder), 10000.0),
            rope_scaling=_rope_scaling(decoder),
            partial_rotary_factor=_or(partial, 1.0),
            layer_types=_layer_types(decoder, layers),
            sliding_window=optional_usize(decoder, ["sliding_window"]),
            tie_word_embeddings=bool(tie),
            attention_scale=scale,
            embedding_multiplier=_or(optional_f64(decoder, ["embedding_multiplier"]), 1.0),
            attention_bias=optional_bool(decoder, "attention_bias"),
            qk_normalization=qk,
            hidden_activation=activation,
            raw=dict(value),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.hidden_size == 0 or self.intermediate_size == 0 or self.vocab_size == 0:
            raise ConfigError("hidden_size, intermediate_size and vocab_size must be greater than zero")
        if self.num_hidden_layers == 0:
            raise ConfigError("num_hidden_layers must be greater than zero")
        if self.num_key_value_heads == 0 or self.head_dim == 0:
            raise ConfigError("KV head count and head_dim must be greater than zero")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if self.sliding_window == 0:
            raise ConfigError("sliding_window must be greater than zero")
        if "sliding_attention" in self.layer_types and self.sliding_window is None:
            raise ConfigError("layer_types names sliding_attention but sliding_window is missing")
        if self.attention_scale is not None and (not math.isfinite(self.attention_scale) or self.attention_scale <= 0):
            raise ConfigError("attention_scale must be finite and greater than zero")
        if not (math.isfinite(self.rms_norm_eps) and self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be finite and greater than zero")
        if not (math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError("rope_theta must be finite and greater than zero")
        if not 0.0 < self.partial_rotary_factor <= 1.0:
            raise ConfigError("partial_rotary_factor must be in (0, 1]")

    @classmethod
    def from_folder(cls, folder) -> "DecoderConfig":
        path = Path(folder) / "config.json"
        if not path.is_file():
            raise ConfigError(f"missing file {path}")
        try:
            value = json.loads(path.read_text())
        except json.JSONDecodeError as error:
            raise ConfigError(f"{path} is not valid JSON: {error}") from error
        return cls.from_dict(value)

    def to_dict(self) -> dict:
        """A config.json that reads back to an equal DecoderConfig (used by the random-weights writer)."""
        out: dict[str, Any] = {
            "architectures": list(self.architectures),
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
        }
        if self.model_type is not None:
            out["model_type"] = self.model_type
        if self.rope_scaling is not None:
            out["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": self.rope_scaling.factor,
                "low_freq_factor": self.rope_scaling.low_freq_factor,
                "high_freq_factor": self.rope_scaling.high_freq_factor,
                "original_max_position_embeddings": self.rope_scaling.original_max_position_embeddings,
            }
        if self.partial_rotary_factor != 1.0:
            out["partial_rotary_factor"] = self.partial_rotary_factor
        if any(kind != "full_attention" for kind in self.layer_types):
            out["layer_types"] = list(self.layer_types)
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
        if self.attention_scale is not None:
            out["attention_scale"] = self.attention_scale
        if self.embedding_multiplier != 1.0:
            out["embedding_multiplier"] = self.embedding_multiplier
        if self.attention_bias is not None:
            out["attention_bias"] = self.attention_bias
        if self.qk_normalization is not None:
            out["qk_normalization"] = self.qk_normalization
        return out


def _or(value, default):
    return default if value is None else value
