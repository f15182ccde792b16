"""The dense SwiGLU decoder (Llama / Mistral / Qwen2 / Qwen3 checkpoints): config.json -> ModelSpec.

Every layer: RMSNorm -> grouped-query softmax attention with rotary positions (optional per-head q/k
RMSNorm, optional q/k/v and output bias, optional sliding window on layers that layer_types marks)
-> residual -> RMSNorm -> SwiGLU feed-forward -> residual; final RMSNorm; tied or untied head.
This is what libmir runs under metal/src/engine/dense/swiglu and cuda/src/backend/dense.

What the name in `architectures` contributes is only a default for options that a checkpoint would
otherwise reveal by its tensors (libmir discovers q/k-norm and biases from tensor presence,
models/src/semantic/compile/tensors.rs:7-18, weights/binding/discovery/mod.rs:179,226-232): with a
checkpoint at hand presence decides, without one (random weights) the table below does.
Tensor names: models/src/weights/binding/roles/parse.rs:17-20,46-57,61-85,101-103.
"""

from __future__ import annotations

from typing import Mapping, Optional

from ..config.decoder import DecoderConfig
from ..config.spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, RmsNormSpec, RotarySpec, ScheduleEntry,
                           SoftmaxAttentionSpec, SwiGluSpec)
from ..errors import ConfigError
from ..registry import register_architecture

STRIP_PREFIXES = ("language_model.model.", "model.language_model.", "language_model.", "model.")
LAYER_NAMES = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.",
               "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}

# defaults used only when no checkpoint is at hand: (qk_norm, qkv_bias)
ARCHITECTURE_DEFAULTS = {
    "LlamaForCausalLM": (False, False),
    "MistralForCausalLM": (False, False),
    "Qwen2ForCausalLM": (False, True),
    "Qwen3ForCausalLM": (True, False),
}


def _discover(config: DecoderConfig, catalog: Optional[Mapping[str, tuple]], architecture: str):
    default_norm, default_bias = ARCHITECTURE_DEFAULTS[architecture]
    if catalog is None:
        qk_norm = config.qk_normalization if config.qk_normalization is not None else default_norm
        qkv_bias = config.attention_bias if config.attention_bias is not None else default_bias
        out_bias = bool(config.attention_bias) and architecture != "Qwen2ForCausalLM"
        return qk_norm, qkv_bias, out_bias
    names = set(catalog)
    first = "layers.0.self_attn."
    has = lambda suffix: any(name.endswith(first + suffix) for name in names)
    qk_norm = has("q_norm.weight") and has("k_norm.weight")
    if config.qk_normalization is True and not qk_norm:
        raise ConfigError("qk_normalization is set but the checkpoint has no q_norm / k_norm weights")
    qkv_bias = has("q_proj.bias") or has("qkv_proj.bias") or has("query_key_value.bias")
    return qk_norm, qkv_bias, has("o_proj.bias")


def build(config_json: Mapping, catalog: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    config = DecoderConfig.from_dict(config_json)
    architecture = config.architectures[0]
    qk_norm, qkv_bias, out_bias = _discover(config, catalog, architecture)
    position = RotarySpec(head_dim=config.head_dim, rotary_dim=config.rotary_dim, theta=config.rope_theta,
                          scaling=config.rope_scaling)
    layers = []
    for index in range(config.num_hidden_layers):
        attention = SoftmaxAttentionSpec(
            hidden_size=config.hidden_size, heads=config.num_attention_heads, kv_heads=config.num_key_value_heads,
            head_dim=config.head_dim, scale=config.softmax_scale, qk_norm=qk_norm, qk_norm_eps=config.rms_norm_eps,
            qkv_bias=qkv_bias, out_bias=out_bias, window=config.layer_sliding_window(index), position=position)
        layers.append(LayerSpec(
            prefix=f"model.layers.{index}.",
            mixer=attention,
            feed_forward=SwiGluSpec(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size),
            mixer_norm=RmsNormSpec(size=config.hidden_size, eps=config.rms_norm_eps),
            feed_forward_norm=RmsNormSpec(size=config.hidden_size, eps=config.rms_norm_eps),
            names=LAYER_NAMES,
        ))
    return ModelSpec(
        architecture=architecture,
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=EmbeddingSpec("model.embed_tokens.weight", config.vocab_size, config.hidden_size,
                                config.embedding_multiplier),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(config.num_hidden_layers)),
        final_norm=RmsNormSpec(size=config.hidden_size, eps=config.rms_norm_eps),
        final_norm_name="model.norm.",
        head=HeadSpec("lm_head.weight", config.vocab_size, config.hidden_size, tied=config.tie_word_embeddings),
        strip_prefixes=STRIP_PREFIXES,
    )


for _name in ARCHITECTURE_DEFAULTS:
    register_architecture(_name, build)
