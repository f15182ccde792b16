"""Configuration reading, the registry, and the model description built from config.json (no GPU)."""

import copy

import pytest

from libmir_b200 import ConfigError, RegistryError, build_spec, known_architectures
from libmir_b200.config import DecoderConfig, GenerationConfig, GenerationOverrides, RuntimeConfig
from libmir_b200.config.spec import PagedKv
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C, TINY_D


def test_tiny_configs_parse_and_differ_in_every_size():
    parsed = {name: DecoderConfig.from_dict(cfg) for name, cfg in ALL.items()}
    a, b = parsed["A"], parsed["B"]
    for field in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings", "rms_norm_eps",
                  "rope_theta", "tie_word_embeddings"):
        assert getattr(a, field) != getattr(b, field), field
    assert a.head_dim == 16 and b.head_dim == 32 and b.head_dim * b.num_attention_heads != b.hidden_size
    c = parsed["C"]
    assert c.rope_scaling.factor == 8.0 and c.rotary_dim == 24 and c.softmax_scale == 0.17
    assert [c.layer_sliding_window(i) for i in range(4)] == [None, 40, None, 40]


def test_defaults_and_aliases():
    config = DecoderConfig.from_dict({"architectures": ["LlamaForCausalLM"], "n_embd": 32, "n_head": 4, "n_layer": 1,
                                      "n_inner": 64, "vocab_size": 10, "layer_norm_epsilon": 1e-4,
                                      "rotary_emb_base": 123.0, "n_positions": 77, "n_kv_heads": None})
    assert (config.hidden_size, config.num_attention_heads, config.num_hidden_layers) == (32, 4, 1)
    assert config.num_key_value_heads == 4 and config.head_dim == 8
    assert config.rms_norm_eps == 1e-4 and config.rope_theta == 123.0 and config.max_position_embeddings == 77
    minimal = DecoderConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 32,
                                       "num_attention_heads": 4, "num_hidden_layers": 1, "intermediate_size": 64,
                                       "vocab_size": 10})
    assert minimal.rms_norm_eps == 1e-5 and minimal.rope_theta == 10000.0
    assert minimal.max_position_embeddings == 4096 and minimal.tie_word_embeddings is False


def test_nested_text_config_and_rope_parameters():
    config = DecoderConfig.from_dict({"architectures": ["Qwen3ForCausalLM"], "tie_word_embeddings": True,
                                      "text_config": {"hidden_size": 32, "num_attention_heads": 4,
                                                      "num_hidden_layers": 1, "intermediate_size": 64,
                                                      "vocab_size": 10,
                                                      "rope_parameters": {"rope_theta": 5e5,
                                                                          "partial_rotary_factor": 0.5}}})
    assert config.rope_theta == 5e5 and config.partial_rotary_factor == 0.5 and config.tie_word_embeddings


@pytest.mark.parametrize("mutation, message", [
    (lambda c: c.pop("hidden_size"), "missing hidden_size or n_embd"),
    (lambda c: c.pop("vocab_size"), "missing vocab_size"),
    (lambda c: c.update(num_attention_heads="4"), "num_attention_heads must be an unsigned integer"),
    (lambda c: c.update(num_attention_heads=0), "num_attention_heads must be greater than zero"),
    (lambda c: c.update(num_key_value_heads=3), "divisible by num_key_value_heads"),
    (lambda c: c.update(rms_norm_eps="x"), "rms_norm_eps must be a number"),
    (lambda c: c.update(tie_word_embeddings=1), "tie_word_embeddings must be a boolean"),
    (lambda c: c.update(hidden_act="gelu"), "hidden_act gelu is not supported"),
    (lambda c: c.update(num_experts=8), "routed experts"),
    (lambda c: c.update(num_kv_shared_layers=2), "shared K/V layers are not supported"),
    (lambda c: c.update(rope_scaling={"rope_type": "yarn", "factor": 2.0}), "unsupported rope_scaling type yarn"),
    (lambda c: c.update(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 4.0,
                                      "high_freq_factor": 1.0, "original_max_position_embeddings": 8192}),
     "invalid piecewise rope_scaling parameters"),
    (lambda c: c.update(layer_types=["full_attention"]), "layer_types has 1 entries, expected 2"),
    (lambda c: c.update(layer_types=["full_attention", "linear_attention"]), "unsupported layer_type"),
    (lambda c: c.update(layer_types=["full_attention", "sliding_attention"]), "sliding_window is missing"),
    (lambda c: c.update(sliding_window=0), "sliding_window must be greater than zero"),
    (lambda c: c.update(attention_scale=-1.0), "attention_scale must be finite and greater than zero"),
    (lambda c: c.update(hidden_size=66, head_dim=None), "hidden_size must be divisible by num_attention_heads"),
])
def test_config_errors(mutation, message):
    config = copy.deepcopy(TINY_A)
    mutation(config)
    with pytest.raises(ConfigError, match=message):
        DecoderConfig.from_dict(config)


def test_registry_names_and_unknown_architecture():
    assert {"LlamaForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM"} <= set(known_architectures())
    config = dict(TINY_A, architectures=["GPT2LMHeadModel"])
    with pytest.raises(RegistryError, match="unknown architecture 'GPT2LMHeadModel'; known: .*LlamaForCausalLM"):
        build_spec(config)
    with pytest.raises(ConfigError, match="architectures"):
        build_spec({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_spec_is_built_layer_by_layer_from_the_configuration():
    spec = build_spec(TINY_C)
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    windows = [layer.mixer.window for layer in spec.layers]
    assert windows == [None, 40, None, 40]
    mixer = spec.layers[0].mixer
    assert (mixer.heads, mixer.kv_heads, mixer.head_dim, mixer.scale) == (6, 3, 48, 0.17)
    assert mixer.qkv_bias and mixer.out_bias and not mixer.qk_norm
    assert mixer.position.rotary_dim == 24 and mixer.position.scaling.original_max_position_embeddings == 32
    assert spec.layers[0].mixer_norm.eps == 3e-6 and spec.final_norm.eps == 3e-6
    assert spec.embedding.multiplier == 1.5 and not spec.head.tied
    qwen3 = build_spec(TINY_B)
    assert qwen3.layers[0].mixer.qk_norm and qwen3.head.tied and not qwen3.layers[0].mixer.qkv_bias
    qwen2 = build_spec(TINY_D)
    assert qwen2.layers[0].mixer.qkv_bias and not qwen2.layers[0].mixer.out_bias


def test_options_are_discovered_from_the_checkpoints_tensors():
    names = {"model.layers.0.self_attn.q_norm.weight": (16,), "model.layers.0.self_attn.k_norm.weight": (16,),
             "model.layers.0.self_attn.q_proj.bias": (64,)}
    spec = build_spec(TINY_A, names)
    assert spec.layers[0].mixer.qk_norm and spec.layers[0].mixer.qkv_bias and not spec.layers[0].mixer.out_bias
    assert not build_spec(TINY_B, {}).layers[0].mixer.qk_norm      # a checkpoint without the weights: off


def test_config_round_trip():
    for config in ALL.values():
        parsed = DecoderConfig.from_dict(config)
        assert DecoderConfig.from_dict(parsed.to_dict()) == parsed


def test_generation_config_resolution():
    generation = GenerationConfig.from_dict({"max_new_tokens": 7, "temperature": 0.6, "top_k": 20, "top_p": 0.9,
                                             "do_sample": True, "eos_token_id": [3, 5]})
    settings = generation.resolve(GenerationOverrides(max_tokens=3))
    assert (settings.max_tokens, settings.temperature, settings.top_k, settings.top_p) == (3, 0.6, 20, 0.9)
    assert settings.stop_token_ids == (3, 5) and not settings.greedy
    assert GenerationConfig.from_dict({"do_sample": False, "temperature": 0.6}).resolve().temperature == 0.0
    assert GenerationConfig.from_dict({"do_sample": True}).resolve().temperature == 1.0
    assert GenerationConfig().resolve().greedy and GenerationConfig().resolve().max_tokens == 2048
    with pytest.raises(ConfigError, match="top_p must be in"):
        GenerationConfig().resolve(GenerationOverrides(top_p=0.0))
    with pytest.raises(ConfigError, match="min_tokens cannot exceed max_tokens"):
        GenerationConfig().resolve(GenerationOverrides(max_tokens=2, min_tokens=3))


def test_runtime_config_validation():
    RuntimeConfig().validate()
    with pytest.raises(ConfigError, match="dtype must be one of"):
        RuntimeConfig(dtype="float16").validate()


def test_cache_plan_groups_layers_by_their_needs():
    import torch
    from libmir_b200.cache import CacheManager
    from libmir_b200.models.decoder import DecoderModel
    from libmir_b200.parts.base import BuildEnv
    model = DecoderModel(build_spec(TINY_C), BuildEnv(torch.float32, torch.device("meta")))
    manager = CacheManager(model.cache_plan(), 16, 8, 4)
    assert [(g.requirement, g.entries) for g in manager.groups] == [
        (PagedKv(3, 48, None), [0, 2]), (PagedKv(3, 48, 40), [1, 3])]
