"""Tiny configurations of the dense SwiGLU decoder for the tests.  They differ in every size and
option: head counts and groups, head size, sizes that are no power of two, layers, vocabulary, eps,
rope theta and scaling, partial rotation, q/k-norm, biases, tied head, window, scale factors."""

TINY_A = {   # Llama style: untied head, no q/k-norm, head_dim = hidden / heads
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 172, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
    "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "tie_word_embeddings": False, "hidden_act": "silu",
}

TINY_B = {   # Qwen3 style: explicit head_dim (heads * head_dim != hidden), one KV head, q/k-norm, tied
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "hidden_act": "silu",
}

TINY_C = {   # everything else: llama3 rope scaling, biases, window on some layers, partial rotation,
             # attention scale and embedding multiplier, head_dim 48, odd sizes, longer context
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 120, "intermediate_size": 200, "num_hidden_layers": 4,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "vocab_size": 515,
    "max_position_embeddings": 1024, "rms_norm_eps": 3e-6, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "partial_rotary_factor": 0.5, "attention_bias": True, "attention_scale": 0.17, "embedding_multiplier": 1.5,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
    "sliding_window": 40, "tie_word_embeddings": False, "hidden_act": "silu",
}

TINY_D = {   # Qwen2 style: q/k/v bias without output bias, MHA (groups of one), head_dim 16
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 80, "intermediate_size": 144, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 5, "vocab_size": 300,
    "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "hidden_act": "silu",
}

TINY_E = {   # head_dim 128: in bfloat16 the tcgen05 prompt and decode kernels; one sliding layer
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "hidden_size": 256, "intermediate_size": 352, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 640,
    "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "layer_types": ["sliding_attention", "full_attention"], "sliding_window": 200,
    "tie_word_embeddings": True, "hidden_act": "silu",
}

TINY_F = {   # head_dim 64: in bfloat16 the mma.sync prompt and decode kernels; groups of three, pages of 8, a window
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 192, "intermediate_size": 272, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 410,
    "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"], "sliding_window": 100,
    "tie_word_embeddings": False, "hidden_act": "silu",
}

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
# page sizes the replay tests give each configuration
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 16, "E": 16, "F": 8}
