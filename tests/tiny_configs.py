"""The tiny configurations the tests use.  They differ in every size and option:
head counts and groups, head_dim tied to or free of hidden/heads, sizes that are
no power of two, layer count, vocabulary, eps, rope theta and scaling, q/k norm,
tied or untied head, page size."""

from __future__ import annotations

TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "intermediate_size": 192,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
}

TINY_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"],
    "hidden_size": 96,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 32,
    "intermediate_size": 160,
    "vocab_size": 384,
    "rope_theta": 1000000.0,
    "max_position_embeddings": 512,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
}

# A third shape for kernels and parts: sizes that are no power of two, one KV
# head (all query heads in one group), head_dim 48, biases on.
TINY_ODD = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 120,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "head_dim": 48,
    "intermediate_size": 200,
    "vocab_size": 331,
    "rope_theta": 50000.0,
    "max_position_embeddings": 640,
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "attention_bias": True,
    "hidden_act": "silu",
}

# A fourth with a head size of 64, the smallest that the TMA-fed decode attention takes
# (the others run its row-copy sibling): three query heads on one KV head, q/k norm, yarn-free
# plain rope, a width that is no multiple of the head size.
TINY_WIDE = {
    "architectures": ["Qwen3ForCausalLM"],
    "hidden_size": 88,
    "num_hidden_layers": 2,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 64,
    "intermediate_size": 136,
    "vocab_size": 203,
    "rope_theta": 20000.0,
    "max_position_embeddings": 384,
    "rms_norm_eps": 2e-5,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
}

# A fifth for yarn position scaling, written in the newer config generation (``rope_parameters``
# with theta nested in it): context stretched 4 times over an original 64 positions, with
# beta_fast/beta_slow such that the head's pairs fall into all three ranges (kept, blended,
# slowed); every query head with a KV head of its own, three layers, a tied head.
TINY_YARN = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 80,
    "num_hidden_layers": 3,
    "num_attention_heads": 4,
    "num_key_value_heads": 4,
    "head_dim": 48,
    "intermediate_size": 112,
    "vocab_size": 149,
    "rope_parameters": {
        "rope_type": "yarn",
        "rope_theta": 10000.0,
        "factor": 4.0,
        "beta_fast": 8.0,
        "beta_slow": 0.5,
        "original_max_position_embeddings": 64,
    },
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
}

TINY = {  # config, seed, page size
    "llama": (TINY_LLAMA, 0, 16), "qwen3": (TINY_QWEN3, 1, 8), "odd": (TINY_ODD, 5, 16), "wide": (TINY_WIDE, 7, 8),
    "yarn": (TINY_YARN, 9, 4),
}
