"""Tiny Qwen3 configurations for the tests.  A and B differ in every size and
option; C adds layers that see a window of keys only."""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 503, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

# Windowed layers beside full ones: two cache groups, pages of the windowed group
# come back while the request still runs.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 311, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
    "use_sliding_window": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
}

# Head size 64 and widths that are multiples of 32: in bfloat16 this one runs on the
# tensor-core attention kernels and the few-rows product, which the smaller head sizes
# above do not reach.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 416, "vocab_size": 777, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

# Head size 128, the checkpoint's own: in bfloat16 a decode step of this one runs the kernel that
# normalises and rotates the heads, stores the new key and value and attends in one, a portion of a
# prompt the tcgen05 kernel; one layer sees a window only.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 160, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 224, "vocab_size": 389, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
    "use_sliding_window": True, "sliding_window": 48,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"],
}

# Head sizes that no kernel is specialised for (80, 96 and 256: the generic attention in both
# precisions), three query heads to a key/value head, seven heads, a width that is no multiple
# of 16, a vocabulary that is a prime.
TINY_F = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 88, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 80, "intermediate_size": 136, "vocab_size": 211, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

TINY_G = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 200, "num_attention_heads": 7, "num_key_value_heads": 7,
    "head_dim": 96, "intermediate_size": 328, "vocab_size": 1031, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

TINY_H = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 256, "intermediate_size": 184, "vocab_size": 467, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
}

# Larger standard deviations than a checkpoint's, so that attention scores and
# logits are far from uniform and a wrong key or a wrong page shows in the result.
INIT = {"std": 0.08, "norm_std": 0.1}

# Bounds of the comparisons with the plain implementation.  float32: sums taken in another order;
# the worst difference seen over all cuts and configurations is 9.7e-6.  bfloat16: activations
# carry 8 bits; the bound is a fraction of the largest logit of the sequence, per configuration
# twice the worst fraction seen over all cuts (A 0.0123, B 0.0118, C 0.0084, D 0.0123, E 0.0139,
# F 0.0102, G 0.0128, H 0.0119).
F32_ATOL = 2e-5
BF16_REL = {"A": 0.025, "B": 0.024, "C": 0.017, "D": 0.025, "E": 0.028, "F": 0.021, "G": 0.026, "H": 0.024}
