"""Tiny LFM2 configurations for tests.  They differ in every size and option: layer
order, heads and groups (2, 3, 1), head size (16, 32, 48, 64, 128), taps (3, 4, 2, 5), conv bias,
rope theta, eps, tied or own head, ff auto-adjust, vocabulary and width that are no
power of two, and a sliding window in C and E."""

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "conv", "full_attention", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 2,
    "block_ff_dim": 192, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 10000.0, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 4096,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 512, "hidden_size": 192, "num_hidden_layers": 6,
    "layer_types": ["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 6, "num_key_value_heads": 2,
    "block_ff_dim": 768, "block_auto_adjust_ff_dim": True, "block_ffn_dim_multiplier": 1.0, "block_multiple_of": 64,
    "conv_L_cache": 4, "conv_bias": True, "rope_theta": 1000000.0, "norm_eps": 1e-6,
    "tie_embedding": False, "max_position_embeddings": 4096,
}

TINY_C = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 331, "hidden_size": 144, "num_hidden_layers": 5,
    "layer_types": ["sliding_attention", "conv", "full_attention", "sliding_attention", "conv"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 48,
    "block_ff_dim": 200, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 2, "conv_bias": False, "rope_theta": 50000.0, "norm_eps": 3e-6,
    "tie_embedding": True, "max_position_embeddings": 4096, "sliding_window": 24,
}

# a width that is no multiple of 8 (no 16-byte rows for the tensor-core product: the library
# product takes over), a prime vocabulary, as many kv heads as heads, head size set by its own key
TINY_D = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 257, "hidden_size": 100, "num_hidden_layers": 3,
    "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
    "block_ff_dim": 118, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 5, "conv_bias": True, "rope_theta": 10000.0, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 4096,
}

# head sizes the tensor-core attention kernels take (64 and 128), so that those kernels (tcgen05
# prompt attention, split-key decode attention on mma.sync) meet the plain implementation too:
# E has two query heads per kv head and a sliding window on one layer, F one kv head for three heads
TINY_E = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 300, "hidden_size": 96, "num_hidden_layers": 4,
    "layer_types": ["full_attention", "conv", "sliding_attention", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "block_ff_dim": 160, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 4096, "sliding_window": 40,
}

TINY_F = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 270, "hidden_size": 72, "num_hidden_layers": 3,
    "layer_types": ["conv", "full_attention", "full_attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128,
    "block_ff_dim": 136, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 4, "conv_bias": True, "rope_theta": 10000.0, "norm_eps": 2e-6,
    "tie_embedding": False, "max_position_embeddings": 4096,
}

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
