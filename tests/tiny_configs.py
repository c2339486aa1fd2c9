"""Tiny Hunyuan Dense configurations for tests.  A and B differ in every size
and option; C adds what neither has (biases, cross-layer cache sharing, a head
size that is no power of two).  Weights are drawn wider than a trained model's
initialisation (std 0.08, not 0.02) so that attention and feed-forward move the
logits enough for a fault in them to show."""

A = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "hidden_act": "silu",
    "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "use_qk_norm": True, "tie_word_embeddings": True, "attention_bias": False,
}

B = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 384, "hidden_size": 160, "intermediate_size": 352, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "hidden_act": "silu",
    "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "rope_scaling": {"alpha": 1000.0, "type": "dynamic"},
    "use_qk_norm": False, "tie_word_embeddings": False, "attention_bias": False,
}

C = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 301, "hidden_size": 96, "intermediate_size": 200, "num_hidden_layers": 4,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "hidden_act": "silu",
    "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 50000.0,
    "rope_scaling": {"alpha": 4.0},
    "use_qk_norm": True, "tie_word_embeddings": False, "attention_bias": True,
    "use_cla": True, "cla_share_factor": 2,
}

# head sizes between the powers of two: 80 (five 16-wide steps of the MMA), and 192
D80 = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 211, "hidden_size": 144, "intermediate_size": 272, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 80, "hidden_act": "silu",
    "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "use_qk_norm": True, "tie_word_embeddings": True, "attention_bias": False,
}
D192 = dict(D80, head_dim=192, num_attention_heads=3, num_key_value_heads=1, use_qk_norm=False)
# a head size for which no tensor-core attention is built: the bfloat16 path takes the plain kernel
D144 = dict(D80, head_dim=144, num_attention_heads=2, num_key_value_heads=1)


def _layer_sizes(hidden, heads, kv_heads, inter, layers, tied, vocab=1000):
    """One or two layers with the layer sizes of a Hunyuan model (a small vocabulary keeps the
    folder small): the sizes at which the serving kernels' tensor-core paths are taken."""
    return {
        "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
        "vocab_size": vocab, "hidden_size": hidden, "intermediate_size": inter,
        "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "head_dim": 128, "hidden_act": "silu", "max_position_embeddings": 2048, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "rope_scaling": {"alpha": 1000.0, "type": "dynamic"},
        "use_qk_norm": True, "tie_word_embeddings": tied, "attention_bias": False,
    }


S18 = _layer_sizes(2048, 16, 4, 6144, 2, True)        # Hunyuan-1.8B layer sizes
S4 = _layer_sizes(3072, 32, 8, 8192, 1, True)         # Hunyuan-4B layer sizes
S7 = _layer_sizes(4096, 32, 8, 14336, 1, False, 1003)  # Hunyuan-7B layer sizes, untied head

TINY = {
    "A": {"config": A, "seed": 0, "std": 0.08, "norm_std": 0.05, "page_size": 64},
    "B": {"config": B, "seed": 1, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "C": {"config": C, "seed": 2, "std": 0.08, "norm_std": 0.05, "page_size": 32},
    "D80": {"config": D80, "seed": 6, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "D192": {"config": D192, "seed": 7, "std": 0.08, "norm_std": 0.05, "page_size": 32},
    "D144": {"config": D144, "seed": 8, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "S18": {"config": S18, "seed": 3, "std": 0.02, "norm_std": 0.05, "page_size": 64},
    "S4": {"config": S4, "seed": 4, "std": 0.02, "norm_std": 0.05, "page_size": 16},
    "S7": {"config": S7, "seed": 5, "std": 0.015, "norm_std": 0.05, "page_size": 128},
}
