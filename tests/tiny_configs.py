"""Small LFM2.5 configurations for the tests: they differ from one another in every size and option."""
from __future__ import annotations

TINY_A = {   # conv, conv, attention, conv; tied embeddings; expert bias; renormalised top-2
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "conv", "full_attention", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "conv_L_cache": 3, "conv_bias": False,
    "num_dense_layers": 1, "intermediate_size": 128,
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 32,
    "norm_topk_prob": True, "use_expert_bias": True, "routed_scaling_factor": 1.0,
    "rope_theta": 10000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}

TINY_B = {   # attention first; widths that are no power of two; untied head; scaled top-4, no bias
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 384, "hidden_size": 96, "num_hidden_layers": 5,
    "layer_types": ["full_attention", "conv", "conv", "full_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 3, "conv_L_cache": 4, "conv_bias": False,
    "num_dense_layers": 2, "intermediate_size": 256,
    "num_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 48,
    "norm_topk_prob": False, "use_expert_bias": False, "routed_scaling_factor": 2.0,
    "rope_theta": 1000000.0, "norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}

TINY_C = {   # other head size (48, explicit), one kv head per q head pair of three, odd vocabulary
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 331, "hidden_size": 80, "num_hidden_layers": 3,
    "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 48, "conv_L_cache": 2,
    "conv_bias": False, "num_dense_layers": 0, "intermediate_size": 64,
    "num_experts": 5, "num_experts_per_tok": 3, "moe_intermediate_size": 24,
    "norm_topk_prob": True, "use_expert_bias": True, "routed_scaling_factor": 0.5,
    "rope_theta": 500.0, "norm_eps": 1e-4, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}

TINY_DENSE = {   # the dense architecture: every feed-forward a SwiGLU
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 200, "hidden_size": 48, "num_hidden_layers": 3,
    "layer_types": ["conv", "full_attention", "conv"],
    "num_attention_heads": 3, "num_key_value_heads": 3, "conv_L_cache": 3, "conv_bias": False,
    "intermediate_size": 112, "rope_theta": 10000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}

TINY_E = {   # head size 64 (the tensor-core attention kernels), one kv head for two q heads, top-1 routing
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 300, "hidden_size": 128, "num_hidden_layers": 3,
    "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 2, "num_key_value_heads": 1, "conv_L_cache": 3, "conv_bias": False,
    "num_dense_layers": 1, "intermediate_size": 192,
    "num_experts": 4, "num_experts_per_tok": 1, "moe_intermediate_size": 64,
    "norm_topk_prob": False, "use_expert_bias": True, "routed_scaling_factor": 1.0,
    "rope_theta": 10000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}

TINY_F = {   # head size 128 (two 64-element panels in the tensor-core attention kernels), three q heads on one kv head
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 272, "hidden_size": 192, "num_hidden_layers": 3,
    "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128, "conv_L_cache": 4, "conv_bias": False,
    "num_dense_layers": 1, "intermediate_size": 160,
    "num_experts": 6, "num_experts_per_tok": 2, "moe_intermediate_size": 40,
    "norm_topk_prob": True, "use_expert_bias": False, "routed_scaling_factor": 1.0,
    "rope_theta": 50000.0, "norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}

TINY_CONV_ONLY = dict(TINY_DENSE, layer_types=["conv", "conv", "conv"], conv_L_cache=5)   # no paged cache at all
TINY_ATTN_ONLY = dict(TINY_A, layer_types=["full_attention"] * 4, num_dense_layers=0,    # no state slots in use
                      hidden_size=104, num_attention_heads=1, num_key_value_heads=1, head_dim=24,
                      moe_intermediate_size=20, vocab_size=250)

ALL = {"tiny_conv_only": TINY_CONV_ONLY, "tiny_attn_only": TINY_ATTN_ONLY, "tiny_e": TINY_E, "tiny_f": TINY_F, "tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_dense": TINY_DENSE}
