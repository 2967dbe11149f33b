"""LFM2 / LFM2.5 as data: configuration -> ModelSpec.

The hybrid stack follows snowllm/models/lfm2/weights.py:58-96 (tensor names, which layer
gets which operator and which feed-forward) and snowllm/models/lfm2/layers.py:91-131 (the
pre-norm layer and the final norm).  This file only names parts and passes them their
constants; the parts themselves know nothing of LFM2.
"""
from __future__ import annotations

from ..config.lfm2 import DENSE_ARCHITECTURE, MOE_ARCHITECTURE, Lfm2Config, read_lfm2_config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def lfm2_model_spec(c: Lfm2Config) -> ModelSpec:
    H = c.hidden_size
    rope = dict(kind="rope", head_dim=c.head_dim, theta=c.rope_theta)
    layers = []
    for i, kind in enumerate(c.layer_types):
        p = f"model.layers.{i}."
        if kind == "conv":
            mixer = PartSpec("short_conv", dict(hidden_size=H, kernel_size=c.conv_L_cache),
                             dict(in_proj=p + "conv.in_proj.weight", conv=p + "conv.conv.weight",
                                  out_proj=p + "conv.out_proj.weight"))
        else:
            a = p + "self_attn."
            mixer = PartSpec("attention",
                             dict(hidden_size=H, num_heads=c.num_attention_heads,
                                  num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim,
                                  qk_norm_eps=c.norm_eps, position=rope, window=None),
                             dict(q_proj=a + "q_proj.weight", k_proj=a + "k_proj.weight",
                                  v_proj=a + "v_proj.weight", out_proj=a + "out_proj.weight",
                                  q_norm=a + "q_layernorm.weight", k_norm=a + "k_layernorm.weight"))
        f = p + "feed_forward."
        if i < c.num_dense_layers:
            ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.intermediate_size),
                           dict(gate=f + "w1.weight", up=f + "w3.weight", down=f + "w2.weight"))
        else:
            ffn = PartSpec("sigmoid_moe",
                           dict(hidden_size=H, intermediate_size=c.moe_intermediate_size,
                                num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                norm_topk_prob=c.norm_topk_prob, use_expert_bias=c.use_expert_bias,
                                routed_scaling_factor=c.routed_scaling_factor),
                           dict(router=f + "gate.weight", expert_bias=f + "expert_bias",
                                experts=f + "experts.", expert_gate="w1.weight",
                                expert_up="w3.weight", expert_down="w2.weight",
                                fused_gate_up=f + "experts.gate_up_proj",
                                fused_down=f + "experts.down_proj"))
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=c.norm_eps), dict(weight=p + name))
        layers.append(LayerSpec("prenorm", mixer, ffn, norm("operator_norm.weight"),
                                norm("ffn_norm.weight")))
    embedding = PartSpec("embedding", dict(vocab_size=c.vocab_size, hidden_size=H),
                         dict(weight="model.embed_tokens.weight"))
    head_name = "model.embed_tokens.weight" if c.tie_word_embeddings else "lm_head.weight"
    head = PartSpec("linear_head", dict(vocab_size=c.vocab_size, hidden_size=H,
                                        tied=c.tie_word_embeddings), dict(weight=head_name))
    final_norm = PartSpec("rmsnorm", dict(size=H, eps=c.norm_eps),
                          dict(weight="model.embedding_norm.weight"))
    return ModelSpec(architecture=c.architecture, vocab_size=c.vocab_size, hidden_size=H,
                     embedding=embedding, layers=layers,
                     run=[RunEntry(i) for i in range(len(layers))],
                     final_norm=final_norm, head=head, max_position=c.max_position_embeddings)


register_architecture(MOE_ARCHITECTURE, read_lfm2_config, lfm2_model_spec)
register_architecture(DENSE_ARCHITECTURE, read_lfm2_config, lfm2_model_spec)
