"""Configuration: typed reading of config.json keys, errors that list everything, the registry."""
import copy
import json

import pytest

from snowllm_b200.config.lfm2 import DEFAULT_ROPE_THETA, read_lfm2_config
from snowllm_b200.config.registry import architectures, read_config_json, resolve
from snowllm_b200.errors import ConfigError
from snowllm_b200.loader import build_model
from tiny_configs import ALL, TINY_A, TINY_B, TINY_DENSE


def test_reads_every_key_of_both_tiny_configs():
    a, b = read_lfm2_config(TINY_A), read_lfm2_config(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 6, 3, 16)
    assert a.layer_types == ("conv", "conv", "full_attention", "conv") and b.conv_L_cache == 4
    assert (a.norm_topk_prob, a.use_expert_bias, a.routed_scaling_factor) == (True, True, 1.0)
    assert (b.norm_topk_prob, b.use_expert_bias, b.routed_scaling_factor) == (False, False, 2.0)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert (a.norm_eps, b.norm_eps, a.rope_theta, b.rope_theta) == (1e-5, 1e-6, 1e4, 1e6)


def test_head_dim_defaults_to_hidden_over_heads_and_may_be_given():
    assert read_lfm2_config(TINY_A).head_dim == 64 // 4
    assert read_lfm2_config(ALL["tiny_c"]).head_dim == 48


def test_rope_theta_sources():
    c = dict(TINY_A)
    c.pop("rope_theta")
    assert read_lfm2_config(c).rope_theta == DEFAULT_ROPE_THETA
    c["rope_parameters"] = {"rope_theta": 123.0}
    c["rope_theta"] = 7.0
    assert read_lfm2_config(c).rope_theta == 123.0


def test_one_error_lists_all_missing_and_bad_keys():
    c = dict(TINY_A)
    for k in ("hidden_size", "norm_eps", "num_experts"):
        c.pop(k)
    c["conv_bias"] = True
    c["num_key_value_heads"] = 3
    c["layer_types"] = ["conv", "conv"]
    with pytest.raises(ConfigError) as e:
        read_lfm2_config(c)
    msg = str(e.value)
    for word in ("hidden_size", "norm_eps", "num_experts", "conv_bias", "layer_types", "no multiple"):
        assert word in msg, (word, msg)


def test_quantized_checkpoints_are_refused():
    c = dict(TINY_A, quantization_config={"bits": 4})
    with pytest.raises(ConfigError, match="quantiz"):
        read_lfm2_config(c)


def test_registry_resolves_names_and_lists_supported_on_error():
    assert {"Lfm2MoeForCausalLM", "Lfm2ForCausalLM"} <= set(architectures())
    assert resolve(["Nope", "Lfm2ForCausalLM"]).name == "Lfm2ForCausalLM"
    with pytest.raises(ConfigError, match="Lfm2MoeForCausalLM"):
        resolve(["GPT2LMHeadModel"])


def test_config_json_round_trip_and_text_config(tmp_path):
    for name, cfg in ALL.items():
        c = read_lfm2_config(copy.deepcopy(cfg))
        (tmp_path / "config.json").write_text(json.dumps(c.to_json_dict()))
        _, again, _ = read_config_json(tmp_path)
        assert again == c, name
    wrapped = {"architectures": ["Lfm2MoeForCausalLM"], "text_config": {k: v for k, v in TINY_B.items()
                                                                        if k != "architectures"}}
    (tmp_path / "config.json").write_text(json.dumps(wrapped))
    assert read_config_json(tmp_path)[1].hidden_size == 96


def test_model_spec_chooses_parts_layer_by_layer():
    m = build_model(TINY_B, "float32")
    kinds = [(type(b.mixer).__name__, type(b.ffn).__name__) for b in m.blocks]
    assert kinds == [("Attention", "SwiGLU"), ("ShortConv", "SwiGLU"), ("ShortConv", "SigmoidMoE"),
                     ("Attention", "SigmoidMoE"), ("ShortConv", "SigmoidMoE")]
    d = build_model(TINY_DENSE, "bfloat16")
    assert all(type(b.ffn).__name__ == "SwiGLU" for b in d.blocks)
    assert sorted(m.cache_specs()) == [0, 1, 2, 3, 4]


def test_unknown_part_kind_is_a_config_error():
    from snowllm_b200.parts.registry import lookup
    with pytest.raises(ConfigError, match="short_conv"):
        lookup("mixer", "mamba9")


def test_trace_spans_cost_nothing_when_off(monkeypatch):
    from snowllm_b200 import trace
    monkeypatch.setattr(trace, "_forced", False)
    a, b = trace.span("one"), trace.span("two")
    assert a is b                                          # the shared do-nothing context
    with a:
        pass
    trace.enable(True)
    try:
        with trace.span("named"):                          # an NVTX range and a record_function region; fine without a GPU
            pass
        assert trace.enabled()
    finally:
        trace.enable(False)
