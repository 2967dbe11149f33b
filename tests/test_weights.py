"""Weights by tensor name: dtypes kept, one error for everything wrong, random-weights mode."""
import json

import pytest
import torch

import plain_lfm2 as plain
from snowllm_b200.errors import WeightError
from snowllm_b200.loader import build_model
from snowllm_b200.weights import (Checkpoint, load_folder, random_tensors, write_model_folder,
                                  write_safetensors)
from tiny_configs import TINY_A, TINY_B


def _folder(tmp_path, cfg, dtype=torch.bfloat16, **kw):
    m = build_model(cfg, "bfloat16")
    t = random_tensors(m, 3, dtype, **kw)
    write_model_folder(tmp_path, m.config.to_json_dict(), t)
    return t


def test_folder_round_trip_matches_the_independent_parser(tmp_path):
    t = _folder(tmp_path, TINY_A)
    other = plain.read_safetensors(tmp_path / "model.safetensors")
    assert set(other) == set(t)
    ck = Checkpoint(tmp_path)
    for k, v in t.items():
        assert torch.equal(other[k], v) and torch.equal(ck.read(k), v), k
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["Lfm2MoeForCausalLM"]


def test_same_seed_same_weights_other_seed_other_weights():
    m = build_model(TINY_A, "bfloat16")
    a, b, c = (random_tensors(m, s, torch.bfloat16) for s in (5, 5, 6))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    norm = a["model.layers.0.operator_norm.weight"]
    assert torch.all(norm == 1)
    assert abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    assert abs(float(a["model.layers.0.conv.conv.weight"].float().std()) - 0.1) < 0.02


def test_kept_dtypes(tmp_path):
    _folder(tmp_path, TINY_A)
    m = build_model(tmp_path, "bfloat16")
    load_folder(m, tmp_path, "cpu")
    moe = m.blocks[1].ffn
    assert moe.bias.dtype == torch.float32                  # stored in 32-bit: stays so
    assert moe.w13.dtype == torch.bfloat16 and moe.w13.shape == (8, 64, 64)
    assert m.blocks[2].mixer.wqkv.shape == ((4 + 2 * 2) * 16, 64)
    assert m.head.weight is m.embedding.weight              # tied
    m32 = build_model(tmp_path, "float32")
    load_folder(m32, tmp_path, "cpu")
    assert m32.blocks[0].mixer.in_proj.dtype == torch.float32


def test_float32_norm_weights_stay_float32_in_a_bfloat16_model(tmp_path):
    t = _folder(tmp_path, TINY_B, torch.float32)
    m = build_model(tmp_path, "bfloat16")
    load_folder(m, tmp_path, "cpu")
    assert m.blocks[0].mixer_norm.weight.dtype == torch.float32
    assert m.blocks[0].mixer.wqkv.dtype == torch.bfloat16
    assert m.blocks[1].mixer.conv.dtype == torch.float32
    assert m.head.weight is not m.embedding.weight and m.head.weight.shape == (384, 96)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    t = _folder(tmp_path, TINY_A)
    t.pop("model.layers.2.self_attn.q_layernorm.weight")
    t.pop("model.embedding_norm.weight")
    t["model.layers.9.bogus.weight"] = torch.zeros(3)
    t["model.layers.0.conv.in_proj.weight"] = torch.zeros(10, 64, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", t)
    m = build_model(tmp_path, "bfloat16")
    with pytest.raises(WeightError) as e:
        load_folder(m, tmp_path, "cpu")
    msg = str(e.value)
    for word in ("missing tensors", "q_layernorm", "embedding_norm", "unexpected tensors", "bogus",
                 "wrong shapes", "conv.in_proj", "(10, 64)"):
        assert word in msg, (word, msg)


def test_fused_expert_tensors_are_accepted(tmp_path):
    t = _folder(tmp_path, TINY_A)
    fused = dict(t)
    for layer in (1, 2, 3):
        p = f"model.layers.{layer}.feed_forward.experts."
        gate = torch.stack([fused.pop(f"{p}{e}.w1.weight") for e in range(8)])
        up = torch.stack([fused.pop(f"{p}{e}.w3.weight") for e in range(8)])
        fused[p + "gate_up_proj"] = torch.cat((gate, up), 1)
        fused[p + "down_proj"] = torch.stack([fused.pop(f"{p}{e}.w2.weight") for e in range(8)])
    a = build_model(tmp_path, "bfloat16")
    load_folder(a, tmp_path, "cpu")
    write_safetensors(tmp_path / "model.safetensors", fused)
    b = build_model(tmp_path, "bfloat16")
    load_folder(b, tmp_path, "cpu")
    assert torch.equal(a.blocks[2].ffn.w13, b.blocks[2].ffn.w13)
    assert torch.equal(a.blocks[3].ffn.w2, b.blocks[3].ffn.w2)


def test_missing_file_and_bad_header(tmp_path):
    with pytest.raises(WeightError, match="no .safetensors"):
        Checkpoint(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00\x00\x00\x00\x00\x00\x00{bad}")
    with pytest.raises(WeightError, match="header"):
        Checkpoint(tmp_path)


def test_weight_bytes_a_step_reads_come_from_what_parts_declared():
    """Every declared tensor once, in the dtype it is kept in; of routed experts the picked share; a tied
    head reads the embedding table; a layer that the run list names twice is read twice."""
    import torch

    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import load_tensors, random_tensors
    from tiny_configs import TINY_A, TINY_B
    for cfg in (TINY_A, TINY_B):
        model = build_model(cfg, "bfloat16")
        tensors = random_tensors(model, 0, torch.bfloat16)
        load_tensors(model, tensors, "cpu")
        kept = {n: (4 if n.endswith("expert_bias") else 2) * t.numel() for n, t in tensors.items()}
        if not cfg["tie_word_embeddings"]:             # the table is then only gathered from: a row per token
            del kept["model.embed_tokens.weight"]
        assert model.weight_bytes_per_step() == sum(kept.values())
        moe_entries = [i for i, e in enumerate(model.run) if hasattr(model.blocks[e.layer].ffn, "route")]
        E = cfg["num_experts"]
        experts = {i: sum(v for n, v in kept.items() if f"layers.{model.run[i].layer}.feed_forward.experts." in n)
                   for i in moe_entries}
        picked = {i: 1 + i % 3 for i in moe_entries}
        want = sum(kept.values()) - sum(experts[i] - experts[i] * picked[i] // E for i in moe_entries)
        assert abs(model.weight_bytes_per_step(picked) - want) <= len(moe_entries)
    from snowllm_b200.parts.spec import RunEntry
    model.run = list(model.run) + [RunEntry(1)]
    twice = sum(v for n, v in kept.items() if ".layers.1." in n)
    assert model.weight_bytes_per_step() == sum(kept.values()) + twice
