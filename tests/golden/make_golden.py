"""Writes tests/golden/plain_tiny.pt: logits of the plain implementation (tests/plain_lfm2.py) on two tiny
random models, as a guard against accidental edits of the oracle.

    python tests/golden/make_golden.py

The plain implementation rests on SnowLLM's formulas alone (its model code cannot be imported on a CPU:
its modules load a closed HIP kernel library at import), so these are its own outputs, not SnowLLM's.
The weights come from a seeded torch.Generator written out here, not from the engine's random-weights mode.
"""
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_lfm2 as plain  # noqa: E402
from tiny_configs import TINY_A, TINY_B  # noqa: E402


def tensors_for(cfg, seed):
    """Every tensor of the checkpoint layout, N(0, 1/sqrt(fan_in)) matrices, norm weights 1 +- 0.1."""
    g = torch.Generator().manual_seed(seed)
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // nh
    mat = lambda n, k: torch.randn(n, k, generator=g) * k ** -0.5
    norm = lambda n: 1 + 0.1 * torch.randn(n, generator=g)
    t = {"model.embed_tokens.weight": torch.randn(V, H, generator=g), "model.embedding_norm.weight": norm(H)}
    if not cfg["tie_word_embeddings"]:
        t["lm_head.weight"] = mat(V, H)
    for i, kind in enumerate(cfg["layer_types"]):
        p = f"model.layers.{i}."
        t[p + "operator_norm.weight"], t[p + "ffn_norm.weight"] = norm(H), norm(H)
        if kind == "conv":
            L = cfg["conv_L_cache"]
            t[p + "conv.in_proj.weight"], t[p + "conv.out_proj.weight"] = mat(3 * H, H), mat(H, H)
            t[p + "conv.conv.weight"] = torch.randn(H, 1, L, generator=g) * 0.5
        else:
            a = p + "self_attn."
            t[a + "q_proj.weight"], t[a + "k_proj.weight"] = mat(nh * hd, H), mat(nkv * hd, H)
            t[a + "v_proj.weight"], t[a + "out_proj.weight"] = mat(nkv * hd, H), mat(H, nh * hd)
            t[a + "q_layernorm.weight"], t[a + "k_layernorm.weight"] = norm(hd), norm(hd)
        f = p + "feed_forward."
        if i < cfg["num_dense_layers"]:
            I = cfg["intermediate_size"]
            t[f + "w1.weight"], t[f + "w3.weight"], t[f + "w2.weight"] = mat(I, H), mat(I, H), mat(H, I)
        else:
            E, I = cfg["num_experts"], cfg["moe_intermediate_size"]
            t[f + "gate.weight"] = mat(E, H)
            if cfg["use_expert_bias"]:
                t[f + "expert_bias"] = 0.1 * torch.randn(E, generator=g)
            for e in range(E):
                q = f"{f}experts.{e}."
                t[q + "w1.weight"], t[q + "w3.weight"], t[q + "w2.weight"] = mat(I, H), mat(I, H), mat(H, I)
    return t


def cases():
    out = {}
    for name, cfg, seed in (("tiny_a", TINY_A, 11), ("tiny_b", TINY_B, 12)):
        g = torch.Generator().manual_seed(seed + 100)
        ids = torch.randint(0, cfg["vocab_size"], (19,), generator=g).tolist()
        out[name] = {"ids": ids, "logits": plain.logits(cfg, tensors_for(cfg, seed), ids)}
    return out


if __name__ == "__main__":
    torch.save(cases(), HERE / "plain_tiny.pt")
    print("wrote", HERE / "plain_tiny.pt")
