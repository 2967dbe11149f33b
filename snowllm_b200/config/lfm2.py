"""Typed configuration of LFM2 / LFM2.5, read from the architecture's own config.json keys.

Keys and their meaning follow snowllm/models/lfm2/weights.py:15-45 (which pins each of them
to the 8B-A1B geometry; here every size is free) and snowllm/context.py:27
(max_position_embeddings).  No size stands in code: what config.json does not give and
has no documented default is an error.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any

from ..errors import ConfigError

LAYER_TYPES = ("conv", "full_attention")
MOE_ARCHITECTURE = "Lfm2MoeForCausalLM"
DENSE_ARCHITECTURE = "Lfm2ForCausalLM"
DEFAULT_ROPE_THETA = 5000000.0          # snowllm/models/lfm2/weights.py:44
DEFAULT_MAX_POSITION = 262144           # snowllm/context.py:27


@dataclass(frozen=True)
class Lfm2Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    layer_types: tuple[str, ...]
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    conv_L_cache: int
    norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    intermediate_size: int
    num_dense_layers: int
    # routed experts (absent in the dense architecture)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = False
    use_expert_bias: bool = False
    routed_scaling_factor: float = 1.0

    @property
    def is_moe(self) -> bool:
        return self.num_dense_layers < self.num_hidden_layers

    def to_json_dict(self) -> dict[str, Any]:
        """config.json content that reads back to this configuration."""
        d = asdict(self)
        arch = d.pop("architecture")
        d["layer_types"] = list(self.layer_types)
        d["architectures"] = [arch]
        d["model_type"] = "lfm2_moe" if arch == MOE_ARCHITECTURE else "lfm2"
        d["conv_bias"] = False
        if arch == DENSE_ARCHITECTURE:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                      "use_expert_bias", "routed_scaling_factor", "num_dense_layers"):
                d.pop(k)
        return d


def _positive_int(cfg, key, bad, missing, default=None):
    if key not in cfg or cfg[key] is None:
        if default is not None:
            return default
        missing.append(key)
        return 0
    v = cfg[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        bad.append(f"{key}={v!r} (want a positive integer)")
        return 0
    return v


def read_lfm2_config(cfg: dict) -> Lfm2Config:
    """Build the typed configuration; one error lists every missing or unusable key."""
    arch = (cfg.get("architectures") or [MOE_ARCHITECTURE])[0]
    moe = arch == MOE_ARCHITECTURE
    missing: list[str] = []
    bad: list[str] = []
    I = lambda k, default=None: _positive_int(cfg, k, bad, missing, default)

    hidden, vocab, layers = I("hidden_size"), I("vocab_size"), I("num_hidden_layers")
    heads, kv_heads = I("num_attention_heads"), I("num_key_value_heads")
    conv_l, inter = I("conv_L_cache"), I("intermediate_size")
    head_dim = I("head_dim", default=(hidden // heads if heads else 0) or None) if heads else 0

    if "norm_eps" not in cfg:
        missing.append("norm_eps")
    eps = cfg.get("norm_eps", 0.0)
    if not isinstance(eps, (int, float)) or isinstance(eps, bool) or (("norm_eps" in cfg) and eps <= 0):
        bad.append(f"norm_eps={eps!r} (want a positive number)")

    types = cfg.get("layer_types")
    if types is None:
        missing.append("layer_types")
        types = []
    elif len(types) != layers or any(t not in LAYER_TYPES for t in types):
        bad.append(f"layer_types must name each of the {layers} layers as one of {LAYER_TYPES}")

    theta = (cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta", DEFAULT_ROPE_THETA))
    if not isinstance(theta, (int, float)) or isinstance(theta, bool) or theta <= 0:
        bad.append(f"rope_theta={theta!r} (want a positive number)")

    if cfg.get("conv_bias", False):
        bad.append("conv_bias=True (the short convolution has no bias path)")
    if cfg.get("quantization_config"):
        bad.append("quantization_config is set (quantized weights are not supported)")
    if cfg.get("block_auto_adjust_ff_dim"):
        bad.append("block_auto_adjust_ff_dim=True (give the feed-forward width as intermediate_size)")
    if heads and kv_heads and heads % kv_heads:
        bad.append(f"num_attention_heads={heads} is no multiple of num_key_value_heads={kv_heads}")
    if head_dim and head_dim % 2:
        bad.append(f"head_dim={head_dim} (rotary halves need an even size)")

    kw: dict[str, Any] = {}
    if moe:
        dense = cfg.get("num_dense_layers")
        if dense is None:
            missing.append("num_dense_layers")
            dense = 0
        elif isinstance(dense, bool) or not isinstance(dense, int) or dense < 0 or dense > layers:
            bad.append(f"num_dense_layers={dense!r} (want 0..{layers})")
            dense = 0
        if dense < layers:
            kw = dict(num_experts=I("num_experts"), num_experts_per_tok=I("num_experts_per_tok"),
                      moe_intermediate_size=I("moe_intermediate_size"),
                      norm_topk_prob=bool(cfg.get("norm_topk_prob", False)),
                      use_expert_bias=bool(cfg.get("use_expert_bias", False)),
                      routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0)))
            if kw["num_experts"] and kw["num_experts_per_tok"] > kw["num_experts"]:
                bad.append(f"num_experts_per_tok={kw['num_experts_per_tok']} exceeds "
                           f"num_experts={kw['num_experts']}")
    else:
        dense = layers

    if missing or bad:
        parts = []
        if missing:
            parts.append("missing keys: " + ", ".join(missing))
        if bad:
            parts.append("unusable values: " + "; ".join(bad))
        raise ConfigError(f"unsupported {arch} configuration: " + " | ".join(parts))

    return Lfm2Config(
        architecture=arch, vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
        layer_types=tuple(types), num_attention_heads=heads, num_key_value_heads=kv_heads,
        head_dim=head_dim, conv_L_cache=conv_l, norm_eps=float(eps), rope_theta=float(theta),
        max_position_embeddings=int(cfg.get("max_position_embeddings", DEFAULT_MAX_POSITION)),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", True)),
        intermediate_size=inter, num_dense_layers=dense, **kw)
