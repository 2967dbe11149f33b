"""Plain, slow LFM2 / LFM2.5 forward pass: the oracle of the test-suite.

Whole sequences, no cache, one function per part, float32 arithmetic throughout,
plain PyTorch on whatever device the tensors live on (the CPU in the tests).  It
shares no code with ``snowllm_b200``: it has its own config reading, its own
safetensors parser and its own formulas.

Anchoring.  SnowLLM's own model code cannot be imported or compiled on a CPU (its
modules load a closed HIP kernel library at import time), so this file rests on
the formulas alone.  Each function cites the place in SnowLLM/SnowLLM (path within
that project) from which its formula is read.

Rounding variant.  Inside ``with stores_rounded_to(torch.bfloat16):`` every intermediate
that a bfloat16 engine keeps in bfloat16 between two kernels is rounded to it (``_store``):
norm outputs, the products that do not feed the residual stream (in_proj, q/k/v, the
SwiGLU activation), the conv's g = B*x and y = C*conv, q and k after head norm and
rotation, the attention output, and the softmax weights P on their way into P.V (written
as 2^(s log2 e - m) with m the row's maximum rounded up to a whole number, so that the
rounded mantissas do not depend on m; the row sum keeps the unrounded values).  The
arithmetic between two stores stays float32, as do
the residual stream, the products that feed it, the router and the logits.  A bfloat16
run is compared with this variant, so that what is left is accumulation order, not the
roundings themselves.  Outside the ``with`` nothing is rounded.
"""
from __future__ import annotations

import json
import math
import pathlib
import struct

import torch
import torch.nn.functional as F

_STORE_DTYPE = None


class stores_rounded_to:
    """Context manager: round what a reduced-precision engine stores between kernels to ``dtype``
    (None or float32: round nothing)."""

    def __init__(self, dtype):
        self.dtype = None if dtype in (None, torch.float32, "float32") else \
            (torch.bfloat16 if dtype == "bfloat16" else dtype)

    def __enter__(self):
        global _STORE_DTYPE
        self.before, _STORE_DTYPE = _STORE_DTYPE, self.dtype

    def __exit__(self, *exc):
        global _STORE_DTYPE
        _STORE_DTYPE = self.before


def _store(x):
    """A value as it comes back after being kept in the engine's storage dtype."""
    return x if _STORE_DTYPE is None else x.to(_STORE_DTYPE).float()


_ST_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
    "I32": torch.int32, "I64": torch.int64, "F64": torch.float64,
}


def read_safetensors(path):
    """name -> tensor, from one .safetensors file (8-byte little-endian header
    length, JSON header, raw bytes; snowllm/checkpoint/reader.py:64-76)."""
    raw = pathlib.Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = bytearray(raw[base + lo:base + hi])
        t = torch.frombuffer(buf, dtype=_ST_DTYPES[meta["dtype"]]) if hi > lo else \
            torch.empty(0, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def read_model_dir(path):
    """(config dict, tensors as float32) of a model folder
    (snowllm/checkpoint/loader.py:203-212: text_config is taken when present)."""
    path = pathlib.Path(path)
    raw = json.loads((path / "config.json").read_text())
    cfg = dict(raw.get("text_config", raw))
    cfg.setdefault("architectures", raw.get("architectures"))
    tensors = {k: v.float() for k, v in read_safetensors(path / "model.safetensors").items()}
    return cfg, tensors


def rope_theta(cfg):
    """snowllm/models/lfm2/weights.py:44: rope_parameters.rope_theta, else rope_theta,
    else 5,000,000."""
    return (cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta", 5000000.0))


def head_dim(cfg):
    """snowllm/models/lfm2/weights.py:36-39: hidden_size // num_attention_heads
    (an explicit head_dim key, where a config gives one, takes precedence)."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def rmsnorm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * weight, the weight multiplying directly
    (tests/test_lfm2_dspark_reference.py:16-19; snowllm/ops/norm.py:11-30)."""
    x = x.float()
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * weight.float()


def rmsnorm_stored(x, weight, eps):
    """The norm of the residual stream as the layer after it reads it (one store)."""
    return _store(rmsnorm(x, weight, eps))


def rope_angles(positions, hd, theta):
    """ang[m, i] = pos[m] * theta^(-2i/hd), float32
    (snowllm/models/lfm2/layers.py:116-117; snowllm/ops/rope.py:11-24)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    return positions.to(torch.float32)[:, None] * inv_freq[None, :].to(positions.device)


def apply_rope(x, ang):
    """Split-half rotation over the whole head: x*cos + rot(x)*sin with
    rot(x) = [-x[hd/2:], x[:hd/2]] (tests/test_lfm2.py:108-118).  x: [T, heads, hd]."""
    cos = torch.cat((ang.cos(), ang.cos()), -1)[:, None, :]
    sin = torch.cat((ang.sin(), ang.sin()), -1)[:, None, :]
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), -1)
    return x * cos + rot * sin


def short_conv_mixer(u, w_in, w_conv, w_out):
    """Gated short convolution (snowllm/models/lfm2/layers.py:26-33;
    tests/test_lfm2.py:41-49): BCx = in_proj(u); B, C, x = thirds; g = B*x; causal
    depthwise conv of length L with zero history (the last tap multiplies the
    current token); y = C*conv; out_proj(y).  u: [T, H]; w_conv: [H, L]."""
    T, H = u.shape
    L = w_conv.shape[-1]
    bcx = _store(u @ w_in.T)
    B, C, x = bcx.chunk(3, dim=-1)
    g = _store(B * x)
    conv = F.conv1d(g.T[None], w_conv.reshape(H, 1, L), padding=L - 1, groups=H)[0, :, :T].T
    return _store(C * conv) @ w_out.T


def attention_mixer(u, wq, wk, wv, wo, q_norm, k_norm, eps, n_heads, n_kv, hd, theta,
                    window=None, positions=None):
    """Causal grouped-query attention with per-head RMSNorm on q and k, then RoPE
    (snowllm/models/lfm2/layers.py:36-70; grouping and mask as in
    tests/test_lfm2_long_attention.py:36-47): q head i reads kv head i // (nh/nkv);
    scale hd^-0.5; softmax in float32.  ``window`` (not an LFM2 option) keeps only the
    last ``window`` keys, the query's own included."""
    T = u.shape[0]
    pos = torch.arange(T, device=u.device) if positions is None else positions
    q = _store(u @ wq.T).view(T, n_heads, hd)
    k = _store(u @ wk.T).view(T, n_kv, hd)
    v = _store(u @ wv.T).view(T, n_kv, hd)
    q = rmsnorm(q, q_norm, eps)
    k = rmsnorm(k, k_norm, eps)
    ang = rope_angles(pos, hd, theta)
    q, k = _store(apply_rope(q, ang)), _store(apply_rope(k, ang))
    group = n_heads // n_kv
    q = q.view(T, n_kv, group, hd)
    scores = torch.einsum("tghd,sgd->tghs", q, k) * hd ** -0.5
    i = torch.arange(T, device=u.device)
    mask = i[None, :] > i[:, None]
    if window is not None:
        mask = mask | (i[None, :] <= i[:, None] - window)
    scores = scores.masked_fill(mask[:, None, None, :], float("-inf"))
    if _STORE_DTYPE is None:
        probs = scores.softmax(-1)
    else:
        # the rounding variant: P = 2^(s log2 e - m), m a whole number; P is stored, the row sum is not
        s2 = scores * 1.4426950408889634
        p = torch.exp2(s2 - torch.ceil(s2.amax(-1, keepdim=True)))
        probs = _store(p) / p.sum(-1, keepdim=True)
    out = torch.einsum("tghs,sgd->tghd", probs, v).reshape(T, n_heads * hd)
    return _store(out) @ wo.T


def dense_ffn(u, w1, w3, w2):
    """SwiGLU: w2(silu(w1 u) * w3 u) (snowllm/models/lfm2/layers.py:81-88).  Rounding variant: the
    activation is stored once; a width that is no multiple of 8 makes the engine store gate and up
    first (its fused store needs gate and up rows interleaved by 8)."""
    g, p = u @ w1.T, u @ w3.T
    if w1.shape[0] % 8:
        g, p = _store(g), _store(p)
    return _store(F.silu(g) * p) @ w2.T


def route(u, gate_w, expert_bias, top_k, norm_topk_prob, scaling, forced_ids=None, margins=None):
    """Sigmoid router in float32 (tests/test_lfm2_reference.py:113-119): p = sigmoid(u W^T);
    the k largest of p + bias select (the bias only selects); weights p[sel], divided by
    (sum + 1e-6) when norm_topk_prob, times routed_scaling_factor.  Ties go to the lower
    expert index.  ``forced_ids`` replaces the selection (the weights still come from p);
    ``margins`` (a list) receives, per row, the gap between the k-th and the (k+1)-th score."""
    p = (u.float() @ gate_w.float().T).sigmoid()
    score = p if expert_bias is None else p + expert_bias.float()
    # stable descending sort: equal scores keep index order, so the lower index wins
    order = torch.sort(score, dim=-1, descending=True, stable=True)
    if margins is not None:
        v = order.values
        margins.append(v[:, top_k - 1] - v[:, top_k] if top_k < v.shape[1]
                       else torch.full((v.shape[0],), float("inf"), device=v.device))
    ids = order.indices[:, :top_k] if forced_ids is None else forced_ids.long()
    w = p.gather(1, ids)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-6)
    return ids, w * scaling


def moe_ffn(u, gate_w, expert_bias, w1, w3, w2, top_k, norm_topk_prob, scaling, forced_ids=None,
            margins=None):
    """Routed SwiGLU experts, no shared expert (snowllm/models/qwen3_5/layers.py:176-188;
    formula tests/test_lfm2_reference.py:113-119).  w1, w3: [E, I, H]; w2: [E, H, I]."""
    ids, w = route(u, gate_w, expert_bias, top_k, norm_topk_prob, scaling, forced_ids, margins)
    out = torch.zeros_like(u)
    for e in range(w1.shape[0]):                 # expert by expert over the rows that picked it
        picked = ids == e
        rows = picked.any(-1)
        if rows.any():
            weight = (w * picked).sum(-1)[rows]
            out[rows] += weight[:, None] * dense_ffn(u[rows], w1[e], w3[e], w2[e])
    return out


def expert_stack(tensors, prefix, n_experts):
    """Per-expert tensors stacked, or the fused gate_up_proj split in two
    (snowllm/models/lfm2/weights.py:84-91)."""
    key = prefix + "feed_forward.experts."
    if key + "gate_up_proj" in tensors:
        w1, w3 = tensors[key + "gate_up_proj"].chunk(2, dim=1)
        return w1, w3, tensors[key + "down_proj"]
    stack = lambda n: torch.stack([tensors[f"{key}{e}.{n}.weight"] for e in range(n_experts)])
    return stack("w1"), stack("w3"), stack("w2")


def layer_mixer(cfg, tensors, i, u):
    """Mixer of layer i chosen by layer_types (snowllm/models/lfm2/weights.py:72-76)."""
    p = f"model.layers.{i}."
    if cfg["layer_types"][i] == "conv":
        H = cfg["hidden_size"]
        return short_conv_mixer(u, tensors[p + "conv.in_proj.weight"],
                                tensors[p + "conv.conv.weight"].reshape(H, -1),
                                tensors[p + "conv.out_proj.weight"])
    a = p + "self_attn."
    return attention_mixer(u, tensors[a + "q_proj.weight"], tensors[a + "k_proj.weight"],
                           tensors[a + "v_proj.weight"], tensors[a + "out_proj.weight"],
                           tensors[a + "q_layernorm.weight"], tensors[a + "k_layernorm.weight"],
                           cfg["norm_eps"], cfg["num_attention_heads"],
                           cfg["num_key_value_heads"], head_dim(cfg), rope_theta(cfg))


def is_dense_model(cfg):
    archs = cfg.get("architectures") or []
    return "Lfm2ForCausalLM" in archs


def layer_ffn(cfg, tensors, i, u, forced_ids=None, margins=None):
    """Dense SwiGLU below num_dense_layers, routed experts from there on
    (snowllm/models/lfm2/weights.py:77-92)."""
    p = f"model.layers.{i}."
    if is_dense_model(cfg) or i < cfg.get("num_dense_layers", 0):
        f = p + "feed_forward."
        return dense_ffn(u, tensors[f + "w1.weight"], tensors[f + "w3.weight"],
                         tensors[f + "w2.weight"])
    w1, w3, w2 = expert_stack(tensors, p, cfg["num_experts"])
    bias = tensors[p + "feed_forward.expert_bias"] if cfg.get("use_expert_bias", False) else None
    return moe_ffn(u, tensors[p + "feed_forward.gate.weight"], bias, w1, w3, w2,
                   cfg["num_experts_per_tok"], cfg.get("norm_topk_prob", False),
                   cfg.get("routed_scaling_factor", 1.0), forced_ids, margins)


def hidden_states(cfg, tensors, ids, forced_routes=None, margins=None, trace=None):
    """Embedding, then per layer x += mixer(norm(x)); x += ffn(norm(x)), then the final
    norm (snowllm/models/lfm2/layers.py:97-104, 119-131).  ``forced_routes``: {layer -> ids [T, k]}
    that replace the router's selection in that layer; ``margins``: a dict that receives
    {layer -> selection margin per position}; ``trace``: a list that receives (name, tensor) of each
    layer's mixer input, mixer output, feed-forward input and feed-forward output, in order."""
    eps = cfg["norm_eps"]
    table = tensors["model.embed_tokens.weight"]
    x = table[torch.as_tensor(ids, dtype=torch.long, device=table.device)].float()
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        u = rmsnorm_stored(x, tensors[p + "operator_norm.weight"], eps)
        d = layer_mixer(cfg, tensors, i, u)
        x = x + d
        got = []
        u2 = rmsnorm_stored(x, tensors[p + "ffn_norm.weight"], eps)
        d2 = layer_ffn(cfg, tensors, i, u2, None if forced_routes is None else forced_routes.get(i), got)
        x = x + d2
        if trace is not None:
            trace += [("mixer_in", u), ("mixer_out", d), ("ffn_in", u2), ("ffn_out", d2)]
        if margins is not None and got:
            margins[i] = got[0]
    return rmsnorm_stored(x, tensors["model.embedding_norm.weight"], eps)


def logits(cfg, tensors, ids, forced_routes=None, margins=None, trace=None):
    """[T, V] float32 logits of one whole sequence; the head is the embedding when
    tie_word_embeddings (snowllm/models/lfm2/weights.py:63-66), else lm_head.weight."""
    tied = cfg.get("tie_word_embeddings", True)
    head = tensors["model.embed_tokens.weight"] if tied else tensors["lm_head.weight"]
    with torch.no_grad():
        return hidden_states(cfg, tensors, ids, forced_routes, margins, trace) @ head.float().T


def greedy(cfg, tensors, prompt, n_new):
    """n_new greedy tokens, each from a whole-sequence pass."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(logits(cfg, tensors, toks)[-1].argmax()))
    return toks[len(prompt):]


def softmax_sample_reference(row, temperature, top_k, top_p, u):
    """Reference of the sampler's draw (snowllm/engine/sampler.py:86-104 order:
    temperature softmax, top-k, top-p, inverse CDF from a supplied uniform):
    keep the k most probable, then the smallest prefix of them whose mass reaches
    top_p (ties at the cut all kept), renormalise, walk the CDF in index order."""
    p = torch.softmax(row.double() / temperature, -1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if 0 < top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        q = torch.where(keep, p, torch.zeros_like(p))
        s = torch.sort(q, descending=True).values
        c = torch.cumsum(s, 0)
        n = int((c < top_p * c[-1]).sum()) + 1
        keep &= p >= s[min(n, s.numel()) - 1]
    q = torch.where(keep, p, torch.zeros_like(p))
    c = torch.cumsum(q, 0)
    return int(torch.searchsorted(c, u * c[-1], right=True).clamp(max=p.numel() - 1))
