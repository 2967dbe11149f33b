"""The plain implementation checked against itself and against hand-written loops: it is the
oracle, so its own parts get a second, even slower, formulation here."""
import math

import torch

import plain_lfm2 as plain
from helpers import make_model_dir, random_prompt
from tiny_configs import ALL


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    got = plain.rmsnorm(x, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(got, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))


def test_rope_is_a_rotation_of_split_halves():
    hd, theta = 8, 100.0
    x = torch.randn(5, 2, hd)
    ang = plain.rope_angles(torch.arange(5), hd, theta)
    y = plain.apply_rope(x, ang)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.allclose(y[0], x[0])                                  # position 0: no rotation
    for i in range(hd // 2):
        a = 3 * theta ** (-2 * i / hd)
        want0 = x[3, 1, i] * math.cos(a) - x[3, 1, i + hd // 2] * math.sin(a)
        want1 = x[3, 1, i + hd // 2] * math.cos(a) + x[3, 1, i] * math.sin(a)
        assert abs(float(y[3, 1, i] - want0)) < 1e-5 and abs(float(y[3, 1, i + hd // 2] - want1)) < 1e-5


def test_short_conv_by_loops():
    T, H, L = 7, 6, 4
    u = torch.randn(T, H)
    w_in, w_conv, w_out = torch.randn(3 * H, H), torch.randn(H, L), torch.randn(H, H)
    got = plain.short_conv_mixer(u, w_in, w_conv, w_out)
    bcx = u @ w_in.T
    B, C, x = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    g = B * x
    y = torch.zeros(T, H)
    for t in range(T):
        for c in range(H):
            acc = 0.0
            for j in range(L):
                s = t - (L - 1) + j
                if s >= 0:
                    acc += float(w_conv[c, j] * g[s, c])
            y[t, c] = C[t, c] * acc
    assert torch.allclose(got, y @ w_out.T, atol=1e-4)


def test_attention_by_loops_with_and_without_window():
    T, H, nh, nkv, hd = 9, 12, 4, 2, 6
    u = torch.randn(T, H)
    wq, wk, wv, wo = torch.randn(nh * hd, H), torch.randn(nkv * hd, H), torch.randn(nkv * hd, H), torch.randn(H, nh * hd)
    qn, kn = torch.rand(hd) + 0.5, torch.rand(hd) + 0.5
    for window in (None, 3):
        got = plain.attention_mixer(u, wq, wk, wv, wo, qn, kn, 1e-5, nh, nkv, hd, 50.0, window=window)
        ang = plain.rope_angles(torch.arange(T), hd, 50.0)
        q = plain.apply_rope(plain.rmsnorm((u @ wq.T).view(T, nh, hd), qn, 1e-5), ang)
        k = plain.apply_rope(plain.rmsnorm((u @ wk.T).view(T, nkv, hd), kn, 1e-5), ang)
        v = (u @ wv.T).view(T, nkv, hd)
        out = torch.zeros(T, nh, hd)
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            for h in range(nh):
                g = h // (nh // nkv)
                s = torch.stack([q[t, h] @ k[j, g] for j in range(lo, t + 1)]) * hd ** -0.5
                p = torch.softmax(s, 0)
                out[t, h] = sum(p[j - lo] * v[j, g] for j in range(lo, t + 1))
        assert torch.allclose(got, out.reshape(T, -1) @ wo.T, atol=1e-4), window


def test_router_bias_only_selects_ties_go_low_and_weights_normalise():
    u = torch.zeros(1, 4)
    gate = torch.zeros(3, 4)                      # every p = 0.5: a three-way tie
    ids, w = plain.route(u, gate, None, 2, True, 3.0)
    assert ids.tolist() == [[0, 1]] and torch.allclose(w, torch.full((1, 2), 0.5 / (1 + 1e-6) * 3.0))
    ids, w = plain.route(u, gate, torch.tensor([0.0, 0.0, 1.0]), 2, False, 1.0)
    assert ids.tolist() == [[2, 0]] and torch.allclose(w, torch.full((1, 2), 0.5))   # bias not in the weight


def test_logits_at_a_position_ignore_later_tokens(tmp_path):
    for name in ("tiny_a", "tiny_b"):
        d = make_model_dir(tmp_path / name, name)
        cfg, tensors = plain.read_model_dir(d)
        ids = random_prompt(cfg["vocab_size"], 24, 3)
        full = plain.logits(cfg, tensors, ids)
        part = plain.logits(cfg, tensors, ids[:11])
        assert torch.allclose(full[:11], part, atol=1e-5)
        assert full.shape == (24, cfg["vocab_size"])
        other = ids[:11] + random_prompt(cfg["vocab_size"], 13, 4)
        assert not torch.allclose(plain.logits(cfg, tensors, other)[12:], full[12:], atol=1e-3)


def test_forced_routes_equal_free_routes_when_they_agree(tmp_path):
    d = make_model_dir(tmp_path / "m", "tiny_b")
    cfg, tensors = plain.read_model_dir(d)
    ids = random_prompt(cfg["vocab_size"], 10, 1)
    margins = {}
    free = plain.logits(cfg, tensors, ids, margins=margins)
    assert sorted(margins) == [2, 3, 4] and all((m >= 0).all() for m in margins.values())
    u = torch.randn(10, 96)
    p = "model.layers.2.feed_forward."
    own, _ = plain.route(u, tensors[p + "gate.weight"], None, 4, False, 2.0)
    again, _ = plain.route(u, tensors[p + "gate.weight"], None, 4, False, 2.0, forced_ids=own)
    assert torch.equal(own, again)
    assert free.isfinite().all()


def test_sampling_reference_cuts():
    row = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))
    assert plain.softmax_sample_reference(row, 1.0, 0, 1.0, 0.0) == 0
    assert plain.softmax_sample_reference(row, 1.0, 0, 1.0, 0.6) == 1
    assert plain.softmax_sample_reference(row, 1.0, 0, 1.0, 0.999) == 3
    assert plain.softmax_sample_reference(row, 1.0, 2, 1.0, 0.999) == 1       # top-2 only
    assert plain.softmax_sample_reference(row, 1.0, 0, 0.7, 0.999) == 1       # 0.5 + 0.3 reaches 0.7
    assert plain.softmax_sample_reference(row, 1.0, 0, 0.81, 0.999) == 2


def test_plain_implementation_still_gives_its_recorded_logits():
    """tests/golden/plain_tiny.pt holds the oracle's own outputs (made by tests/golden/make_golden.py)."""
    import importlib.util
    import pathlib
    here = pathlib.Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_golden", here / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    recorded = torch.load(here / "plain_tiny.pt")
    for name, case in mod.cases().items():
        assert case["ids"] == recorded[name]["ids"]
        assert torch.allclose(case["logits"], recorded[name]["logits"], atol=1e-5, rtol=1e-5), name
