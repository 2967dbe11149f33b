"""(c)'s generality with the framework's own parts: a toy architecture, defined here, whose run list holds an
attention layer with a window (its pages are given back as the window passes), a layer that keeps every key,
a third layer that reads the second layer's cache instead of owning one, and a partial rotary encoding.  It is
registered from outside the package, loaded from a folder, replayed whole and in small portions through a pool
that is too small without the window's releases, and compared with a plain computation written out below."""
import pytest
import torch

import plain_lfm2 as plain
from helpers import random_prompt, rel_rows

pytestmark = pytest.mark.gpu
H, NH, NKV, HD, WINDOW, ROT, THETA, EPS, V = 64, 4, 2, 16, 24, 8, 300.0, 1e-5, 120


def register():
    from snowllm_b200.config.registry import register_architecture
    from snowllm_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry

    def attention(p, window):
        return PartSpec("attention",
                        dict(hidden_size=H, num_heads=NH, num_kv_heads=NKV, head_dim=HD, qk_norm_eps=EPS,
                             position=dict(kind="rope", head_dim=HD, theta=THETA, rot_dim=ROT), window=window),
                        {k: p + k for k in ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm")})

    def model_spec(c):
        layers = []
        for i, window in enumerate((WINDOW, None, None)):
            p = f"t.{i}."
            ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=96), dict(gate=p + "g", up=p + "u", down=p + "d"))
            norm = lambda n: PartSpec("rmsnorm", dict(size=H, eps=EPS), dict(weight=p + n))
            layers.append(LayerSpec("prenorm", attention(p, window), ffn, norm("n1"), norm("n2")))
        return ModelSpec("ToyWindowLM", V, H, PartSpec("embedding", dict(vocab_size=V, hidden_size=H), dict(weight="t.emb")),
                         layers, [RunEntry(0), RunEntry(1), RunEntry(2, cache_of=1)],
                         PartSpec("rmsnorm", dict(size=H, eps=EPS), dict(weight="t.norm")),
                         PartSpec("linear_head", dict(vocab_size=V, hidden_size=H, tied=True), dict(weight="t.emb")))

    register_architecture("ToyWindowLM", dict, model_spec)


def plain_logits(t, toks):
    """The same model written out: layer 0 sees the last WINDOW keys, layer 2 attends over layer 1's keys and
    values with its own queries; only the first ROT elements of a head rotate."""
    T = len(toks)
    ang = plain.rope_angles(torch.arange(T), ROT, THETA)

    def qkv(p, u):
        def rot(x, w):
            x = plain.rmsnorm(x, w, EPS)
            return torch.cat((plain.apply_rope(x[..., :ROT], ang), x[..., ROT:]), -1)
        q = rot((u @ t[p + "q_proj"].T).view(T, NH, HD), t[p + "q_norm"])
        k = rot((u @ t[p + "k_proj"].T).view(T, NKV, HD), t[p + "k_norm"])
        return q, k, (u @ t[p + "v_proj"].T).view(T, NKV, HD)

    def attend(q, k, v, window):
        out = torch.zeros(T, NH, HD)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            for h in range(NH):
                g = h // (NH // NKV)
                p = torch.softmax((k[lo:i + 1, g] @ q[i, h]) * HD ** -0.5, 0)
                out[i, h] = p @ v[lo:i + 1, g]
        return out.reshape(T, NH * HD)

    x = t["t.emb"][toks]
    shared = None
    for i, window in enumerate((WINDOW, None, None)):
        p = f"t.{i}."
        q, k, v = qkv(p, plain.rmsnorm(x, t[p + "n1"], EPS))
        if i == 1:
            shared = (k, v)
        if i == 2:
            k, v = shared
        x = x + attend(q, k, v, window) @ t[p + "out_proj"].T
        x = x + plain.dense_ffn(plain.rmsnorm(x, t[p + "n2"], EPS), t[p + "g"], t[p + "u"], t[p + "d"])
    return plain.rmsnorm(x, t["t.norm"], EPS) @ t["t.emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_group_shared_cache_and_partial_rotary(tmp_path, dtype):
    import snowllm_b200
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.loader import build_model, parse_dtype
    from snowllm_b200.weights import random_tensors, write_model_folder
    register()
    cfg = {"architectures": ["ToyWindowLM"]}
    tensors = random_tensors(build_model(cfg, dtype), 5, parse_dtype(dtype), fan_in_scaled=True, norm_jitter=0.1)
    write_model_folder(tmp_path, cfg, tensors)
    model = snowllm_b200.load(tmp_path, dtype)
    specs = model.cache_specs()
    assert sorted(specs) == [0, 1] and specs[0].window == WINDOW and specs[1].window is None   # entry 2 owns none
    P = 8
    toks = random_prompt(V, 200, 9)
    want = plain_logits({k: v.float() for k, v in tensors.items()}, toks)
    # the window group gets 6 pages only: 200 tokens need 25, so a missing release would stop the run
    pages = {("paged", WINDOW): 6, ("paged", None): 26}
    tol = 2e-5 if dtype == "float32" else 0.1
    for cuts in ([16] * 13, [5, 2, 9, 1, 1, 7, 16, 3] * 5):
        cache = CacheManager(specs, P, pages, 1, model.dtype, "cuda")
        runner = ModelRunner(model, cache)
        rc = cache.admit()
        outs, i = [], 0
        for n in cuts:
            n = min(n, len(toks) - i)
            if n <= 0:
                break
            assert cache.ensure(rc, i + n), f"no pages at token {i}: {cache.free_pages()}"
            outs.append(runner.step([StepEntry(rc, toks[i:i + n], list(range(n)))]).float().cpu())
            i += n
            assert cache.groups[("paged", WINDOW)].held() <= 6
        assert i == len(toks)
        err = rel_rows(torch.cat(outs), want)
        bad = torch.nonzero(err > tol).flatten().tolist()
        assert not bad, f"first wrong position {bad[0]} (rel {float(err[bad[0]]):.3g})"
        cache.free(rc)
        assert all(p.free_count == p.total for p in cache.groups.values())
