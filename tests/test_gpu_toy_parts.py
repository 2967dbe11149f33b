"""(c)'s generality: a feed-forward with routing of its own and a position encoding of its own, both
defined here, are registered, built into a model by a new architecture beside the framework's attention and
short-conv mixers, and stepped whole and in portions, without a change to any file of the framework."""
import pytest
import torch

import plain_lfm2 as plain
from helpers import TOL_UNROUNDED as TOL, rel_all, rel_rows, tol_request_unrounded as tol_request

pytestmark = pytest.mark.gpu
H, NH, NKV, HD, V, EPS = 64, 4, 2, 16, 113, 1e-5
FREQ0, STEP = 0.9, 0.35           # the toy position encoding: inv_freq[i] = 1 / (FREQ0 + STEP * i), no powers of a base


def register_toy():
    from snowllm_b200.config.registry import register_architecture
    from snowllm_b200.ops import linear, linear_swiglu
    from snowllm_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry, TensorSpec, register_ffn, register_position
    from snowllm_b200.parts.base import Part

    class HarmonicPosition:
        """Rotary angles with frequencies 1 / (first + step * i): the interface is `rotary(device)`."""

        def __init__(self, *, head_dim, first, step):
            self.inv = 1.0 / (first + step * torch.arange(head_dim // 2, dtype=torch.float32))
            self.head_dim = head_dim

        def rotary(self, device):
            return self.inv.to(device), self.head_dim

    class SignRoutedFFN(Part):
        """Two SwiGLU experts; a token goes to expert 1 where x . r > 0, else to expert 0, and the expert's
        output is scaled by sigmoid(|x . r|).  The routing is plain torch on the device; the products are
        the framework's."""
        libraries = ("gemm", "gemm_skinny", "gemm_tc", "elementwise")

        def __init__(self, dtype, names, *, hidden_size, intermediate_size):
            super().__init__(dtype, names)
            self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

        def declare(self, has):
            Hs, I = self.hidden_size, self.intermediate_size
            specs = [TensorSpec("r", self.names["r"], (1, Hs))]
            for e in (0, 1):
                specs += [TensorSpec(f"gu{e}", self.names[f"gu{e}"], (2 * I, Hs)), TensorSpec(f"d{e}", self.names[f"d{e}"], (Hs, I))]
            return specs

        def bind(self, tensors):
            self.t = tensors

        def forward(self, ctx, x):
            score = linear(x, self.t["r"], out_dtype=torch.float32)[:, 0]
            out = torch.zeros(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            for e in (0, 1):
                rows = torch.nonzero((score > 0) == bool(e))[:, 0]
                if rows.numel():
                    act = linear_swiglu(x[rows].contiguous(), self.t[f"gu{e}"], interleaved=False)
                    out[rows] = linear(act, self.t[f"d{e}"], out_dtype=torch.float32) * torch.sigmoid(score[rows].abs())[:, None]
            return out

    register_position("toy_harmonic", HarmonicPosition)
    register_ffn("toy_sign_routed", SignRoutedFFN)

    def model_spec(c):
        layers = []
        for i in range(3):
            p = f"y.{i}."
            mixer = (PartSpec("short_conv", dict(hidden_size=H, kernel_size=3), dict(in_proj=p + "in", conv=p + "conv", out_proj=p + "out"))
                     if i == 1 else
                     PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=NKV, head_dim=HD, qk_norm_eps=EPS,
                                                position=dict(kind="toy_harmonic", head_dim=HD, first=FREQ0, step=STEP), window=None),
                              {k: p + k for k in ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm")}))
            ffn = (PartSpec("swiglu", dict(hidden_size=H, intermediate_size=80), dict(gate=p + "g", up=p + "u", down=p + "d")) if i == 2 else
                   PartSpec("toy_sign_routed", dict(hidden_size=H, intermediate_size=40),
                            dict(r=p + "r", gu0=p + "gu0", d0=p + "d0", gu1=p + "gu1", d1=p + "d1")))
            norm = lambda n: PartSpec("rmsnorm", dict(size=H, eps=EPS), dict(weight=p + n))
            layers.append(LayerSpec("prenorm", mixer, ffn, norm("n1"), norm("n2")))
        return ModelSpec("ToyRoutedLM", V, H, PartSpec("embedding", dict(vocab_size=V, hidden_size=H), dict(weight="y.emb")),
                         layers, [RunEntry(0), RunEntry(1), RunEntry(2)],
                         PartSpec("rmsnorm", dict(size=H, eps=EPS), dict(weight="y.norm")),
                         PartSpec("linear_head", dict(vocab_size=V, hidden_size=H, tied=True), dict(weight="y.emb")))

    register_architecture("ToyRoutedLM", dict, model_spec)


def plain_logits(t, toks, flips):
    """The same model written out with the plain implementation's functions.  `flips` collects, per routed
    layer, the router scores, so that the caller can leave out rows whose pick rounding may turn."""
    T = len(toks)
    inv = 1.0 / (FREQ0 + STEP * torch.arange(HD // 2, dtype=torch.float32))
    ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]
    x = t["y.emb"][toks]
    for i in range(3):
        p = f"y.{i}."
        u = plain.rmsnorm(x, t[p + "n1"], EPS)
        if i == 1:
            x = x + plain.short_conv_mixer(u, t[p + "in"], t[p + "conv"].reshape(H, 3), t[p + "out"])
        else:
            q = plain.apply_rope(plain.rmsnorm((u @ t[p + "q_proj"].T).view(T, NH, HD), t[p + "q_norm"], EPS), ang)
            k = plain.apply_rope(plain.rmsnorm((u @ t[p + "k_proj"].T).view(T, NKV, HD), t[p + "k_norm"], EPS), ang)
            v = (u @ t[p + "v_proj"].T).view(T, NKV, HD)
            out = torch.zeros(T, NH, HD)
            for h in range(NH):
                g = h // (NH // NKV)
                s = (q[:, h] @ k[:, g].T) * HD ** -0.5
                s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
                out[:, h] = torch.softmax(s, -1) @ v[:, g]
            x = x + out.reshape(T, NH * HD) @ t[p + "out_proj"].T
        u = plain.rmsnorm(x, t[p + "n2"], EPS)
        if i == 2:
            x = x + plain.dense_ffn(u, t[p + "g"], t[p + "u"], t[p + "d"])
        else:
            score = (u @ t[p + "r"].T)[:, 0]
            flips.append(score)
            y = torch.zeros(T, H)
            for e in (0, 1):
                rows = (score > 0) == bool(e)
                gu = u[rows] @ t[p + f"gu{e}"].T
                act = torch.nn.functional.silu(gu[:, :40]) * gu[:, 40:]
                y[rows] = (act @ t[p + f"d{e}"].T) * torch.sigmoid(score[rows].abs())[:, None]
            x = x + y
    return plain.rmsnorm(x, t["y.norm"], EPS) @ t["y.emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_ffn_and_position_register_build_and_step(tmp_path, dtype):
    import snowllm_b200
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.loader import build_model, parse_dtype
    from snowllm_b200.weights import random_tensors, write_model_folder
    register_toy()
    cfg = {"architectures": ["ToyRoutedLM"]}
    model = build_model(cfg, dtype)
    tensors = random_tensors(model, 5, parse_dtype(dtype), fan_in_scaled=True)
    for name in list(tensors):
        if name.endswith(".r"):                            # clear routing decisions: scores far from zero
            tensors[name] = (tensors[name].float() * 40).to(tensors[name].dtype)
    write_model_folder(tmp_path, cfg, tensors)
    model = snowllm_b200.load(tmp_path, dtype)
    cache = CacheManager(model.cache_specs(), 16, 6, 2, model.dtype, "cuda")
    runner = ModelRunner(model, cache)
    toks = [int(t) for t in torch.randint(0, V, (37,), generator=torch.Generator().manual_seed(3))]
    a = cache.admit()
    assert cache.ensure(a, len(toks))
    whole = runner.step([StepEntry(a, toks, list(range(len(toks))))]).cpu()
    cache.free(a)
    b = cache.admit()
    assert cache.ensure(b, len(toks))
    outs, i = [], 0
    for n in (5, 1, 2, 17, 1, 1, 10):                    # portions down to single decoded tokens
        outs.append(runner.step([StepEntry(b, toks[i:i + n], list(range(n)))]).cpu())
        i += n
    cut = torch.cat(outs)
    flips = []
    want = plain_logits({k: v.float() for k, v in tensors.items()}, toks, flips)
    # a row (and what follows it, through attention) is compared only before the first pick that rounding may turn
    margin = 1e-4 if dtype == "float32" else 3e-2
    risky = torch.stack([s.abs() < margin for s in flips]).any(0)
    upto = int(torch.nonzero(risky)[0]) if risky.any() else len(toks)
    assert upto >= 8
    # the suite's bounds against an oracle that does not round (helpers.TOL_UNROUNDED, helpers.tol_request_unrounded): single positions and the request as a whole
    assert float(rel_rows(whole[:upto], want[:upto]).max()) < TOL[dtype]
    assert rel_all(whole[:upto], want[:upto]) < tol_request(dtype, 3)
    assert float(rel_rows(cut[:upto], whole[:upto]).max()) < (1e-5 if dtype == "float32" else TOL[dtype])
