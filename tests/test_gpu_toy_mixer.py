"""(c)'s generality: a mixer with state of its own, defined here, is registered, built into a model
by a new architecture and stepped, without a change to any file of the framework."""
import pytest
import torch

from helpers import rel_rows

pytestmark = pytest.mark.gpu


def register_toy():
    from snowllm_b200.config.registry import register_architecture
    from snowllm_b200.ops import linear
    from snowllm_b200.parts import (LayerSpec, ModelSpec, PartSpec, RunEntry, SlotStateSpec, TensorSpec,
                                    register_mixer)
    from snowllm_b200.parts.base import Part

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t per channel, y_t = W s_t; the state s is float32 and lives in
        the request's slot.  Plain torch inside: what matters here is the interface."""
        libraries = ("gemm",)

        def __init__(self, dtype, names, *, hidden_size, decay):
            super().__init__(dtype, names)
            self.hidden_size, self.decay = hidden_size, decay

        def cache_spec(self):
            return SlotStateSpec(((self.hidden_size,),), ("f32",))

        def declare(self, has):
            return [TensorSpec("w", self.names["w"], (self.hidden_size, self.hidden_size))]

        def bind(self, tensors):
            self.w = tensors["w"]

        def forward(self, ctx, x, cache, owns_cache=True):
            state = cache.tensors[0]
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for b in range(ctx.B):
                lo, n = ctx.host_seg_start[b], ctx.host_seg_len[b]
                first = sum(ctx.host_seg_len[:b])
                slot = int(ctx.seg_slot[b])
                s = state[slot].clone() if lo > 0 else torch.zeros_like(state[slot])
                for t in range(n):
                    s = self.decay * s + x[first + t].float()
                    out[first + t] = s
                state[slot] = s
            return linear(out.to(self.dtype), self.w, out_dtype=torch.float32)

    register_mixer("toy_decay", DecayMixer)

    def read_config(cfg):
        return dict(cfg)

    def model_spec(c):
        H = c["hidden_size"]
        layers = []
        for i in range(c["num_hidden_layers"]):
            p = f"toy.{i}."
            mixer = (PartSpec("toy_decay", dict(hidden_size=H, decay=c["decay"]), dict(w=p + "mix.w")) if i % 2 == 0
                     else PartSpec("short_conv", dict(hidden_size=H, kernel_size=2),
                                   dict(in_proj=p + "in", conv=p + "conv", out_proj=p + "out")))
            ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=2 * H),
                           dict(gate=p + "g", up=p + "u", down=p + "d"))
            norm = lambda n: PartSpec("rmsnorm", dict(size=H, eps=1e-5), dict(weight=p + n))
            layers.append(LayerSpec("prenorm", mixer, ffn, norm("n1"), norm("n2")))
        return ModelSpec("ToyDecayLM", c["vocab_size"], H,
                         PartSpec("embedding", dict(vocab_size=c["vocab_size"], hidden_size=H), dict(weight="toy.emb")),
                         layers, [RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(0)],    # layer 0 runs twice
                         PartSpec("rmsnorm", dict(size=H, eps=1e-5), dict(weight="toy.norm")),
                         PartSpec("linear_head", dict(vocab_size=c["vocab_size"], hidden_size=H, tied=True),
                                  dict(weight="toy.emb")))

    register_architecture("ToyDecayLM", read_config, model_spec)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_registers_builds_and_steps(tmp_path, dtype):
    import snowllm_b200
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.loader import build_model, parse_dtype
    from snowllm_b200.weights import random_tensors, write_model_folder
    register_toy()
    cfg = {"architectures": ["ToyDecayLM"], "vocab_size": 97, "hidden_size": 48, "num_hidden_layers": 3,
           "decay": 0.8}
    model = build_model(cfg, dtype)
    tensors = random_tensors(model, 2, parse_dtype(dtype), fan_in_scaled=True)
    write_model_folder(tmp_path, cfg, tensors)
    model = snowllm_b200.load(tmp_path, dtype)
    specs = model.cache_specs()
    assert sorted(specs) == [0, 1, 2, 3]              # the layer that runs twice owns two states
    cache = CacheManager(specs, 16, 4, 2, model.dtype, "cuda")
    runner = ModelRunner(model, cache)
    toks = [int(t) for t in torch.randint(0, 97, (29,))]
    a = cache.admit()
    whole = runner.step([StepEntry(a, toks, list(range(29)))]).cpu()
    cache.free(a)
    b, c = cache.admit(), cache.admit()
    other = [int(t) for t in torch.randint(0, 97, (11,))]
    outs, i = [], 0
    for n in (4, 1, 9, 2, 13):
        entries = [StepEntry(b, toks[i:i + n], list(range(n)))]
        if i == 5:
            entries.append(StepEntry(c, other, []))       # another request beside it
        outs.append(runner.step(entries).cpu())
        i += n
    cut = torch.cat(outs)
    assert float(rel_rows(cut, whole).max()) < (1e-5 if dtype == "float32" else 4e-2)
    # against the recurrence written out
    t = {k: v.float() for k, v in tensors.items()}
    import plain_lfm2 as plain
    x = t["toy.emb"][toks]
    def decay_mixer(u, w):
        s, ys = torch.zeros(48), []
        for row in u:
            s = 0.8 * s + row
            ys.append(s)
        return torch.stack(ys) @ w.T
    for layer in (0, 1, 2, 0):
        p = f"toy.{layer}."
        u = plain.rmsnorm(x, t[p + "n1"], 1e-5)
        x = x + (decay_mixer(u, t[p + "mix.w"]) if layer % 2 == 0 else
                 plain.short_conv_mixer(u, t[p + "in"], t[p + "conv"].reshape(48, 2), t[p + "out"]))
        x = x + plain.dense_ffn(plain.rmsnorm(x, t[p + "n2"], 1e-5), t[p + "g"], t[p + "u"], t[p + "d"])
    want = plain.rmsnorm(x, t["toy.norm"], 1e-5) @ t["toy.emb"].T
    assert float(rel_rows(whole, want).max()) < (2e-5 if dtype == "float32" else 4e-2)


def register_hybrid():
    """A mixer that asks for pages AND for state of fixed size: its cache_spec() is a tuple, and so is the
    view it is handed.  The pages hold one latent row per position (a cache of keys only, no values, kept
    in float32 whatever the compute dtype); the slot holds a running sum."""
    from snowllm_b200.config.registry import register_architecture
    from snowllm_b200.ops import linear
    from snowllm_b200.parts import (LayerSpec, ModelSpec, PagedKVSpec, PartSpec, RunEntry, SlotStateSpec, TensorSpec,
                                    register_mixer)
    from snowllm_b200.parts.base import Part

    class LatentMeanMixer(Part):
        """z_t = x_t kept per position in pages; y_t = W (max over the cached z_0..z_t, elementwise, plus
        decay-sum s_t = decay * s_{t-1} + x_t from the slot)."""
        libraries = ("gemm",)

        def __init__(self, dtype, names, *, hidden_size, decay):
            super().__init__(dtype, names)
            self.hidden_size, self.decay = hidden_size, decay

        def cache_spec(self):
            return (PagedKVSpec(1, self.hidden_size, v_head_dim=0, cache_dtype="float32"),
                    SlotStateSpec(((self.hidden_size,),), ("f32",)))

        def declare(self, has):
            return [TensorSpec("w", self.names["w"], (self.hidden_size, self.hidden_size))]

        def bind(self, tensors):
            self.w = tensors["w"]

        def forward(self, ctx, x, cache, owns_cache=True):
            pages, slots = cache                                   # in the order of cache_spec()
            assert pages.pool.dtype == torch.float32 and pages.pool.shape[1:] == (1, pages.page_size, self.hidden_size)
            state = slots.tensors[0]
            P = pages.page_size
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for b in range(ctx.B):
                lo, n = ctx.host_seg_start[b], ctx.host_seg_len[b]
                first = sum(ctx.host_seg_len[:b])
                table = pages.block_table[b].tolist()
                slot = int(ctx.seg_slot[b])
                s = state[slot].clone() if lo > 0 else torch.zeros_like(state[slot])
                for t in range(n):
                    pos = lo + t
                    xt = x[first + t].float()
                    pages.pool[table[pos // P], 0, pos % P] = xt
                    seen = torch.stack([pages.pool[table[p // P], 0, p % P] for p in range(pos + 1)])
                    s = self.decay * s + xt
                    out[first + t] = seen.max(0).values + s
                state[slot] = s
            return linear(out.to(self.dtype), self.w, out_dtype=torch.float32)

    register_mixer("toy_latent", LatentMeanMixer)

    def model_spec(c):
        H = c["hidden_size"]
        layers = []
        for i in range(2):
            p = f"toy.{i}."
            mixer = PartSpec("toy_latent", dict(hidden_size=H, decay=0.5), dict(w=p + "mix.w"))
            ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=2 * H), dict(gate=p + "g", up=p + "u", down=p + "d"))
            norm = lambda n: PartSpec("rmsnorm", dict(size=H, eps=1e-5), dict(weight=p + n))
            layers.append(LayerSpec("prenorm", mixer, ffn, norm("n1"), norm("n2")))
        return ModelSpec("ToyLatentLM", c["vocab_size"], H,
                         PartSpec("embedding", dict(vocab_size=c["vocab_size"], hidden_size=H), dict(weight="toy.emb")),
                         layers, [RunEntry(0), RunEntry(1)],
                         PartSpec("rmsnorm", dict(size=H, eps=1e-5), dict(weight="toy.norm")),
                         PartSpec("linear_head", dict(vocab_size=c["vocab_size"], hidden_size=H, tied=True),
                                  dict(weight="toy.emb")))

    register_architecture("ToyLatentLM", lambda cfg: dict(cfg), model_spec)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixer_with_pages_and_state_at_once(tmp_path, dtype):
    import plain_lfm2 as plain
    import snowllm_b200
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.loader import build_model, parse_dtype
    from snowllm_b200.weights import random_tensors, write_model_folder
    register_hybrid()
    cfg = {"architectures": ["ToyLatentLM"], "vocab_size": 61, "hidden_size": 40}
    model = build_model(cfg, dtype)
    tensors = random_tensors(model, 4, parse_dtype(dtype), fan_in_scaled=True)
    write_model_folder(tmp_path, cfg, tensors)
    model = snowllm_b200.load(tmp_path, dtype)
    cache = CacheManager(model.cache_specs(), 8, 9, 2, model.dtype, "cuda")
    assert all(t.dtype == torch.float32 for t in cache.paged_tensors()) and len(cache.state_tensors()) == 2
    runner = ModelRunner(model, cache)
    toks = [int(t) for t in torch.randint(0, 61, (27,))]
    other = [int(t) for t in torch.randint(0, 61, (19,))]
    a = cache.admit()
    assert cache.ensure(a, len(toks))
    whole = runner.step([StepEntry(a, toks, list(range(27)))]).cpu()
    cache.free(a)
    b, c = cache.admit(), cache.admit()
    outs, i = [], 0
    for n in (3, 1, 10, 2, 11):                              # the other request beside it from the third step on
        assert cache.ensure(b, i + n)
        entries = [StepEntry(b, toks[i:i + n], list(range(n)))]
        if i >= 4 and c.num_tokens < len(other):
            m = min(7, len(other) - c.num_tokens)
            assert cache.ensure(c, c.num_tokens + m)
            entries.append(StepEntry(c, other[c.num_tokens:c.num_tokens + m], []))
        outs.append(runner.step(entries).cpu())
        i += n
    cut = torch.cat(outs)
    assert float(rel_rows(cut, whole).max()) < (1e-5 if dtype == "float32" else 4e-2)
    cache.free(b)
    cache.free(c)
    assert all(p.free_count == p.total for p in cache.groups.values()) and cache.slots.free_count == 2
    # against the computation written out
    t = {k: v.float() for k, v in tensors.items()}
    x = t["toy.emb"][toks]
    for layer in range(2):
        p = f"toy.{layer}."
        u = plain.rmsnorm(x, t[p + "n1"], 1e-5)
        s, ys = torch.zeros(40), []
        for i, row in enumerate(u):
            s = 0.5 * s + row
            ys.append(u[:i + 1].max(0).values + s)
        x = x + torch.stack(ys) @ t[p + "mix.w"].T
        x = x + plain.dense_ffn(plain.rmsnorm(x, t[p + "n2"], 1e-5), t[p + "g"], t[p + "u"], t[p + "d"])
    want = plain.rmsnorm(x, t["toy.norm"], 1e-5) @ t["toy.emb"].T
    assert float(rel_rows(whole, want).max()) < (2e-5 if dtype == "float32" else 4e-2)
