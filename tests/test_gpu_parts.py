"""Each part alone (norm, position encoding, attention mixer, short-conv mixer, dense and routed
feed-forward, block arrangement, embedding and head): built from the registry with constants of
its own, stepped through a hand-made batch, against the plain function of the same part."""
import pytest
import torch

import plain_lfm2 as plain
from helpers import rel_rows

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
# bfloat16 parts are compared with the plain functions' rounding variant (plain.stores_rounded_to): what is
# left is summation order and single elements that fall to the other side of a rounding boundary
TOL = {torch.float32: 1e-5, torch.bfloat16: 5e-3}


def make_part(family, kind, dtype, names, params, seed=0, scale=None):
    """Build a part, draw its tensors (fan-in scaled), bind them on the GPU; returns (part, tensors as float)."""
    from snowllm_b200.parts.registry import lookup
    from snowllm_b200.parts.spec import INIT_ONES
    part = lookup(family, kind)(dtype, names, **params)
    g = torch.Generator().manual_seed(seed)
    tensors, bound = {}, {}
    for spec in part.declare(lambda n: False):
        if spec.init == INIT_ONES:
            t = 1 + 0.2 * torch.randn(spec.stored_shape, generator=g)
        else:
            t = torch.randn(spec.stored_shape, generator=g) * (scale or spec.stored_shape[-1] ** -0.5)
        keep32 = spec.keep == "f32"
        t = t if keep32 else t.to(dtype).float()
        tensors[spec.name] = t
        bound[spec.local] = t.reshape(spec.shape).to("cuda", torch.float32 if keep32 else dtype)
    part.bind(bound)
    return part, tensors


def make_ctx(cache, entries, dtype):
    from snowllm_b200.engine.context import HostStaging
    from snowllm_b200.engine.runner import StepEntry, build_context
    es = [StepEntry(rc, toks, []) for rc, toks in entries]
    return build_context(es, cache, dtype, torch.device("cuda"), HostStaging(torch.device("cuda")), 1 << 20)


def step_mixer(part, dtype, xs, cuts, page_size=16, pages=64):
    """Run a mixer over several requests' inputs xs[b] [T_b, H], cut into steps as cuts[b] says
    (requests with steps left go into each step together); returns outputs per request."""
    from snowllm_b200.cache import CacheManager
    cache = CacheManager({0: part.cache_spec()}, page_size, pages, len(xs), dtype, "cuda")
    for t in cache.paged_tensors() + cache.state_tensors():
        t.fill_(float("nan"))
    rcs = [cache.admit() for _ in xs]
    done = [0] * len(xs)
    outs = [[] for _ in xs]
    for step in range(max(len(c) for c in cuts)):
        seg = [(b, cuts[b][step]) for b in range(len(xs)) if step < len(cuts[b])]
        for b, n in seg:
            assert cache.ensure(rcs[b], done[b] + n)
        ctx = make_ctx(cache, [(rcs[b], [0] * n) for b, n in seg], dtype)
        x = torch.cat([xs[b][done[b]:done[b] + n] for b, n in seg]).to("cuda", dtype)
        y = part.forward(ctx, x, cache.view(0, ctx.block_tables), True)
        assert y.dtype == torch.float32
        row = 0
        for b, n in seg:
            outs[b].append(y[row:row + n].cpu())
            row += n
            done[b] += n
            cache.commit(rcs[b], done[b])
    return [torch.cat(o) for o in outs]


CUTS = [[[41], [17], [64]], [[5, 2, 30, 1, 3], [1] * 17, [63, 1]], [[40, 1], [2, 15], [16, 16, 16, 16]]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window,norm", [(4, 2, 16, None, True), (6, 3, 48, None, True),
                                                   (5, 1, 32, 11, False), (2, 2, 80, None, True)])
def test_attention_mixer(dtype, nh, nkv, hd, window, norm):
    H, theta, eps = 72, 3000.0, 1e-5
    names = {k: k for k in ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm")}
    part, t = make_part("mixer", "attention", dtype, names,
                        dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                             qk_norm_eps=eps if norm else None, position=dict(kind="rope", head_dim=hd, theta=theta),
                             window=window))
    torch.manual_seed(1)
    xs = [torch.randn(n, H).to(dtype).float() for n in (41, 17, 64)]
    ones = torch.ones(hd)
    with plain.stores_rounded_to(dtype):
        want = [plain.attention_mixer(x, t["q_proj"], t["k_proj"], t["v_proj"], t["out_proj"],
                                      t.get("q_norm", ones), t.get("k_norm", ones), eps if norm else 0.0, nh, nkv,
                                      hd, theta, window=window) for x in xs]
        if not norm:      # without a q/k norm the plain function's norm must be the identity: compare unnormalised
            want = [attention_no_norm(x, t, nh, nkv, hd, theta, window) for x in xs]
    first = None
    for cuts in CUTS:
        got = step_mixer(part, dtype, xs, cuts)
        for g, w in zip(got, want):
            assert float(rel_rows(g, w).max()) < TOL[dtype] * 2
        if first is None:
            first = got
        elif dtype == torch.float32:
            for g, f in zip(got, first):
                assert float(rel_rows(g, f).max()) < 1e-6


def attention_no_norm(x, t, nh, nkv, hd, theta, window):
    T = x.shape[0]
    st = plain._store
    q = st(x @ t["q_proj"].T).view(T, nh, hd)
    k = st(x @ t["k_proj"].T).view(T, nkv, hd)
    v = st(x @ t["v_proj"].T).view(T, nkv, hd)
    ang = plain.rope_angles(torch.arange(T), hd, theta)
    q, k = st(plain.apply_rope(q, ang)), st(plain.apply_rope(k, ang))
    out = torch.zeros(T, nh, hd)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(nh):
            g = h // (nh // nkv)
            sc = (k[lo:i + 1, g] @ q[i, h]) * hd ** -0.5
            if plain._STORE_DTYPE is None:
                p = torch.softmax(sc, 0)
            else:                                          # P stored on its way into P.V (see plain_lfm2)
                s2 = sc * 1.4426950408889634
                e = torch.exp2(s2 - torch.ceil(s2.max()))
                p = st(e) / e.sum()
            out[i, h] = p @ v[lo:i + 1, g]
    return st(out.reshape(T, -1)) @ t["out_proj"].T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,L", [(72, 3), (40, 5), (96, 2)])
def test_short_conv_mixer(dtype, H, L):
    names = dict(in_proj="in", conv="conv", out_proj="out")
    part, t = make_part("mixer", "short_conv", dtype, names, dict(hidden_size=H, kernel_size=L))
    torch.manual_seed(2)
    xs = [torch.randn(n, H).to(dtype).float() for n in (41, 17, 64)]
    with plain.stores_rounded_to(dtype):
        want = [plain.short_conv_mixer(x, t["in"], t["conv"].reshape(H, L), t["out"]) for x in xs]
    first = None
    for cuts in CUTS:
        got = step_mixer(part, dtype, xs, cuts)
        for g, w in zip(got, want):
            assert float(rel_rows(g, w).max()) < TOL[dtype] * 2
        if first is None:
            first = got
        elif dtype == torch.float32:    # bfloat16 products of few and of many rows come from different kernels
            assert all(torch.equal(g, f) for g, f in zip(got, first)), "the cut changed the bits"


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forwards(dtype):
    H = 80
    torch.manual_seed(3)
    x = torch.randn(37, H).to(dtype).float()
    part, t = make_part("ffn", "swiglu", dtype, dict(gate="g", up="u", down="d"),
                        dict(hidden_size=H, intermediate_size=112))
    got = part.forward(None, x.to("cuda", dtype)).cpu()
    with plain.stores_rounded_to(dtype):
        assert float(rel_rows(got, plain.dense_ffn(x, t["g"], t["u"], t["d"])).max()) < TOL[dtype]
    for E, k, norm, bias, scaling in ((6, 2, True, True, 1.0), (9, 4, False, False, 2.5)):
        names = dict(router="r", expert_bias="b", experts="e.", expert_gate="w1", expert_up="w3",
                     expert_down="w2", fused_gate_up="gu", fused_down="dn")
        part, t = make_part("ffn", "sigmoid_moe", dtype, names,
                            dict(hidden_size=H, intermediate_size=24, num_experts=E, top_k=k, norm_topk_prob=norm,
                                 use_expert_bias=bias, routed_scaling_factor=scaling))
        ids, _ = part.route(x.to("cuda", dtype))
        w1 = torch.stack([t[f"e.{e}.w1"] for e in range(E)])
        w3 = torch.stack([t[f"e.{e}.w3"] for e in range(E)])
        w2 = torch.stack([t[f"e.{e}.w2"] for e in range(E)])
        with plain.stores_rounded_to(dtype):
            want = plain.moe_ffn(x, t["r"], t.get("b") if bias else None, w1, w3, w2, k, norm, scaling,
                                 forced_ids=ids.cpu())
        delta = part.forward(None, x.to("cuda", dtype))          # an ExpertSum: the weighted sum is still to be formed
        got = delta.dense().cpu()
        assert float(rel_rows(got, want).max()) < TOL[dtype]
        # the norm that follows forms the sum itself: same residual as adding the dense delta
        norm, tn = make_part("norm", "rmsnorm", dtype, dict(weight="w"), dict(size=H, eps=1e-5))
        res_a, res_b = torch.randn(37, H).cuda(), None
        res_b = res_a.clone()
        out_a = norm.forward(None, res_a, delta)
        out_b = norm.forward(None, res_b, delta.dense())
        assert torch.allclose(res_a, res_b, atol=1e-6) and torch.equal(out_a, out_b)
        rows = torch.tensor([3, 36, 0], dtype=torch.int32, device="cuda")
        assert torch.equal(norm.forward(None, res_a.clone(), delta, rows=rows), norm.forward(None, res_b.clone(), delta.dense(), rows=rows))
        # a single row
        one = part.forward(None, x[:1].to("cuda", dtype)).dense().cpu()
        assert float(rel_rows(one, want[:1]).max()) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_embedding_head_and_position(dtype):
    from snowllm_b200.parts.registry import lookup
    H, V = 56, 203
    norm, t = make_part("norm", "rmsnorm", dtype, dict(weight="w"), dict(size=H, eps=1e-4))
    res, delta = torch.randn(5, H), torch.randn(5, H)
    r = res.cuda()
    out = norm.forward(None, r, delta.cuda()).cpu()
    assert torch.allclose(r.cpu(), res + delta, atol=1e-6)
    with plain.stores_rounded_to(dtype):
        assert float(rel_rows(out, plain.rmsnorm_stored(res + delta, t["w"], 1e-4)).max()) < TOL[dtype]
    emb, te = make_part("embedding", "embedding", dtype, dict(weight="e"), dict(vocab_size=V, hidden_size=H))
    head, th = make_part("head", "linear_head", dtype, dict(weight="h"), dict(vocab_size=V, hidden_size=H, tied=False))
    x = torch.randn(4, H).to(dtype)
    logits = head.forward(None, x.cuda()).cpu()
    assert logits.dtype == torch.float32 and logits.shape == (4, V)
    assert float(rel_rows(logits, x.float() @ th["h"].T).max()) < 1e-5     # float accumulation, float output
    rope = lookup("position", "rope")(head_dim=32, theta=777.0, rot_dim=16)
    inv, rot = rope.rotary("cuda")
    assert rot == 16 and torch.allclose(inv.cpu(), 1.0 / (777.0 ** (torch.arange(0, 16, 2).float() / 16)))
    assert lookup("position", "none")().rotary("cuda") == (None, 0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_arrangement(dtype):
    """x += mixer(norm(x)); x += ffn(norm(x)) with the sums carried in float."""
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.parts.registry import lookup
    H, L = 64, 3
    mixer, tm = make_part("mixer", "short_conv", dtype, dict(in_proj="in", conv="conv", out_proj="out"),
                          dict(hidden_size=H, kernel_size=L), seed=1)
    ffn, tf = make_part("ffn", "swiglu", dtype, dict(gate="g", up="u", down="d"),
                        dict(hidden_size=H, intermediate_size=96), seed=2)
    n1, t1 = make_part("norm", "rmsnorm", dtype, dict(weight="w"), dict(size=H, eps=1e-5), seed=3)
    n2, t2 = make_part("norm", "rmsnorm", dtype, dict(weight="w"), dict(size=H, eps=1e-5), seed=4)
    block = lookup("block", "prenorm")(mixer, ffn, n1, n2)
    cache = CacheManager({0: mixer.cache_spec()}, 16, 4, 1, dtype, "cuda")
    rc = cache.admit()
    ctx = make_ctx(cache, [(rc, [0] * 12)], dtype)
    x0, d0 = torch.randn(12, H), torch.randn(12, H)
    residual = x0.cuda()
    delta = block.forward(ctx, residual, d0.cuda(), cache.view(0, ctx.block_tables), True).cpu()
    x = x0 + d0
    with plain.stores_rounded_to(dtype):
        x = x + plain.short_conv_mixer(plain.rmsnorm_stored(x, t1["w"], 1e-5), tm["in"], tm["conv"].reshape(H, L),
                                       tm["out"])
        want_delta = plain.dense_ffn(plain.rmsnorm_stored(x, t2["w"], 1e-5), tf["g"], tf["u"], tf["d"])
    assert float(rel_rows(residual.cpu(), x).max()) < TOL[dtype]
    assert float(rel_rows(delta, want_delta).max()) < TOL[dtype] * 3
