"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same op, at sizes other
than the engine's tiny models use (head sizes in steps of 16, odd head counts and groups, widths
and vocabularies that are no power of two), in float32 and in bfloat16."""
import math

import pytest
import torch
import torch.nn.functional as F

import plain_lfm2 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
ATOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def K():
    from snowllm_b200.ops import kernels
    assert torch.cuda.is_available(), "the gpu tests need a CUDA device"
    return kernels


def dev(t, dtype=None):
    t = t.cuda()
    return t.to(dtype) if dtype is not None else t


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def close(got, want, dtype, scale=1.0):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs().max().item()
    bound = ATOL[dtype] * scale * max(1.0, want.abs().max().item())
    assert err <= bound, f"max abs error {err} > {bound}"


def rnd(dtype, *shape, scale=1.0):
    """Random values that the dtype holds exactly, as float32 on the CPU."""
    return (torch.randn(*shape) * scale).to(dtype).float()


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,M", [(331, 80, 7), (1000, 2048, 3)])
def test_embedding(K, dtype, V, H, M):
    torch.manual_seed(0)
    table = rnd(dtype, V, H)
    ids = torch.randint(0, V, (M,))
    out = K.embedding(i32(ids.tolist()), dev(table, dtype))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table[ids])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [80, 96, 2048, 5000])
def test_add_rmsnorm(K, dtype, H):
    torch.manual_seed(1)
    M, eps = 9, 1e-5
    res, delta = torch.randn(M, H), torch.randn(M, H)
    for gamma_f32 in (False, True):
        g = rnd(dtype, H) + 1.0 if not gamma_f32 else torch.randn(H) + 1.0
        r = dev(res.clone())
        out = K.add_rmsnorm(r, dev(delta), dev(g, None if gamma_f32 else dtype), eps, dtype)
        assert torch.allclose(r.cpu(), res + delta, atol=1e-6)           # the residual sum is float
        close(out, plain.rmsnorm(res + delta, g, eps), dtype)
    # rows: only those rows, residual untouched
    rows = [5, 0, 5, 8]
    r = dev(res.clone())
    g = rnd(dtype, H) + 1.0
    out = K.add_rmsnorm(r, dev(delta), dev(g, dtype), eps, dtype, rows=i32(rows))
    assert torch.equal(r.cpu(), res)
    close(out, plain.rmsnorm((res + delta)[rows], g, eps), dtype)
    out = K.add_rmsnorm(r, None, dev(g, dtype), eps, dtype)
    close(out, plain.rmsnorm(res, g, eps), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(K, dtype):
    torch.manual_seed(2)
    gu = rnd(dtype, 11, 2 * 56, scale=2.0)
    out = K.swiglu(dev(gu, dtype))
    close(out, F.silu(gu[:, :56]) * gu[:, 56:], dtype)


# ---------------------------------------------------------------------------------------------
def make_pool(dtype, pages, nkv, P, hd):
    return torch.zeros(pages, 2, nkv, P, hd, dtype=dtype, device="cuda")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot", [(5, 5, 48, 48), (6, 2, 80, 80), (3, 1, 128, 64), (2, 1, 16, 16),
                                           (7, 2, 64, 64), (4, 2, 128, 128), (3, 1, 256, 256), (9, 3, 32, 32)])
def test_qk_norm_rope_cache(K, dtype, nh, nkv, hd, rot):
    torch.manual_seed(3)
    P, pages, eps, theta = 8, 16, 1e-6, 1234.5
    # two segments at odd positions, pages given out of order
    seg_pos = [list(range(13, 13 + 9)), list(range(0, 5))]
    tables = [[7, 3, 11, 0], [5, 0, 0, 0]]
    positions = sum(seg_pos, [])
    row_seg = [0] * 9 + [1] * 5
    M = len(positions)
    qkv = rnd(dtype, M, (nh + 2 * nkv) * hd)
    qg, kg = rnd(dtype, hd) + 1.0, rnd(dtype, hd) + 1.0
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    pool = make_pool(dtype, pages, nkv, P, hd)
    q = K.qk_norm_rope_cache(dev(qkv, dtype), dev(qg, dtype), dev(kg, dtype), eps, dev(inv_freq), rot,
                             i32(positions), i32(row_seg), i32(tables), P, pool, nh, nkv, hd)
    x = qkv.view(M, nh + 2 * nkv, hd)
    ang = torch.tensor(positions, dtype=torch.float32)[:, None] * inv_freq[None]

    def rope(t):
        out = t.clone()
        out[..., :rot] = plain.apply_rope(t[..., :rot], ang)
        return out
    want_q = rope(plain.rmsnorm(x[:, :nh], qg, eps))
    want_k = rope(plain.rmsnorm(x[:, nh:nh + nkv], kg, eps))
    want_v = x[:, nh + nkv:]
    close(q, want_q, dtype, scale=2)
    for m, (pos, seg) in enumerate(zip(positions, row_seg)):
        page, off = tables[seg][pos // P], pos % P
        close(pool[page, 0, :, off], want_k[m], dtype, scale=2)
        close(pool[page, 1, :, off], want_v[m], dtype)
    untouched = sorted(set(range(pages)) - {3, 11, 5})          # page 7 holds positions 0..7: not in this step
    assert float(pool[untouched].abs().max()) == 0.0            # nothing written elsewhere
    assert float(pool[3, :, :, :5].abs().max()) == 0.0          # page 3 holds 8..15: only 13, 14, 15 written
    assert float(pool[11, :, :, 6:].abs().max()) == 0.0         # page 11 holds 16..23: only 16..21 written
    assert float(pool[5, :, :, 5:].abs().max()) == 0.0          # second segment: positions 0..4


def test_qk_norm_rope_without_norm_or_rope_and_q_only(K):
    dtype = torch.float32
    nh, nkv, hd, P = 2, 1, 32, 4
    qkv = rnd(dtype, 3, (nh + 2 * nkv) * hd)
    pool = make_pool(dtype, 2, nkv, P, hd)
    q = K.qk_norm_rope_cache(dev(qkv), None, None, 0.0, None, 0, i32([0, 1, 2]), i32([0, 0, 0]), i32([[1]]),
                             P, pool, nh, nkv, hd)
    assert torch.equal(q.cpu().reshape(3, -1), qkv[:, :nh * hd])
    assert torch.equal(pool[1, 0, 0, :3].cpu(), qkv[:, nh * hd:(nh + 1) * hd])
    before = pool.clone()
    q2 = K.qk_norm_rope_cache(dev(qkv[:, :nh * hd].contiguous()), None, None, 0.0, None, 0, i32([0, 1, 2]),
                              i32([0, 0, 0]), i32([[1]]), P, pool, nh, nkv, hd, write_kv=False)
    assert torch.equal(q2.cpu(), q.cpu()) and torch.equal(pool, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(7, 2, 64), (5, 5, 48)])
def test_qk_norm_rope_rows_do_not_depend_on_the_batch(K, dtype, nh, nkv, hd):
    """A portion of 90 rows (one block per row) and the same rows three at a time (a row's heads spread over
    blocks) give the same bits: q, and the keys and values in the pages."""
    torch.manual_seed(4)
    M, P, eps = 90, 16, 1e-5
    qkv = dev(rnd(dtype, M, (nh + 2 * nkv) * hd), dtype)
    qg, kg = dev(rnd(dtype, hd) + 1.0, dtype), dev(rnd(dtype, hd) + 1.0, dtype)
    inv_freq = dev(1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)))
    positions = list(range(1000, 1000 + M))
    pages = (1000 + M) // P + 1
    table = i32([list(range(pages))[::-1]])
    pool_a, pool_b = make_pool(dtype, pages, nkv, P, hd), make_pool(dtype, pages, nkv, P, hd)
    seg = i32([0] * M)
    qa = K.qk_norm_rope_cache(qkv, qg, kg, eps, inv_freq, hd, i32(positions), seg, table, P, pool_a, nh, nkv, hd)
    qb = torch.cat([K.qk_norm_rope_cache(qkv[i:i + 3].contiguous(), qg, kg, eps, inv_freq, hd, i32(positions[i:i + 3]),
                                         i32([0] * 3), table, P, pool_b, nh, nkv, hd) for i in range(0, M, 3)])
    assert torch.equal(qa, qb) and torch.equal(pool_a, pool_b)


# ---------------------------------------------------------------------------------------------
def ref_attention(q, k, v, positions, scale, window):
    """q [M, nh, hd] against full k, v [T, nkv, hd] of one request; row m sees keys <= positions[m]."""
    M, nh, hd = q.shape
    T, nkv, _ = k.shape
    out = torch.zeros(M, nh, hd, dtype=torch.float64)
    for m in range(M):
        lo = 0 if not window else max(0, positions[m] - window + 1)
        for h in range(nh):
            g = h // (nh // nkv)
            s = (k[lo:positions[m] + 1, g].double() @ q[m, h].double()) * scale
            out[m, h] = torch.softmax(s, 0) @ v[lo:positions[m] + 1, g].double()
    return out.float().reshape(M, nh * hd)


def scatter_kv(pool, k, v, table, P):
    for t in range(k.shape[0]):
        pool[table[t // P], 0, :, t % P] = k[t].to(pool.dtype).cuda()
        pool[table[t // P], 1, :, t % P] = v[t].to(pool.dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 2, 16, 16, None), (6, 2, 48, 8, None), (3, 3, 80, 64, None),
                                                (16, 1, 128, 16, None), (10, 1, 32, 16, None),
                                                (4, 2, 64, 16, 37), (4, 4, 16, 4, 5)])
def test_paged_attention_mixed_rows(K, dtype, nh, nkv, hd, P, window):
    """A prompt portion in the middle of one request beside single rows of two others, pages
    scattered and shared out of order, one chunk and many chunks."""
    torch.manual_seed(4)
    lens = [150, 33, 700]
    rows = [list(range(90, 150)), [32], [699]]
    pages = sum(-(-n // P) for n in lens) + 3
    perm = torch.randperm(pages).tolist()
    pool = torch.full((pages, 2, nkv, P, hd), float("nan"), dtype=dtype, device="cuda")  # unwritten = NaN
    tables, ks, vs = [], [], []
    for n in lens:
        need = -(-n // P)
        table, perm = perm[:need], perm[need:]
        k, v = rnd(dtype, n, nkv, hd), rnd(dtype, n, nkv, hd)
        scatter_kv(pool, k, v, table, P)
        tables.append(table)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    positions = sum(rows, [])
    row_seg = sum(([b] * len(r) for b, r in enumerate(rows)), [])
    M = len(positions)
    q = rnd(dtype, M, nh, hd)
    scale = hd ** -0.5
    want = torch.cat([ref_attention(q[[i for i, s in enumerate(row_seg) if s == b]], ks[b], vs[b], rows[b],
                                    scale, window) for b in range(3)])
    for chunk, n_chunks in ((None, 1), (64, None), (256, None)):
        if chunk is not None:
            lo = [0 if not window else max(0, p - window + 1) for p in positions]
            n_chunks = max(p // chunk - l // chunk for p, l in zip(positions, lo)) + 1
        out = K.paged_attention(dev(q, dtype), pool, bt, P, i32(positions), i32(row_seg), scale, window=window,
                                chunk=chunk, num_chunks=n_chunks)
        assert out.isfinite().all(), "an unwritten (NaN) cache entry was read"
        close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(K, dtype):
    """One key far back is made to stand out (query and key scaled along one direction): the
    output must be that key's value, whatever page it lies on and however the keys are chunked."""
    torch.manual_seed(5)
    nh, nkv, hd, P, T = 2, 1, 64, 16, 900
    for far in (0, 15, 16, 255, 256, 511, 640, 899):
        k, v = rnd(dtype, T, nkv, hd, scale=0.1), rnd(dtype, T, nkv, hd)
        direction = F.normalize(torch.randn(hd), dim=0)
        k[far, 0] = (direction * 16).to(dtype).float()
        q = (direction * 16).to(dtype).float().expand(1, nh, hd).contiguous()
        table = torch.randperm(-(-T // P)).tolist()
        pool = make_pool(dtype, len(table), nkv, P, hd)
        scatter_kv(pool, k, v, table, P)
        for chunk, n in ((None, 1), (256, 4)):
            out = K.paged_attention(dev(q, dtype), pool, i32([table]), P, i32([T - 1]), i32([0]), hd ** -0.5,
                                    chunk=chunk, num_chunks=n)
            want = v[far, 0].repeat(nh)
            assert (out.float().cpu()[0] - want).abs().max() < 0.02, (far, chunk)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(K, dtype):
    """The key just outside the window is huge and must not be seen; the one just inside must win."""
    torch.manual_seed(6)
    nh, nkv, hd, P, T, W = 2, 2, 32, 8, 300, 100
    pos = T - 1
    direction = F.normalize(torch.randn(hd), dim=0)
    q = (direction * 12).to(dtype).float().expand(1, nh, hd).contiguous()
    for which, expect in ((pos - W, "ignored"), (pos - W + 1, "wins")):
        k, v = rnd(dtype, T, nkv, hd, scale=0.1), rnd(dtype, T, nkv, hd)
        k[which] = (direction * 20).to(dtype).float()
        table = list(range(-(-T // P)))
        pool = make_pool(dtype, len(table), nkv, P, hd)
        scatter_kv(pool, k, v, table, P)
        for chunk, n in ((None, 1), (64, 3)):
            out = K.paged_attention(dev(q, dtype), pool, i32([table]), P, i32([pos]), i32([0]), hd ** -0.5,
                                    window=W, chunk=chunk, num_chunks=n).float().cpu()[0]
            hit = (out - v[which].reshape(-1)).abs().max().item()
            assert (hit < 0.02) == (expect == "wins"), (which, expect, hit)
            close(out[None], ref_attention(q, k, v, [pos], hd ** -0.5, W), dtype)


# ---------------------------------------------------------------------------------------------
def ref_conv(bcx, w, hist):
    """bcx [T, 3H] of one request with history hist [L-1, H]; returns (y, new history)."""
    H = w.shape[0]
    L = w.shape[1]
    B, C, x = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    g = torch.cat((hist, B * x))
    conv = torch.stack([sum(w[:, j] * g[t + j] for j in range(L)) for t in range(bcx.shape[0])])
    return C * conv, g[g.shape[0] - (L - 1):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,L", [(80, 3), (2048, 3), (96, 4), (40, 2), (33, 7)])
def test_short_conv_whole_chunked_and_state(K, dtype, H, L):
    torch.manual_seed(7)
    lens, slots = [11, 1, 30], [2, 0, 3]
    n_slots = 5
    bcx = [rnd(dtype, n, 3 * H, scale=0.5) for n in lens]
    w = rnd(dtype, H, L, scale=0.5)
    state = torch.full((n_slots, L - 1, H), float("nan"), dtype=dtype, device="cuda")   # stale slots
    cu = [0, 11, 12, 42]
    row_seg = sum(([b] * n for b, n in enumerate(lens)), [])
    out = K.short_conv(dev(torch.cat(bcx), dtype), dev(w, dtype), state, i32(cu), i32([0, 0, 0]), i32(slots),
                       i32(row_seg))
    assert out.isfinite().all(), "a fresh request read its slot's old contents"
    refs = [ref_conv(b, w, torch.zeros(L - 1, H)) for b in bcx]
    close(out, torch.cat([r[0] for r in refs]), dtype)
    for b, s in enumerate(slots):
        if dtype == torch.float32:
            assert torch.equal(state[s].cpu(), refs[b][1])
        else:   # the state holds round(B*x): exactly representable products of two bfloat16 are rounded once
            assert torch.equal(state[s].float().cpu(), refs[b][1].to(dtype).float())
    assert state[[1, 4]].isnan().all()                                         # other slots untouched
    # the same sequences in portions (with other cuts per request): bit-identical outputs and state
    state2 = torch.full_like(state, float("nan"))
    done = [0, 0, 0]
    got = [[], [], []]
    cuts = [[1, 3, 7], [1], [2, 2, 1, 25]]
    for step in range(4):
        seg = [(b, cuts[b][step]) for b in range(3) if step < len(cuts[b])]
        rows = torch.cat([bcx[b][done[b]:done[b] + n] for b, n in seg])
        cu2 = [0]
        for _, n in seg:
            cu2.append(cu2[-1] + n)
        o = K.short_conv(dev(rows, dtype), dev(w, dtype), state2, i32(cu2), i32([done[b] for b, _ in seg]),
                         i32([slots[b] for b, _ in seg]),
                         i32(sum(([i] * n for i, (_, n) in enumerate(seg)), [])))
        for i, (b, n) in enumerate(seg):
            got[b].append(o[cu2[i]:cu2[i + 1]])
            done[b] += n
    assert done == lens
    assert torch.equal(torch.cat([torch.cat(g) for g in got]), out), "portions differ from the whole"
    assert torch.equal(state2[slots], state[slots])


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 331, 80), (7, 96, 48), (65, 130, 2048), (200, 64, 24), (5, 17, 13)])
def test_gemm(K, dtype, M, N, K_):
    torch.manual_seed(8)
    a, w = rnd(dtype, M, K_), rnd(dtype, N, K_)
    want = a @ w.T
    close(K.gemm_simt(dev(a, dtype), dev(w, dtype)), want, dtype, scale=math.sqrt(K_) / 4)
    out32 = K.gemm_simt(dev(a, dtype), dev(w, dtype), out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    close(out32, want, torch.float32, scale=math.sqrt(K_))


def test_gemm_rows_do_not_depend_on_the_batch(K):
    """A row's result is the same bits alone, among others, and at another place in the batch."""
    torch.manual_seed(9)
    for dtype in DTYPES:
        a, w = dev(rnd(dtype, 150, 96), dtype), dev(rnd(dtype, 77, 96), dtype)
        whole = K.gemm_simt(a, w, out_dtype=torch.float32)
        assert torch.equal(K.gemm_simt(a[70:71].contiguous(), w, out_dtype=torch.float32), whole[70:71])
        assert torch.equal(K.gemm_simt(a[3:140].contiguous(), w, out_dtype=torch.float32), whole[3:140])


@pytest.mark.parametrize("dtype", DTYPES)
def test_grouped_gemm_with_gather(K, dtype):
    torch.manual_seed(10)
    E, N, K_, M, k = 5, 50, 40, 23, 2
    x, w = rnd(dtype, M, K_), rnd(dtype, E, N, K_)
    counts = [7, 0, 20, 1, 18]                       # an expert without rows, one with a single row
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    pairs = torch.randperm(M * k).tolist()            # sorted row r holds pair pairs[r] of token pairs[r] // k
    out = K.gemm_simt(dev(x, dtype), dev(w, dtype), a_rows=i32(pairs), a_div=k, offsets=i32(offsets),
                      rows_out=M * k, max_rows_per_group=M, out_dtype=torch.float32)
    for e in range(E):
        for r in range(offsets[e], offsets[e + 1]):
            want = x[pairs[r] // k] @ w[e].T
            close(out[r], want, dtype, scale=2)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,H,norm,use_bias,scaling", [(8, 2, 64, True, True, 1.0), (16, 4, 96, False, False, 2.0),
                                                         (5, 3, 80, True, True, 0.5), (40, 6, 2048, True, False, 1.0),
                                                         (7, 7, 48, False, True, 1.5)])
def test_moe_route(K, dtype, E, k, H, norm, use_bias, scaling):
    torch.manual_seed(11)
    M = 50
    x = rnd(dtype, M, H)
    wr = rnd(dtype, E, H, scale=H ** -0.5)
    bias = torch.randn(E) * 0.1 if use_bias else None
    ids, wts = K.moe_route(dev(x, dtype), dev(wr, dtype), dev(bias) if use_bias else None, k, norm, scaling)
    margins = []
    want_ids, want_w = plain.route(x, wr, bias, k, norm, scaling, margins=margins)
    clear = margins[0] > 1e-5                        # rows whose selection no rounding can change
    assert clear.float().mean() > 0.9
    assert torch.equal(ids.cpu().long()[clear], want_ids[clear])
    assert torch.allclose(wts.cpu()[clear], want_w[clear], atol=2e-6, rtol=1e-5)
    # float32 router weights with bfloat16 activations give the same
    ids2, _ = K.moe_route(dev(x, dtype), dev(wr), dev(bias) if use_bias else None, k, norm, scaling)
    assert torch.equal(ids2.cpu()[clear], ids.cpu()[clear])
    if dtype == torch.bfloat16 and H % 8 == 0:      # many rows: logits by the tensor-core product
        xm = rnd(dtype, 300, H)
        ids3, w3 = K.moe_route(dev(xm, dtype), dev(wr, dtype), dev(bias) if use_bias else None, k, norm, scaling)
        mg = []
        want3, ww3 = plain.route(xm, wr, bias, k, norm, scaling, margins=mg)
        ok = mg[0] > 1e-4
        assert ok.float().mean() > 0.9 and torch.equal(ids3.cpu().long()[ok], want3[ok])
        assert torch.allclose(w3.cpu()[ok], ww3[ok], atol=1e-5, rtol=1e-4)


def test_moe_route_ties_go_to_the_lower_index_and_bias_only_selects(K):
    x = torch.zeros(2, 32, device="cuda")
    wr = torch.zeros(6, 32, device="cuda")
    ids, wts = K.moe_route(x, wr, None, 3, True, 1.0)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 2
    assert torch.allclose(wts.cpu(), torch.full((2, 3), 0.5 / (1.5 + 1e-6)))
    bias = torch.tensor([0.0, 0.3, 0.0, 0.3, 0.0, 0.1], device="cuda")
    ids, wts = K.moe_route(x, wr, bias, 3, False, 2.0)
    assert ids.cpu().tolist() == [[1, 3, 5]] * 2 and torch.allclose(wts.cpu(), torch.full((2, 3), 1.0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,E,k,H", [(1, 8, 2, 64), (8, 32, 4, 2048), (13, 5, 3, 80), (32, 40, 6, 104), (9, 7, 7, 50)])
def test_moe_route_sort_few_rows_is_the_same_routing_and_a_valid_sort(K, dtype, M, E, k, H):
    torch.manual_seed(13)
    x, wr = dev(rnd(dtype, M, H), dtype), dev(rnd(dtype, E, H, scale=H ** -0.5), dtype)
    bias = dev(torch.randn(E) * 0.1)
    ids, wts, offsets, pair_pos, sorted_pair = K.moe_route_sort(x, wr, bias, k, True, 1.5)
    # bit for bit what the one-block-per-token kernel selects: a token's routing does not depend on the path
    big_x = torch.cat([x, dev(rnd(dtype, 64 - M, H), dtype)])        # more rows than the few-rows path takes
    ids2, wts2 = K.moe_route(big_x, wr, bias, k, True, 1.5)
    assert torch.equal(ids, ids2[:M]) and torch.equal(wts, wts2[:M])
    ids3, wts3, *_ = K.moe_route_sort(big_x, wr, bias, k, True, 1.5)
    assert torch.equal(ids3, ids2) and torch.equal(wts3, wts2)
    flat = ids.cpu().reshape(-1).long()
    offsets, pair_pos, sorted_pair = offsets.cpu(), pair_pos.cpu(), sorted_pair.cpu()
    assert offsets[0] == 0 and offsets[-1] == M * k
    assert torch.equal(offsets[1:] - offsets[:-1], torch.bincount(flat, minlength=E).int())
    assert sorted(sorted_pair.tolist()) == list(range(M * k))
    for p_ in range(M * k):
        r = int(pair_pos[p_])
        assert int(sorted_pair[r]) == p_ and offsets[flat[p_]] <= r < offsets[flat[p_] + 1]


def test_moe_sort_and_combine(K):
    torch.manual_seed(12)
    M, k, E, H = 37, 3, 9, 70
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(M)]).int()
    ids[:, 0] = torch.where(torch.rand(M) < 0.3, torch.tensor(8), ids[:, 0].long()).int()   # crowd one expert
    for m in range(M):                                # keep a token's experts distinct
        seen = set()
        for j in range(k):
            while int(ids[m, j]) in seen:
                ids[m, j] = (int(ids[m, j]) + 1) % E
            seen.add(int(ids[m, j]))
    offsets, pair_pos, sorted_pair = K.moe_sort(ids.cuda(), E)
    offsets, pair_pos, sorted_pair = offsets.cpu(), pair_pos.cpu(), sorted_pair.cpu()
    flat = ids.reshape(-1)
    assert offsets[0] == 0 and offsets[-1] == M * k
    assert torch.equal(offsets[1:] - offsets[:-1], torch.bincount(flat, minlength=E).int())
    assert sorted(sorted_pair.tolist()) == list(range(M * k))
    for p in range(M * k):
        r = int(pair_pos[p])
        assert int(sorted_pair[r]) == p and offsets[flat[p]] <= r < offsets[flat[p] + 1]
    y, w = torch.randn(M * k, H), torch.rand(M, k)
    out = K.moe_combine(y.cuda(), pair_pos.cuda(), w.cuda())
    want = torch.stack([sum(w[m, j] * y[pair_pos[m * k + j]] for j in range(k)) for m in range(M)])
    assert torch.allclose(out.cpu(), want, atol=1e-5)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("V", [31, 256, 4097, 65536, 100003])
def test_argmax(K, V):
    """NaN counts as -inf, ties give the lowest index (tests/test_sampling_argmax.py:13-44 in SnowLLM)."""
    torch.manual_seed(13)
    x = torch.randn(6, V)
    x[1, V // 2] = x[1, V - 1] = 50.0              # a tie: the lower index wins
    x[2, 3] = float("nan")
    x[2, V - 2] = 60.0
    x[3] = float("nan")                             # every value NaN
    x[4] = float("-inf")
    x[5, 0] = float("inf")
    out = K.argmax(x.cuda()).cpu()
    want = torch.argmax(torch.nan_to_num(x, nan=float("-inf")), dim=-1)
    assert out.tolist() == want.tolist()
    assert out[1] == V // 2 and out[3] == 0 and out[4] == 0


def test_penalties_and_bans(K):
    V = 50
    logits = torch.arange(V, dtype=torch.float32).repeat(3, 1) - 20.0
    before = logits.clone()
    ids = [3, 30, 45, 10, 25]                       # row 0: three seen tokens; row 1: none; row 2: ban + one seen
    counts = [0, 2, 1, -1, 3]
    K.apply_penalties(x := logits.cuda(), i32([0, 3, 3, 5]), i32(ids), i32(counts),
                      torch.tensor([0.5, 0.0, 0.0]).cuda(), torch.tensor([0.25, 0.0, 1.0]).cuda(),
                      torch.tensor([2.0, 1.0, 1.0]).cuda())
    got = x.cpu()
    want = before.clone()
    want[0, 3] = before[0, 3] * 2.0                 # negative: times r; count 0: no presence, no frequency
    want[0, 30] = before[0, 30] / 2.0 - 0.25 * 2 - 0.5
    want[0, 45] = before[0, 45] / 2.0 - 0.25 - 0.5
    want[2, 10] = float("-inf")
    want[2, 25] = before[2, 25] - 3.0
    assert torch.equal(got, want)


def test_sample_matches_the_reference_draw(K):
    torch.manual_seed(14)
    V, B = 997, 64
    logits = torch.randn(B, V) * 3
    temperature = torch.rand(B) * 1.5 + 0.2
    top_k = torch.tensor([0, 1, 5, 50, 996, 997, 2000, 17] * 8, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 0.5, 0.99, 0.1, 1.0, 0.7, 0.3] * 8).roll(3)
    uniform = torch.rand(B)
    uniform[:4] = torch.tensor([0.0, 0.999999, 0.5, 1e-7])
    temperature[8] = 0.0                            # a greedy row among the others
    out = K.sample(logits.cuda(), temperature.cuda(), top_k.cuda(), top_p.cuda(), uniform.cuda()).cpu()
    miss = 0
    for b in range(B):
        if temperature[b] <= 0:
            assert out[b] == logits[b].argmax()
            continue
        want = plain.softmax_sample_reference(logits[b], float(temperature[b]), int(top_k[b]), float(top_p[b]),
                                              float(uniform[b]))
        # float32 against float64 sums may put the draw on the other side of a CDF step: a neighbour
        if out[b] != want:
            p = torch.softmax(logits[b].double() / float(temperature[b]), -1)
            c = torch.cumsum(p, 0)
            assert abs(float(c[min(out[b], want)]) - float(uniform[b])) < 1e-3 or p[out[b]] > 0, b
            miss += 1
    assert miss <= 3


def test_sample_respects_top_k_and_top_p_sets(K):
    torch.manual_seed(15)
    V = 300
    logits = torch.randn(1, V).repeat(400, 1) * 2
    for top_k, top_p in ((5, 1.0), (0, 0.6), (20, 0.8)):
        out = K.sample(logits.cuda(), torch.ones(400).cuda(), torch.full((400,), top_k, dtype=torch.int32).cuda(),
                       torch.full((400,), top_p).cuda(), torch.rand(400).cuda()).cpu()
        p = torch.softmax(logits[0].double(), -1)
        order = torch.argsort(p, descending=True)
        allowed = set(order[:top_k].tolist()) if top_k else set(range(V))
        if top_p < 1:
            kept = order[:top_k] if top_k else order
            c = torch.cumsum(p[kept], 0)
            n = int((c < top_p * c[-1]).sum()) + 1
            allowed &= set(kept[:n].tolist())
        assert set(out.tolist()) <= allowed
        assert len(set(out.tolist())) > 1


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K_", [(1, 331, 80), (8, 96, 48), (9, 2048, 2048), (33, 130, 264), (64, 17, 8),
                                    (5, 64, 7168), (3, 40003, 72), (17, 32768, 264)])
def test_gemm_skinny(K, M, N, K_):
    """The few-rows bfloat16 kernel against the float product, and row by row against itself."""
    torch.manual_seed(20)
    dtype = torch.bfloat16
    a, w = rnd(dtype, M, K_), rnd(dtype, N, K_)
    want = a @ w.T
    out = K.gemm_skinny(dev(a, dtype), dev(w, dtype), out_dtype=torch.float32)
    close(out, want, torch.float32, scale=math.sqrt(K_))
    close(K.gemm_skinny(dev(a, dtype), dev(w, dtype)), want, dtype, scale=math.sqrt(K_) / 4)
    for m in (0, M - 1):       # a row alone gives the same bits as among the others
        alone = K.gemm_skinny(dev(a[m:m + 1], dtype), dev(w, dtype), out_dtype=torch.float32)
        assert torch.equal(alone, out[m:m + 1])


def test_gemm_skinny_grouped_with_gather(K):
    torch.manual_seed(21)
    dtype = torch.bfloat16
    E, N, K_, M, k = 5, 50, 40, 40, 2
    x, w = rnd(dtype, M, K_), rnd(dtype, E, N, K_)
    counts = [7, 0, 38, 1, 34]                        # more rows than one pass holds, none, one
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    pairs = torch.randperm(M * k).tolist()
    for hint in (8, 16, 64):
        out = K.gemm_skinny(dev(x, dtype), dev(w, dtype), a_rows=i32(pairs), a_div=k, offsets=i32(offsets),
                            rows_out=M * k, rows_hint=hint, out_dtype=torch.float32)
        for e in range(E):
            for r in range(offsets[e], offsets[e + 1]):
                close(out[r], x[pairs[r] // k] @ w[e].T, torch.float32, scale=8)
    # many groups
    E, N, M = 64, 520, 70
    x, w = rnd(dtype, M, K_), rnd(dtype, E, N, K_)
    ids = torch.randint(0, E, (M,))
    order = torch.argsort(ids, stable=True)
    offsets = [0] + torch.cumsum(torch.bincount(ids, minlength=E), 0).tolist()
    out = K.gemm_skinny(dev(x, dtype), dev(w, dtype), a_rows=i32(order.tolist()), a_div=1, offsets=i32(offsets),
                        rows_out=M, rows_hint=8, out_dtype=torch.float32)
    for r in range(M):
        close(out[r], x[order[r]] @ w[ids[order[r]]].T, torch.float32, scale=8)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (65, 17, 8), (200, 136, 72), (300, 100, 1000), (257, 384, 2048),
                                    (64, 2048, 2048), (40, 6144, 2048), (100, 256, 1800), (17, 128, 328),   # few tiles: split along K
                                    (1000, 96, 48), (2000, 4000, 72), (1930, 4104, 136)])   # the last two: 256-wide tiles
def test_gemm_tc(K, M, N, K_):
    """The tcgen05 kernel (TMA loads, accumulator in tensor memory) against the float product: tiles
    cut by M, N and K, float and bfloat16 stores; no wait inside the kernel ran out."""
    torch.manual_seed(30)
    dtype = torch.bfloat16
    a, w = rnd(dtype, M, K_), rnd(dtype, N, K_)
    want = a @ w.T
    out = K.gemm_tc(dev(a, dtype), dev(w, dtype), out_dtype=torch.float32)
    close(out, want, torch.float32, scale=math.sqrt(K_))
    close(K.gemm_tc(dev(a, dtype), dev(w, dtype)), want, dtype, scale=math.sqrt(K_) / 4)
    assert K.gemm_tc_status() == 0
    # a row's result does not depend on the rows around it: not by a bit while the product keeps its form
    # (whole, or split along K the same way), by rounding otherwise
    rows = slice(3, min(70, M))
    part = K.gemm_tc(dev(a[rows], dtype), dev(w, dtype), out_dtype=torch.float32)
    if not K.gemm_tc_is_split(M, N, K_) and not K.gemm_tc_is_split(rows.stop - rows.start, N, K_):
        assert torch.equal(part, out[rows])
    else:
        assert torch.allclose(part, out[rows], rtol=1e-5, atol=1e-5 * math.sqrt(K_))


@pytest.mark.parametrize("M,N,K_", [(256, 256, 64), (300, 520, 200), (1000, 96, 48), (2000, 4000, 72), (513, 264, 2048)])
def test_gemm_tc2_pairs_of_sms(K, M, N, K_):
    """The product on pairs of SMs (cta_group::2) against the float product, to float and to bfloat16, with
    SwiGLU at the store, and grouped with ragged groups."""
    from snowllm_b200.ops import interleave_gate_up
    torch.manual_seed(33)
    dtype = torch.bfloat16
    a, w = rnd(dtype, M, K_), rnd(dtype, N, K_)
    want = a @ w.T
    close(K.gemm_tc2(dev(a, dtype), dev(w, dtype), out_dtype=torch.float32), want, torch.float32, scale=math.sqrt(K_))
    close(K.gemm_tc2(dev(a, dtype), dev(w, dtype)), want, dtype, scale=math.sqrt(K_) / 4)
    status, tmem = K.gemm_tc2_status()
    assert status == 0 and tmem[0] == tmem[1]            # the pair holds one accumulator address
    I = (N // 16) * 8
    if I:
        gate, up = rnd(dtype, I, K_, scale=K_ ** -0.5), rnd(dtype, I, K_, scale=K_ ** -0.5)
        act = K.gemm_tc2(dev(a, dtype), interleave_gate_up(dev(gate, dtype), dev(up, dtype)), swiglu=True)
        close(act, F.silu(a @ gate.T) * (a @ up.T), dtype, scale=2)
    counts = [M // 3, 0, 1, M - M // 3 - 1 - 257, 257]
    if min(counts) >= 0:
        offsets = [0]
        for c in counts:
            offsets.append(offsets[-1] + c)
        wg = rnd(dtype, len(counts), N, K_)
        out = K.gemm_tc2(dev(a, dtype), dev(wg, dtype), out_dtype=torch.float32, offsets=i32(offsets))
        for e, c in enumerate(counts):
            r = slice(offsets[e], offsets[e + 1])
            if c:
                close(out[r], a[r] @ wg[e].T, torch.float32, scale=math.sqrt(K_))
    assert K.gemm_tc2_status()[0] == 0


@pytest.mark.parametrize("N,K_", [(256, 64), (520, 200), (96, 2048), (1792, 72)])
def test_gemm_tc2_grouped_rows_on_the_n_side(K, N, K_):
    """The grouped product on pairs of SMs, where a group's rows are the N side of the MMA in steps of 16:
    groups of no, one, 16, 17, 255, 256, 257 and 530 rows; to float, to bfloat16 and with SwiGLU at the store."""
    from snowllm_b200.ops import interleave_gate_up
    torch.manual_seed(35)
    dtype = torch.bfloat16
    counts = [270, 0, 1, 16, 17, 255, 0, 256, 257, 530, 100, 31]
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    M, G = offsets[-1], len(counts)
    a, wg = rnd(dtype, M, K_), rnd(dtype, G, N, K_)
    want = torch.cat([a[offsets[e]:offsets[e + 1]] @ wg[e].T for e in range(G)])
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    K.gemm_tc2(dev(a, dtype), dev(wg, dtype), out_dtype=torch.float32, offsets=i32(offsets), out=out)
    assert K.gemm_tc2_status()[0] == 0
    close(out, want, torch.float32, scale=math.sqrt(K_))
    close(K.gemm_tc2(dev(a, dtype), dev(wg, dtype), offsets=i32(offsets)), want, dtype, scale=math.sqrt(K_) / 4)
    I = (N // 16) * 8
    gate, up = rnd(dtype, G, I, K_, scale=K_ ** -0.5), rnd(dtype, G, I, K_, scale=K_ ** -0.5)
    act = K.gemm_tc2(dev(a, dtype), interleave_gate_up(dev(gate, dtype), dev(up, dtype)), offsets=i32(offsets), swiglu=True)
    want_act = torch.cat([F.silu(a[offsets[e]:offsets[e + 1]] @ gate[e].T) * (a[offsets[e]:offsets[e + 1]] @ up[e].T)
                          for e in range(G)])
    close(act, want_act, dtype, scale=2)
    assert K.gemm_tc2_status()[0] == 0


def test_gemm_tc_grouped_after_gather(K):
    torch.manual_seed(31)
    dtype = torch.bfloat16
    E, N, K_, M, k = 5, 200, 192, 280, 2
    x, w = rnd(dtype, M, K_), rnd(dtype, E, N, K_)
    counts = [130, 0, 1, 300, 129]                    # more than one tile, none, one row, tile edge + 1
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    pairs = torch.randperm(M * k).tolist()
    xs = K.gather_rows(dev(x, dtype), i32(pairs), k)
    assert torch.equal(xs.float().cpu(), x[[p // k for p in pairs]])
    out = K.gemm_tc(xs, dev(w, dtype), out_dtype=torch.float32, offsets=i32(offsets))
    assert K.gemm_tc_status() == 0
    for e in range(E):
        r = slice(offsets[e], offsets[e + 1])
        if counts[e]:
            close(out[r], xs[r].float().cpu() @ w[e].T, torch.float32, scale=16)
    # enough tiles for the 256-wide form: many rows, several groups, N past a tile edge
    E, N, K_ = 6, 1100, 72
    counts = [700, 0, 1300, 129, 1, 870]
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    x, w = rnd(dtype, offsets[-1], K_), rnd(dtype, E, N, K_)
    out = K.gemm_tc(dev(x, dtype), dev(w, dtype), out_dtype=torch.float32, offsets=i32(offsets))
    assert K.gemm_tc_status() == 0
    for e in range(E):
        r = slice(offsets[e], offsets[e + 1])
        if counts[e]:
            close(out[r], x[r] @ w[e].T, torch.float32, scale=16)
    # the same groups through the store that applies SwiGLU, and to bfloat16 (tiles of 60, 20, 1 and 1 rows
    # are multiplied the other way round)
    from snowllm_b200.ops import interleave_gate_up
    I = 552
    gate, up = rnd(dtype, E, I, K_, scale=K_ ** -0.5), rnd(dtype, E, I, K_, scale=K_ ** -0.5)
    w13 = interleave_gate_up(dev(gate, dtype), dev(up, dtype))
    act = K.gemm_tc(dev(x, dtype), w13, offsets=i32(offsets), swiglu=True)
    half = K.gemm_tc(dev(x, dtype), dev(w, dtype), offsets=i32(offsets))
    assert K.gemm_tc_status() == 0 and act.shape == (offsets[-1], I)
    for e in range(E):
        r = slice(offsets[e], offsets[e + 1])
        if counts[e]:
            close(act[r], F.silu(x[r] @ gate[e].T) * (x[r] @ up[e].T), dtype, scale=4)
            close(half[r], x[r] @ w[e].T, dtype, scale=16)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 2, 64, 16, None), (6, 1, 128, 16, None), (2, 2, 64, 64, None),
                                                (4, 2, 64, 16, 100), (3, 1, 128, 8, 37), (2, 1, 64, 4, None),
                                                (2, 2, 64, 32, 70)])
def test_attention_prefill_tiles(K, nh, nkv, hd, P, window):
    """The tensor-core prompt kernel: a portion from position 0, one in the middle of a long request
    (not aligned to tiles or pages), a short one; pages scattered; unwritten cache entries are NaN."""
    from snowllm_b200.parts.attention_plan import prefill_tiles
    torch.manual_seed(40)
    dtype = torch.bfloat16
    starts, lens = [0, 333, 700], [200, 150, 17]
    totals = [s + n for s, n in zip(starts, lens)]
    pages = sum(-(-n // P) for n in totals) + 2
    perm = torch.randperm(pages).tolist()
    pool = torch.full((pages, 2, nkv, P, hd), float("nan"), dtype=dtype, device="cuda")
    tables, ks, vs = [], [], []
    for n in totals:
        need = -(-n // P)
        table, perm = perm[:need], perm[need:]
        k, v = rnd(dtype, n, nkv, hd), rnd(dtype, n, nkv, hd)
        scatter_kv(pool, k, v, table, P)
        tables.append(table)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    tiles, rest = prefill_tiles(starts, lens, 64)
    assert not rest and len(tiles) == 4 + 3 + 1
    M = sum(lens)
    q = rnd(dtype, M, nh, hd)
    out = torch.full((M, nh * hd), float("nan"), dtype=dtype, device="cuda")
    K.attention_prefill(dev(q, dtype), pool, bt, P, i32(tiles), hd ** -0.5, out, window=window)
    assert out.isfinite().all(), "a row was not written, or an unwritten cache entry was read"
    if K.prefill_tma_page_ok(P):                   # keys brought in by TMA or by 16-byte copies: the same bits
        by_copies = torch.full((M, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attention_prefill(dev(q, dtype), pool, bt, P, i32(tiles), hd ** -0.5, by_copies, window=window, tma=False)
        assert torch.equal(by_copies, out)
        assert K.attention_decode_status() == 0
    first = 0
    for b in range(3):
        rows = list(range(starts[b], totals[b]))
        want = ref_attention(q[first:first + lens[b]], ks[b], vs[b], rows, hd ** -0.5, window)
        close(out[first:first + lens[b]], want, dtype)
        first += lens[b]
    # the row-wise kernel on the same rows agrees (it serves the rows the tiles leave out)
    positions = sum((list(range(s, t)) for s, t in zip(starts, totals)), [])
    row_seg = sum(([b] * n for b, n in enumerate(lens)), [])
    some = [0, 5, 199, 200, 349, 350, 366]
    other = K.paged_attention(dev(q, dtype), pool, bt, P, i32(positions), i32(row_seg), hd ** -0.5, window=window,
                              out=torch.zeros_like(out), rows=i32(some))
    close(other[some], out[some].float(), dtype)
    untouched = [i for i in range(M) if i not in some]
    assert float(other[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("nh,nkv,P,window", [(4, 2, 16, None), (2, 2, 64, None), (4, 2, 16, 100), (3, 1, 8, 37),
                                             (2, 1, 128, None), (2, 2, 32, 170), (6, 3, 16, 300)])
def test_attention_prefill_tc_tiles(K, nh, nkv, P, window):
    """The tcgen05 prompt kernel (head size 64): a portion from position 0, one in the middle of a long request
    (not aligned to tiles or pages), a short one; pages scattered; unwritten cache entries are NaN."""
    from snowllm_b200.parts.attention_plan import prefill_tiles
    torch.manual_seed(42)
    dtype, hd = torch.bfloat16, 64
    starts, lens = [0, 333, 700], [300, 150, 17]
    totals = [s + n for s, n in zip(starts, lens)]
    pages = sum(-(-n // P) for n in totals) + 2
    perm = torch.randperm(pages).tolist()
    pool = torch.full((pages, 2, nkv, P, hd), float("nan"), dtype=dtype, device="cuda")
    tables, ks, vs = [], [], []
    for n in totals:
        need = -(-n // P)
        table, perm = perm[:need], perm[need:]
        k, v = rnd(dtype, n, nkv, hd), rnd(dtype, n, nkv, hd)
        scatter_kv(pool, k, v, table, P)
        tables.append(table)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    tiles, rest = prefill_tiles(starts, lens, K.PREFILL_TC_TILE_ROWS)
    assert not rest and len(tiles) == 3 + 2 + 1
    M = sum(lens)
    q = rnd(dtype, M, nh, hd)
    out = torch.full((M, nh * hd), float("nan"), dtype=dtype, device="cuda")
    assert K.attention_prefill_tc_ok(dev(q, dtype), P) or not K.PREFILL_TC      # the switch only turns the choice off
    K.attention_prefill_tc(dev(q, dtype), pool, bt, P, i32(tiles), hd ** -0.5, out, window=window)
    assert K.attention_tc_status() == 0
    assert out.isfinite().all(), "a row was not written, or an unwritten cache entry was read"
    first = 0
    for b in range(3):
        rows = list(range(starts[b], totals[b]))
        want = ref_attention(q[first:first + lens[b]], ks[b], vs[b], rows, hd ** -0.5, window)
        close(out[first:first + lens[b]], want, dtype)
        first += lens[b]
    # rows do not depend on the tile they are in: the same rows in tiles of other sizes give the same bits
    other_tiles = [[b, f + r, min(48, n - r), s + r] for b, (f, n, s) in enumerate(zip([0, 300, 450], lens, starts))
                   for r in range(0, n, 48)]
    again = torch.full((M, nh * hd), float("nan"), dtype=dtype, device="cuda")
    K.attention_prefill_tc(dev(q, dtype), pool, bt, P, i32(other_tiles), hd ** -0.5, again, window=window)
    assert torch.equal(again, out)
    assert K.attention_tc_status() == 0


def test_attention_prefill_tc_far_key_and_diagonal(K):
    """As the next test, on the tcgen05 kernel: a key far back stands out for the last row, every row's own key
    for itself."""
    torch.manual_seed(41)
    dtype, nh, nkv, hd, P, T = torch.bfloat16, 2, 1, 64, 16, 640
    k, v = rnd(dtype, T, nkv, hd, scale=0.05), rnd(dtype, T, nkv, hd)
    q = rnd(dtype, T, nh, hd, scale=0.05)
    direction = F.normalize(torch.randn(hd), dim=0)
    k[7, 0] = (direction * 16).to(dtype).float()
    q[T - 1] = (direction * 16).to(dtype).float()
    table = torch.randperm(T // P).tolist()
    pool = make_pool(dtype, len(table), nkv, P, hd)
    scatter_kv(pool, k, v, table, P)
    tiles = [[0, r, min(128, T - r), r] for r in range(0, T, 128)]
    out = torch.zeros(T, nh * hd, dtype=dtype, device="cuda")
    K.attention_prefill_tc(dev(q, dtype), pool, i32([table]), P, i32(tiles), hd ** -0.5, out)
    assert K.attention_tc_status() == 0
    got = out.float().cpu()
    assert (got[T - 1] - v[7, 0].repeat(nh)).abs().max() < 0.02
    close(got, ref_attention(q, k, v, list(range(T)), hd ** -0.5, None), dtype)
    assert torch.allclose(got[0], v[0, 0].repeat(nh), atol=1e-2)     # the first row sees its own key only


def test_attention_prefill_far_key_and_diagonal(K):
    """A key far back is made to stand out for the last row of a portion, and every row's own key for
    itself: the far key must win in the one row, the diagonal in all others (the causal edge)."""
    torch.manual_seed(41)
    dtype, nh, nkv, hd, P, T = torch.bfloat16, 2, 1, 64, 16, 640
    k, v = rnd(dtype, T, nkv, hd, scale=0.05), rnd(dtype, T, nkv, hd)
    q = rnd(dtype, T, nh, hd, scale=0.05)
    direction = F.normalize(torch.randn(hd), dim=0)
    k[7, 0] = (direction * 16).to(dtype).float()
    q[T - 1] = (direction * 16).to(dtype).float()
    table = torch.randperm(T // P).tolist()
    pool = make_pool(dtype, len(table), nkv, P, hd)
    scatter_kv(pool, k, v, table, P)
    tiles = [[0, r, min(64, T - r), r] for r in range(0, T, 64)]
    out = torch.zeros(T, nh * hd, dtype=dtype, device="cuda")
    K.attention_prefill(dev(q, dtype), pool, i32([table]), P, i32(tiles), hd ** -0.5, out)
    got = out.float().cpu()
    assert (got[T - 1] - v[7, 0].repeat(nh)).abs().max() < 0.02
    close(got, ref_attention(q, k, v, list(range(T)), hd ** -0.5, None), dtype)
    assert torch.allclose(got[0], v[0, 0].repeat(nh), atol=1e-2)     # the first row sees its own key only


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,I,K_", [(5, 24, 48), (64, 1792, 256), (65, 56, 72), (2000, 2048, 64),
                                    (300, 120, 136), (1930, 2056, 72), (129, 1032, 64),    # these three end in a tile of few rows
                                    (64, 1024, 2048), (33, 200, 520)])                      # few tiles: split along K, SwiGLU in the sum
def test_products_with_swiglu_store(K, M, I, K_):
    """Gate and up rows interleaved by 8: the few-rows and the tcgen05 products store silu(gate) * up,
    and the stand-alone kernel reads the same layout."""
    from snowllm_b200.ops import interleave_gate_up, linear_swiglu
    torch.manual_seed(50)
    dtype = torch.bfloat16
    x, gate, up = rnd(dtype, M, K_), rnd(dtype, I, K_, scale=K_ ** -0.5), rnd(dtype, I, K_, scale=K_ ** -0.5)
    want = F.silu(x @ gate.T) * (x @ up.T)
    w13 = interleave_gate_up(dev(gate, dtype), dev(up, dtype))
    assert torch.equal(w13[:8].cpu().float(), gate[:8]) and torch.equal(w13[8:16].cpu().float(), up[:8])
    got = linear_swiglu(dev(x, dtype), w13, True)
    assert got.shape == (M, I) and got.dtype == dtype
    close(got, want, dtype, scale=2)
    for dt in DTYPES:         # the stand-alone kernel on the interleaved product
        h = (x @ w13.cpu().float().T).to(dt)
        close(K.swiglu(dev(h), interleaved=True), want, dt, scale=2)
    if dtype == torch.bfloat16:
        assert K.gemm_tc_status() == 0


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 1, 64, 16, None), (32, 8, 64, 16, None), (16, 1, 128, 64, None),
                                                (6, 2, 128, 8, None), (8, 2, 64, 16, 300), (3, 3, 64, 16, 37),
                                                (4, 2, 64, 4, None), (2, 1, 128, 32, 520), (8, 2, 64, 64, None),
                                                (4, 2, 64, 64, 300), (32, 8, 64, 128, None)])
def test_attention_decode_mma(K, nh, nkv, hd, P, window):
    """The tensor-core kernel for decoded rows: requests of very different lengths (one chunk, a chunk
    edge, many chunks), scattered pages, unwritten cache entries NaN, a row list, windows."""
    torch.manual_seed(60)
    dtype = torch.bfloat16
    lens = [1, 255, 256, 257, 700, 1500]
    pages = sum(-(-n // P) for n in lens) + 2
    perm = torch.randperm(pages).tolist()
    pool = torch.full((pages, 2, nkv, P, hd), float("nan"), dtype=dtype, device="cuda")
    tables, ks, vs = [], [], []
    for n in lens:
        need = -(-n // P)
        table, perm = perm[:need], perm[need:]
        k, v = rnd(dtype, n, nkv, hd), rnd(dtype, n, nkv, hd)
        scatter_kv(pool, k, v, table, P)
        tables.append(table)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    positions = [n - 1 for n in lens]
    B = len(lens)
    q = rnd(dtype, B, nh, hd)
    scale = hd ** -0.5
    want = torch.cat([ref_attention(q[b:b + 1], ks[b], vs[b], [positions[b]], scale, window) for b in range(B)])
    lo = [0 if not window else max(0, p - window + 1) for p in positions]
    n_chunks = max(p // 256 - l // 256 for p, l in zip(positions, lo)) + 1
    for extra in (0, 3):                           # more chunks than any row needs (a captured step)
        out = torch.full((B, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attention_decode_mma(dev(q, dtype), pool, bt, P, i32(positions), i32(list(range(B))), scale,
                               n_chunks + extra, out, window=window)
        assert out.isfinite().all(), "an unwritten (NaN) cache entry was read, or a row was not written"
        close(out, want, dtype)
    if K.decode_tma_page_ok(P):                    # keys brought in by TMA or by 16-byte copies: the same bits
        by_copies = torch.full((B, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attention_decode_mma(dev(q, dtype), pool, bt, P, i32(positions), i32(list(range(B))), scale,
                               n_chunks, by_copies, window=window, tma=False)
        assert torch.equal(by_copies, out)
        assert K.attention_decode_status() == 0
    some = [5, 0, 3]
    out = torch.zeros(B, nh * hd, dtype=dtype, device="cuda")
    K.attention_decode_mma(dev(q, dtype), pool, bt, P, i32(positions), i32(list(range(B))), scale, n_chunks, out,
                           window=window, rows=i32(some))
    close(out[some], want[some], dtype)
    assert float(out[[1, 2, 4]].abs().max()) == 0.0
    # the far key: one key of the longest request made to stand out
    far = 300
    direction = F.normalize(torch.randn(hd), dim=0)
    k2 = ks[5].clone()
    k2[far, :] = (direction * 16).to(dtype).float()
    scatter_kv(pool, k2, vs[5], tables[5], P)
    q2 = q.clone()
    q2[5] = (direction * 16).to(dtype).float()
    out = torch.zeros(B, nh * hd, dtype=dtype, device="cuda")
    K.attention_decode_mma(dev(q2, dtype), pool, bt, P, i32(positions), i32(list(range(B))), scale, n_chunks, out,
                           window=None if not window or window > 1300 else window)
    if not window:
        got = out[5].float().cpu().view(nh, hd)
        for h in range(nh):
            assert (got[h] - vs[5][far, h // (nh // nkv)]).abs().max() < 0.02


# ---------------------------------------------------------------------------------------------
def paged_sequence(dtype, N, nkv, hd, P, seed, scale=1.0):
    """A sequence of N random keys and values in scattered pages: (pool with NaN where nothing was written,
    block table as a list, keys, values as float on the GPU)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages = -(-N // P)
    k = (torch.randn(pages * P, nkv, hd, device="cuda", generator=g) * scale).to(dtype)
    v = torch.randn(pages * P, nkv, hd, device="cuda", generator=g).to(dtype)
    table = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed))[:pages]
    pool = torch.full((pages + 3, 2, nkv, P, hd), float("nan"), dtype=dtype, device="cuda")
    pool[table.cuda(), 0] = k.view(pages, P, nkv, hd).transpose(1, 2)
    pool[table.cuda(), 1] = v.view(pages, P, nkv, hd).transpose(1, 2)
    if N % P:                                                  # the last page's tail was never written
        pool[int(table[-1]), :, :, N % P:] = float("nan")
    return pool, table.tolist(), k[:N].float(), v[:N].float()


def attention_from_pages(q, pool, table, P, positions, scale):
    """float64 attention of rows q [M, nh, hd] at ``positions``, recomputed from the cache pages themselves
    (the check of tests/test_lfm2_long_attention.py:28-47 in SnowLLM)."""
    M, nh, hd = q.shape
    nkv = pool.shape[2]
    kv = pool[torch.tensor(table, device="cuda")].double()         # [pages, 2, nkv, P, hd]
    k = kv[:, 0].transpose(1, 2).reshape(-1, nkv, hd)
    v = kv[:, 1].transpose(1, 2).reshape(-1, nkv, hd)
    out = torch.zeros(M, nh, hd, dtype=torch.float64, device="cuda")
    for m, p in enumerate(positions):
        for g in range(nkv):
            heads = slice(g * (nh // nkv), (g + 1) * (nh // nkv))
            s = (q[m, heads].double().cuda() @ k[:p + 1, g].T) * scale
            out[m, heads] = torch.softmax(s, -1) @ v[:p + 1, g]
    return out.reshape(M, nh * hd)


def rel_l2(got, want):
    got, want = got.double().cuda(), want.double().cuda()
    return float(((got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)).max())


@pytest.mark.parametrize("N,P", [(8192, 16), (33000, 16), (33000, 64), (131072, 64)])
def test_attention_over_long_contexts(K, N, P):
    """8,192, 33,000 and 131,072 cached keys (the lengths the measurements run, beyond the longest prompts of
    the dense configurations, and the longest context the reference publishes a run for), in pages of 16 and
    of 64 tokens: decoded rows over 32, 129 and 512 chunks of keys, exactly as many chunks as needed and
    rounded up as a captured step has them; the last rows of a 2,048-row and of an 8,192-row portion through
    the tcgen05 prompt kernel (16 to 1,024 key tiles per block); head size 128 through the mma.sync prompt
    kernel.  Each against float64 attention recomputed from the cache pages, rel-L2 < 0.005 per row."""
    dtype, nh, nkv, hd = torch.bfloat16, 8, 2, 64
    scale = hd ** -0.5
    pool, table, k, v = paged_sequence(dtype, N, nkv, hd, P, seed=N)
    other_pool_rows = N - 300
    # decoded rows: two requests in one launch, the long one and a shorter one in the same pool's pages
    bt = i32([table, table])
    positions = [N - 1, other_pool_rows - 1]
    q = rnd(dtype, 2, nh, hd)
    want = attention_from_pages(q, pool, table, P, positions, scale)
    need = (N - 1) // 256 + 1
    for chunks in (need, 1 << (need - 1).bit_length()):
        out = torch.full((2, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attention_decode_mma(dev(q, dtype), pool, bt, P, i32(positions), i32([0, 1]), scale, chunks, out)
        assert out.isfinite().all()
        assert rel_l2(out, want) < 0.005, f"{chunks} chunks"
    assert K.attention_decode_status() == 0
    # the row-wise kernel (what float32 and other head sizes use) over the same keys, in chunks and whole
    for chunk, chunks in ((256, need), (None, 1)):
        out = K.paged_attention(dev(q, dtype), pool, bt, P, i32(positions), i32([0, 1]), scale, chunk=chunk,
                                num_chunks=chunks)
        assert rel_l2(out, want) < 0.005
    # a far key among thousands: the last row's query points at key 3, in the first of all chunks
    direction = F.normalize(torch.randn(hd), dim=0)
    page, slot = table[0], 3
    saved = pool[page, 0, :, slot].clone()
    pool[page, 0, :, slot] = (direction * 24).to(dtype).cuda()
    q_far = q.clone()
    q_far[0] = (direction * 24).to(dtype).float()
    out = torch.zeros(2, nh * hd, dtype=dtype, device="cuda")
    K.attention_decode_mma(dev(q_far, dtype), pool, bt, P, i32(positions), i32([0, 1]), scale, need, out)
    got = out[0].float().cpu().view(nh, hd)
    for h in range(nh):
        assert (got[h] - v[3, h // (nh // nkv)].cpu()).abs().max() < 0.02
    pool[page, 0, :, slot] = saved
    # prompt portions that end at the sequence's end: their last rows, the first row, rows at tile edges
    for rows in (2048, 8192):
        first = N - rows
        tiles = [[0, r, min(128, rows - r), first + r] for r in range(0, rows, 128)]
        qp = rnd(dtype, rows, nh, hd)
        out = torch.full((rows, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attention_prefill_tc(dev(qp, dtype), pool, i32([table]), P, i32(tiles), scale, out)
        assert K.attention_tc_status() == 0 and out.isfinite().all()
        check = [0, 127, 128, rows // 2 + 5, rows - 3, rows - 2, rows - 1]
        want_p = attention_from_pages(qp[check], pool, table, P, [first + r for r in check], scale)
        assert rel_l2(out[check], want_p) < 0.005, f"portion of {rows} rows"
    # head size 128: the mma.sync prompt kernel and the decode kernel
    hd2 = 128
    pool2, table2, _, _ = paged_sequence(dtype, N, 1, hd2, P, seed=N + 1)
    rows, first = 2048, N - 2048
    tiles = [[0, r, min(64, rows - r), first + r] for r in range(0, rows, 64)]
    qp = rnd(dtype, rows, 3, hd2)
    out = torch.full((rows, 3 * hd2), float("nan"), dtype=dtype, device="cuda")
    K.attention_prefill(dev(qp, dtype), pool2, i32([table2]), P, i32(tiles), hd2 ** -0.5, out)
    check = [0, 63, 64, rows - 3, rows - 2, rows - 1]
    want_p = attention_from_pages(qp[check], pool2, table2, P, [first + r for r in check], hd2 ** -0.5)
    assert rel_l2(out[check], want_p) < 0.005
    out = torch.full((1, 3 * hd2), float("nan"), dtype=dtype, device="cuda")
    K.attention_decode_mma(dev(qp[-1:], dtype), pool2, i32([table2]), P, i32([N - 1]), i32([0]), hd2 ** -0.5, need, out)
    assert rel_l2(out, want_p[-1:]) < 0.005
    assert K.attention_decode_status() == 0


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,H,E,k,bias,norm_topk,scaling", [(1, 2048, 32, 4, True, True, 1.0), (8, 2048, 32, 4, True, True, 1.0),
                                                             (32, 96, 16, 4, False, False, 2.0), (5, 80, 5, 3, True, True, 0.5),
                                                             (3, 1000, 64, 8, True, False, 1.0), (17, 128, 4, 1, True, False, 1.0)])
def test_norm_route_sort_in_one_launch(K, dtype, M, H, E, k, bias, norm_topk, scaling):
    """The one-launch front of a routed feed-forward against the three launches it replaces: the same bits for
    the residual, the normalised rows, the picks and their weights; a valid sort; and again on a second
    call (the ticket counter went back to zero)."""
    from helpers import Guards
    torch.manual_seed(70)
    eps = 1e-5
    gamma = dev(rnd(dtype, H) + 1.0, dtype)
    wr = dev(rnd(dtype, E, H, scale=H ** -0.5), dtype)
    b = dev(torch.randn(E) * 0.01) if bias else None
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    prev_k = 3
    for round_ in range(2):
        start = torch.randn(M, H, device="cuda")
        pieces = K.ExpertSum(torch.randn(M * prev_k, H, device="cuda"), torch.randperm(M * prev_k).int().cuda(),
                             torch.rand(M, prev_k, device="cuda"))
        for delta in (torch.randn(M, H, device="cuda"), pieces, None):
            assert K.norm_route_sort_ok(start, delta, gamma, wr, k)
            res_a, res_b = start.clone(), start.clone()
            x_a = K.add_rmsnorm(res_a, delta, gamma, eps, dtype)
            ids_a, w_a, off_a, pos_a, sorted_a = K.moe_route_sort(x_a, wr, b, k, norm_topk, scaling)
            x_b, ids_b, w_b, off_b, pos_b, sorted_b = K.norm_route_sort(res_b, delta, gamma, eps, dtype, wr, b, k,
                                                                         norm_topk, scaling, ticket)
            assert torch.equal(res_a, res_b) and torch.equal(x_a, x_b)
            assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b) and torch.equal(off_a, off_b)
            assert int(ticket) == 0
            # the sort: every pair once, inside its expert's rows, and pair_pos its inverse
            flat = ids_b.flatten().long().cpu()
            sp, pp, off = sorted_b.long().cpu(), pos_b.long().cpu(), off_b.long().cpu()
            assert sorted(sp.tolist()) == list(range(M * k)) and torch.equal(pp[sp], torch.arange(M * k))
            for e in range(E):
                assert bool((flat[sp[off[e]:off[e + 1]]] == e).all())
    # nothing outside the buffers the caller sized (the outputs are made inside the wrapper; the residual is not)
    g = Guards()
    res = g((M, H), torch.float32, like=torch.randn(M, H, device="cuda"))
    tk = g((1,), torch.int32, fill=0)
    K.norm_route_sort(res, torch.randn(M, H, device="cuda"), gamma, eps, dtype, wr, b, k, norm_topk, scaling, tk)
    g.check("norm_route_sort")
