"""Sentinel bounds: every kernel that writes into a buffer its caller sized is run with that buffer lying
between two bands of a fixed pattern; nothing before the buffer's start or past its end may change.  Sizes are
odd on purpose (rows, widths and vocabularies that no tile divides), so that a kernel that rounds its extent
up to a tile, a vector or a warp would write into a band.  The results themselves are compared with the same
call on ordinary buffers (whose values other tests check against plain references).
(SnowLLM guards its argmax output the same way: tests/test_sampling_argmax.py:13-44.)"""
import pytest
import torch

from helpers import Guards

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from snowllm_b200.ops import kernels
    return kernels


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def rnd(dtype, *shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_elementwise_kernels_stay_inside_their_outputs(K, dtype):
    torch.manual_seed(0)
    g = Guards()
    V, H, M = 331, 1000, 7                             # H: no multiple of 16 bytes x a power of two
    table = rnd(dtype, V, H)
    ids = i32([5, 330, 0, 17, 200, 1, 99])
    pending = g((4,), torch.int32, like=i32([7, 8, 9, 10]))
    out = K.embedding(i32([5, -2, 330, -4, 0, 17, 1]), table, out=g((M, H), torch.float32, fill=float("nan")),
                      pending=pending)
    assert torch.equal(out, K.embedding(i32([5, 8, 330, 10, 0, 17, 1]), table))
    gamma = rnd(dtype, H)
    for rows in (None, i32([6, 0, 6])):
        start, delta = torch.randn(M, H, device="cuda"), torch.randn(M, H, device="cuda")
        res, plain_res = g((M, H), torch.float32, like=start), start.clone()
        R = M if rows is None else rows.numel()
        out = K.add_rmsnorm(res, delta, gamma, 1e-5, dtype, rows=rows, out=g((R, H), dtype, fill=float("nan")))
        assert torch.equal(out, K.add_rmsnorm(plain_res, delta, gamma, 1e-5, dtype, rows=rows))
        assert torch.equal(res, plain_res)
        # the delta still in pieces: the routed experts' outputs, summed by the norm itself
        k = 3
        pieces = K.ExpertSum(torch.randn(M * k, H, device="cuda"), torch.randperm(M * k).int().cuda(),
                             torch.rand(M, k, device="cuda"))
        res, plain_res = g((M, H), torch.float32, like=start), start.clone()
        out = K.add_rmsnorm(res, pieces, gamma, 1e-5, dtype, rows=rows, out=g((R, H), dtype, fill=float("nan")))
        assert torch.equal(out, K.add_rmsnorm(plain_res, pieces, gamma, 1e-5, dtype, rows=rows))
        assert torch.equal(res, plain_res)
    gu = rnd(dtype, M, 2 * 57)
    out = K.swiglu(gu, out=g((M, 57), dtype, fill=float("nan")))
    assert torch.equal(out, K.swiglu(gu))
    r = g((M, H), torch.float32, like=torch.randn(M, H, device="cuda"))
    K.residual_add(r, torch.randn(M, H, device="cuda"))
    g.check("elementwise")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(3, 1, 48), (5, 5, 64), (2, 1, 128)])
def test_rope_and_cache_write_stay_inside_q_and_the_pool(K, dtype, nh, nkv, hd):
    torch.manual_seed(1)
    g = Guards()
    P, pages = 8, 6
    positions, row_seg = [13, 14, 15, 16, 0, 1, 47], [0, 0, 0, 0, 1, 1, 0]     # position 47: the pool's very last row
    tables = i32([[4, 1, 2, 0, 3, 5], [3, 0, 0, 0, 0, 0]])
    M = len(positions)
    qkv = rnd(dtype, M, (nh + 2 * nkv) * hd)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32, device="cuda") / hd))
    pool = g((pages, 2, nkv, P, hd), dtype, fill=0.0)
    plain_pool = torch.zeros_like(pool)
    q = K.qk_norm_rope_cache(qkv, rnd(dtype, hd), rnd(dtype, hd), 1e-6, inv, hd, i32(positions), i32(row_seg),
                             tables, P, pool, nh, nkv, hd, q_out=g((M, nh, hd), dtype, fill=float("nan")))
    assert q.isfinite().all() and pool.isfinite().all()
    g.check("qk_norm_rope_cache")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_kernels_stay_inside_their_outputs_and_scratch(K, dtype):
    torch.manual_seed(2)
    g = Guards()
    nh, nkv, hd, P = 6, 2, 64, 16
    lens = [700, 33, 300]
    pages = sum(-(-n // P) for n in lens)
    pool = rnd(dtype, pages, 2, nkv, P, hd)
    tables, at = [], 0
    for n in lens:
        need = -(-n // P)
        tables.append(list(range(at, at + need)) + [0] * (44 - need))
        at += need
    bt = i32(tables)
    # rows: a portion of the first request, single rows of the others
    positions = list(range(600, 700)) + [32, 299]
    row_seg = [0] * 100 + [1, 2]
    M = len(positions)
    q = rnd(dtype, M, nh, hd)
    scale = hd ** -0.5
    for chunk, chunks in ((None, 1), (256, 3)):
        need = K.attention_scratch_bytes(M, nh, hd, chunks) if chunks > 1 else 1
        out = K.paged_attention(q, pool, bt, P, i32(positions), i32(row_seg), scale, chunk=chunk, num_chunks=chunks,
                                scratch=g((need,), torch.uint8) if chunks > 1 else None,
                                out=g((M, nh * hd), dtype, fill=float("nan")))
        assert torch.equal(out, K.paged_attention(q, pool, bt, P, i32(positions), i32(row_seg), scale, chunk=chunk,
                                                  num_chunks=chunks))
    some = i32([101, 3, 100])
    need = K.attention_scratch_bytes(3, nh, hd, 3)
    out = K.paged_attention(q, pool, bt, P, i32(positions), i32(row_seg), scale, chunk=256, num_chunks=3,
                            scratch=g((need,), torch.uint8), out=g((M, nh * hd), dtype, fill=0.0), rows=some)
    if dtype == torch.bfloat16:
        need = K.attention_scratch_bytes(M, nh, hd, 3)
        out = K.attention_decode_mma(q, pool, bt, P, i32(positions), i32(row_seg), scale, 3,
                                     g((M, nh * hd), dtype, fill=float("nan")), scratch=g((need,), torch.uint8))
        assert torch.equal(out, K.attention_decode_mma(q, pool, bt, P, i32(positions), i32(row_seg), scale, 3,
                                                       torch.empty(M, nh * hd, dtype=dtype, device="cuda")))
        for tile_rows, call in ((64, K.attention_prefill), (128, K.attention_prefill_tc)):
            tiles = i32([[0, r, min(tile_rows, 100 - r), 600 + r] for r in range(0, 100, tile_rows)])
            out = call(q, pool, bt, P, tiles, scale, g((M, nh * hd), dtype, fill=0.0))
            assert torch.equal(out[:100], call(q, pool, bt, P, tiles, scale, torch.zeros(M, nh * hd, dtype=dtype,
                                                                                       device="cuda"))[:100])
            assert float(out[100:].abs().max()) == 0.0             # rows outside the tiles are not touched
        assert K.attention_tc_status() == 0 and K.attention_decode_status() == 0
    g.check("attention")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,L", [(72, 3), (1000, 4), (2048, 2)])
def test_short_conv_stays_inside_its_output_and_state(K, dtype, H, L):
    torch.manual_seed(3)
    g = Guards()
    lens, starts, slots = [19, 1, 1, 40], [0, 5, 0, 7], [2, 0, 3, 1]
    M, B = sum(lens), len(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    row_seg = sum(([b] * n for b, n in enumerate(lens)), [])
    bcx = rnd(dtype, M, 3 * H)
    w = rnd(dtype, H, L)
    state = g((4, L - 1, H), dtype, like=rnd(dtype, 4, L - 1, H))
    plain_state = state.clone()
    out = K.short_conv(bcx, w, state, i32(cu), i32(starts), i32(slots), i32(row_seg), out=g((M, H), dtype, fill=float("nan")))
    assert torch.equal(out, K.short_conv(bcx, w, plain_state, i32(cu), i32(starts), i32(slots), i32(row_seg)))
    assert torch.equal(state, plain_state)
    # one-token segments only: the fused kernel
    ones = [1, 1, 1]
    state = g((4, L - 1, H), dtype, like=rnd(dtype, 4, L - 1, H))
    out = K.short_conv(bcx[:3].contiguous(), w, state, i32([0, 1, 2, 3]), i32([4, 0, 9]), i32([3, 1, 0]), i32([0, 1, 2]),
                       out=g((3, H), dtype, fill=float("nan")))
    assert out.isfinite().all()
    g.check("short_conv")


@pytest.mark.parametrize("M,N,K_", [(3, 200, 72), (13, 1000, 136), (130, 264, 200), (300, 2056, 72), (4100, 520, 64)])
def test_products_stay_inside_their_outputs(K, M, N, K_):
    """Every product kernel at shapes whose last tiles are ragged in both directions, to float and to bfloat16,
    plain and with SwiGLU at the store."""
    from snowllm_b200.ops import interleave_gate_up, linear, linear_swiglu
    torch.manual_seed(4)
    g = Guards()
    for dtype in DTYPES:
        x, w = rnd(dtype, M, K_), rnd(dtype, N, K_, scale=K_ ** -0.5)
        for out_dtype in {dtype, torch.float32}:
            out = linear(x, w, out_dtype=out_dtype, out=g((M, N), out_dtype, fill=float("nan")))
            assert torch.equal(out, linear(x, w, out_dtype=out_dtype))
    x = rnd(torch.bfloat16, M, K_)
    simt = K.gemm_simt(x, w.to(torch.bfloat16), out=g((M, N), torch.bfloat16, fill=float("nan")))
    assert simt.isfinite().all()
    if M > 16:
        for call in (K.gemm_tc, K.gemm_tc2):
            for out_dtype in (torch.bfloat16, torch.float32):
                out = call(x, w.to(torch.bfloat16), out_dtype=out_dtype, out=g((M, N), out_dtype, fill=float("nan")))
                assert torch.equal(out, call(x, w.to(torch.bfloat16), out_dtype=out_dtype))
    else:
        out = K.gemm_skinny(x, w.to(torch.bfloat16), out=g((M, N), torch.bfloat16, fill=float("nan")))
        assert torch.equal(out, K.gemm_skinny(x, w.to(torch.bfloat16)))
    I = N // 16 * 8
    w13 = interleave_gate_up(rnd(torch.bfloat16, I, K_, scale=K_ ** -0.5), rnd(torch.bfloat16, I, K_, scale=K_ ** -0.5))
    want = linear_swiglu(x, w13, True)
    if M <= 16:
        out = K.gemm_skinny(x, w13, swiglu=True, out=g((M, I), torch.bfloat16, fill=float("nan")))
        assert torch.equal(out, want)
    else:
        for call in (K.gemm_tc, K.gemm_tc2):
            out = call(x, w13, swiglu=True, out=g((M, I), torch.bfloat16, fill=float("nan")))
            assert out.isfinite().all()
    assert K.gemm_tc_status() == 0 and K.gemm_tc2_status()[0] == 0
    g.check("products")


@pytest.mark.parametrize("rows_per_group", [[3, 0, 1, 7], [270, 0, 1, 16, 17, 255, 130]])
def test_grouped_products_and_gather_stay_inside_their_outputs(K, rows_per_group):
    torch.manual_seed(5)
    g = Guards()
    dtype, N, K_ = torch.bfloat16, 264, 136
    G = len(rows_per_group)
    offsets = [0]
    for c in rows_per_group:
        offsets.append(offsets[-1] + c)
    R = offsets[-1]
    src = rnd(dtype, max(R // 2, 4), K_)
    pairs = torch.randint(0, 2 * src.shape[0], (R,)).tolist()
    w = rnd(dtype, G, N, K_, scale=K_ ** -0.5)
    xs = K.gather_rows(src, i32(pairs), 2, out=g((R, K_), dtype, fill=float("nan")))
    assert torch.equal(xs, src[[p // 2 for p in pairs]])
    for out_dtype in (torch.bfloat16, torch.float32):
        calls = [lambda out: K.gemm_simt(src, w, out_dtype=out_dtype, out=out, a_rows=i32(pairs), a_div=2,
                                         offsets=i32(offsets), rows_out=R, max_rows_per_group=max(rows_per_group)),
                 lambda out: K.gemm_skinny(src, w, out_dtype=out_dtype, out=out, a_rows=i32(pairs), a_div=2,
                                           offsets=i32(offsets), rows_out=R, rows_hint=8),
                 lambda out: K.gemm_tc(xs, w, out_dtype=out_dtype, out=out, offsets=i32(offsets)),
                 lambda out: K.gemm_tc2(xs, w, out_dtype=out_dtype, out=out, offsets=i32(offsets))]
        for call in calls:
            out = call(g((R, N), out_dtype, fill=float("nan")))
            assert out.isfinite().all()
    assert K.gemm_tc_status() == 0 and K.gemm_tc2_status()[0] == 0
    y = torch.randn(R, 72, device="cuda")
    M, k = R // 2 if R % 2 == 0 else R, 2 if R % 2 == 0 else 1
    pos = torch.randperm(R).int().cuda()
    wts = torch.rand(M, k, device="cuda")
    out = K.moe_combine(y, pos, wts, out=g((M, 72), torch.float32, fill=float("nan")))
    assert torch.equal(out, K.moe_combine(y, pos, wts))
    g.check("grouped products")


@pytest.mark.parametrize("B,V", [(1, 331), (5, 65536), (3, 50001)])
def test_sampling_kernels_stay_inside_their_outputs(K, B, V):
    torch.manual_seed(6)
    g = Guards()
    logits = g((B, V), torch.float32, like=torch.randn(B, V, device="cuda"))
    out = K.argmax(logits, out=g((B,), torch.int32, fill=-1))
    assert torch.equal(out.long(), logits.argmax(-1))
    temp = torch.full((B,), 0.8, device="cuda")
    out = K.sample(logits, temp, i32([40] * B), torch.full((B,), 0.9, device="cuda"), torch.rand(B, device="cuda"),
                   out=g((B,), torch.int32, fill=-1))
    assert bool(((out >= 0) & (out < V)).all())
    offsets = [0]
    ids, counts = [], []
    for b in range(B):
        mine = {0: 1, (7 * b + 3) % V: 2, V - 1: -1}             # a count of -1 bans the token
        ids += sorted(mine)
        counts += [mine[t] for t in sorted(mine)]
        offsets.append(len(ids))
    K.apply_penalties(logits, i32(offsets), i32(ids), i32(counts), torch.full((B,), 0.5, device="cuda"),
                      torch.full((B,), 0.25, device="cuda"), torch.full((B,), 1.3, device="cuda"))
    assert bool((logits[:, V - 1] == float("-inf")).all())
    g.check("sampling")
