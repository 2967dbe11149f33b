"""One kernel at one shape, timed on the device: the small case that profiles are taken on.

    python -m snowllm_b200.ops.microbench gemm_skinny --m 8 --n 3584 --k 2048 --groups 32 --active 21
    python -m snowllm_b200.ops.microbench gemm_tc --m 2048 --n 6144 --k 2048
    python -m snowllm_b200.ops.microbench attention_decode --batch 8 --context 8192
    python -m snowllm_b200.ops.microbench attention_prefill --tokens 2048
    python -m snowllm_b200.ops.microbench short_conv --tokens 2048 --n 2048
    python -m snowllm_b200.ops.microbench qk_norm_rope --tokens 2048

Prints one JSON line: microseconds per launch (CUDA events around ``--iters`` launches after 3 warm-up
launches, a buffer larger than L2 written between launches) and the achieved GB/s or TFLOP/s from the
bytes or flops the kernel has to move.  Inputs are seeded random values.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from . import kernels

L2_FLUSH_BYTES = 256 << 20


def timed(fn, iters: int, flush: bool = True) -> float:
    """Mean microseconds of ``fn()`` over ``iters`` launches, L2 flushed (a 256 MB buffer read) before each."""
    scrub = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scrub is not None:
            scrub.max()          # a READ of 256 MB: L2 then holds clean lines of the scrub buffer.  (A fill's lines
                                 # leave L2 first and the last turn's operands stay; a buffer written leaves L2 full
                                 # of lines that must go back to memory while the timed kernel runs.)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    return total / iters * 1e3


def bf16(*shape, scale=1.0, gen=None):
    return (torch.randn(*shape, device="cuda", generator=gen) * scale).to(torch.bfloat16)


def gemm_skinny(a):
    gen = torch.Generator(device="cuda").manual_seed(0)
    G = a.groups
    w = bf16(G, a.n, a.k, scale=a.k ** -0.5, gen=gen) if G > 1 else bf16(a.n, a.k, scale=a.k ** -0.5, gen=gen)
    if G > 1:
        active = min(a.active or G, G)
        rows = a.m * active                       # a.m rows for each group that owns rows
        counts = [a.m if e < active else 0 for e in range(G)]
        offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
        x = bf16(rows, a.k, gen=gen)
        fn = lambda: kernels.gemm_skinny(x, w, offsets=offsets, rows_out=rows, rows_hint=a.m,
                                         out_dtype=torch.float32 if a.f32 else None, swiglu=a.swiglu)
        nbytes = active * a.n * a.k * 2
    else:
        x = bf16(a.m, a.k, gen=gen)
        fn = lambda: kernels.gemm_skinny(x, w, out_dtype=torch.float32 if a.f32 else None, swiglu=a.swiglu)
        nbytes = a.n * a.k * 2
    us = timed(fn, a.iters)
    return {"us": us, "GB/s": nbytes / us / 1e3, "bytes": nbytes}


def gemm_tc(a):
    gen = torch.Generator(device="cuda").manual_seed(0)
    G = a.groups
    product = kernels.gemm_tc2 if a.pairs else kernels.gemm_tc      # --pairs: the kernel on pairs of SMs
    if G > 1:
        w = bf16(G, a.n, a.k, scale=a.k ** -0.5, gen=gen)
        per = a.m // G
        if a.ragged:                              # rows dealt to the groups at random, as a router does
            counts = torch.bincount(torch.randint(0, G, (per * G,), generator=torch.Generator().manual_seed(1)), minlength=G)
            offsets = torch.cat((torch.zeros(1, dtype=torch.int64), counts.cumsum(0))).to(torch.int32).cuda()
        else:
            offsets = torch.arange(0, G + 1, dtype=torch.int32, device="cuda") * per
        x = bf16(per * G, a.k, gen=gen)
        fn = lambda: product(x, w, offsets=offsets, out_dtype=torch.float32 if a.f32 else None, swiglu=a.swiglu)
        flops = 2.0 * per * G * a.n * a.k
    else:
        w, x = bf16(a.n, a.k, scale=a.k ** -0.5, gen=gen), bf16(a.m, a.k, gen=gen)
        fn = lambda: product(x, w, out_dtype=torch.float32 if a.f32 else None, swiglu=a.swiglu)
        flops = 2.0 * a.m * a.n * a.k
    us = timed(fn, a.iters)
    assert kernels.gemm_tc_status() == 0 and (not a.pairs or kernels.gemm_tc2_status()[0] == 0)
    return {"us": us, "TFLOP/s": flops / us / 1e6, "flops": flops}


def _cache(a, tokens_each, batch):
    gen = torch.Generator(device="cuda").manual_seed(0)
    P = a.page_size
    pages_each = -(-tokens_each // P)
    pool = bf16(batch * pages_each, 2, a.kv_heads, P, a.head_dim, gen=gen)
    perm = torch.randperm(batch * pages_each, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    return pool, perm.view(batch, pages_each).cuda(), gen


def attention_decode(a):
    pool, bt, gen = _cache(a, a.context, a.batch)
    q = bf16(a.batch, a.heads, a.head_dim, gen=gen)
    positions = torch.full((a.batch,), a.context - 1, dtype=torch.int32, device="cuda")
    row_seg = torch.arange(a.batch, dtype=torch.int32, device="cuda")
    chunk = a.chunk
    n = -(-a.context // chunk)
    scratch = torch.empty(kernels.attention_scratch_bytes(a.batch, a.heads, a.head_dim, n), dtype=torch.uint8,
                          device="cuda")
    out = torch.empty(a.batch, a.heads * a.head_dim, dtype=torch.bfloat16, device="cuda")
    if a.rowwise:      # the CUDA-core kernel of csrc/attention.cu
        fn = lambda: kernels.paged_attention(q, pool, bt, a.page_size, positions, row_seg, a.head_dim ** -0.5,
                                             chunk=chunk, num_chunks=n, scratch=scratch, out=out)
    else:              # the tensor-core kernel of csrc/attention_mma.cu (chunks of 256 keys)
        n = -(-a.context // kernels.DECODE_MMA_CHUNK)
        fn = lambda: kernels.attention_decode_mma(q, pool, bt, a.page_size, positions, row_seg,
                                                  a.head_dim ** -0.5, n, out, scratch=scratch)
    nbytes = a.batch * a.context * 2 * a.kv_heads * a.head_dim * 2
    us = timed(fn, a.iters)
    return {"us": us, "GB/s": nbytes / us / 1e3, "bytes": nbytes}


def attention_prefill(a):
    from ..parts.attention_plan import prefill_tiles
    pool, bt, gen = _cache(a, a.tokens, 1)
    q = bf16(a.tokens, a.heads, a.head_dim, gen=gen)
    tc = not a.rowwise and kernels.attention_prefill_tc_ok(q, a.page_size)       # --rowwise: the mma.sync kernel
    tiles, _ = prefill_tiles([0], [a.tokens], kernels.PREFILL_TC_TILE_ROWS if tc else kernels.PREFILL_TILE_ROWS)
    tiles = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    out = torch.empty(a.tokens, a.heads * a.head_dim, dtype=torch.bfloat16, device="cuda")
    if tc:
        fn = lambda: kernels.attention_prefill_tc(q, pool, bt, a.page_size, tiles, a.head_dim ** -0.5, out)
    else:
        fn = lambda: kernels.attention_prefill(q, pool, bt, a.page_size, tiles, a.head_dim ** -0.5, out)
    flops = 4.0 * a.heads * a.head_dim * a.tokens * (a.tokens + 1) / 2
    us = timed(fn, a.iters)
    return {"us": us, "TFLOP/s": flops / us / 1e6, "flops": flops}


def short_conv(a):
    """The gated short convolution over one fresh segment of --tokens rows, hidden size --n, --taps taps."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    M, H, L = a.tokens, a.n, a.taps
    sets = 6                                              # distinct inputs in turn: each launch reads cold rows
    bcx = [bf16(M, 3 * H, gen=gen) for _ in range(sets)]
    w = bf16(H, L, gen=gen)
    state = torch.zeros(2, L - 1, H, dtype=torch.bfloat16, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    cu, start, slot, row_seg = i32([0, M]), i32([0]), i32([0]), torch.zeros(M, dtype=torch.int32, device="cuda")
    out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    turn = [0]

    def fn():
        turn[0] += 1
        kernels.short_conv(bcx[turn[0] % sets], w, state, cu, start, slot, row_seg, out=out)
    nbytes = M * H * 2 * 4
    us = timed(fn, a.iters)
    return {"us": us, "GB/s": nbytes / us / 1e3, "bytes": nbytes}


def qk_norm_rope(a):
    """Per-head q/k RMSNorm, rotary encoding and the cache write over --tokens rows of one fresh request."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    M, nh, nkv, hd, P = a.tokens, a.heads, a.kv_heads, a.head_dim, a.page_size
    qkv = bf16(M, (nh + 2 * nkv) * hd, gen=gen)
    g = torch.ones(hd, dtype=torch.bfloat16, device="cuda")
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32, device="cuda") / hd))
    pages = -(-M // P)
    pool = torch.zeros(pages, 2, nkv, P, hd, dtype=torch.bfloat16, device="cuda")
    bt = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    pos = torch.arange(M, dtype=torch.int32, device="cuda")
    seg = torch.zeros(M, dtype=torch.int32, device="cuda")
    fn = lambda: kernels.qk_norm_rope_cache(qkv, g, g, 1e-5, inv, hd, pos, seg, bt, P, pool, nh, nkv, hd)
    nbytes = M * (nh + 2 * nkv) * hd * 2 * 2
    us = timed(fn, a.iters)
    return {"us": us, "GB/s": nbytes / us / 1e3, "bytes": nbytes}


KINDS = {"short_conv": short_conv, "qk_norm_rope": qk_norm_rope, "gemm_skinny": gemm_skinny, "gemm_tc": gemm_tc, "attention_decode": attention_decode,
         "attention_prefill": attention_prefill}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m snowllm_b200.ops.microbench", description=__doc__.split("\n\n")[0])
    ap.add_argument("kind", choices=sorted(KINDS))
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=3584)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--groups", type=int, default=1)
    ap.add_argument("--active", type=int, default=0, help="groups that own rows (gemm_skinny)")
    ap.add_argument("--f32", action="store_true", help="float32 output")
    ap.add_argument("--swiglu", action="store_true", help="SwiGLU at the store (w rows interleaved by 8)")
    ap.add_argument("--ragged", action="store_true", help="gemm_tc with --groups: random rows per group, not m / groups")
    ap.add_argument("--pairs", action="store_true", help="gemm_tc: the kernel on pairs of SMs (cta_group::2)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--taps", type=int, default=3, help="short_conv: kernel length")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--chunk", type=int, default=256)
    ap.add_argument("--rowwise", action="store_true", help="attention_decode: the CUDA-core kernel; attention_prefill: the mma.sync kernel")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)
    out = {"kernel": a.kind, **{k: v for k, v in vars(a).items() if k != "kind"}}
    out.update({k: (round(v, 2) if isinstance(v, float) else v) for k, v in KINDS[a.kind](a).items()})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
