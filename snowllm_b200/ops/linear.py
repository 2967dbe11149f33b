"""Matrix products of the model: the one place that picks a kernel for a shape and dtype.

float32: the CUDA-core kernel of csrc/gemm.cu (true 32-bit, sums in k order).
bfloat16, up to 16 rows (decode; grouped: up to 4 rows per group on average): csrc/gemm_skinny.cu, which
streams W once into mma.sync fragments.
bfloat16, more rows (prefill): csrc/gemm_tc.cu, 128 x 256 tiles on the tcgen05 tensor cores with TMA
loads and the accumulator in tensor memory; from 4,096 rows on, and for all grouped products, csrc/gemm_tc2.cu
on pairs of SMs (grouped: W is the 256-row operand and a group's rows the N side, in steps of 16).
bfloat16 operands that neither takes (K no multiple of 8, unaligned views): the CUDA-core kernel.
(the role of snowllm/models/projection.py:27-35)
"""
from __future__ import annotations

import os

import torch

from . import kernels

# Products of very many rows run on pairs of SMs (csrc/gemm_tc2.cu: 256 x 256 tiles, a third less operand traffic).
# Measured against the one-SM kernel: 2,048 rows no gain (the launch is short; tile rounds and the epilogue
# decide), 4,096 rows +6 %, 8,192 rows +7 %.  Grouped (32 experts, top 4): the 2,048-token prefill step
# 9.78 -> 9.38 ms, the 64-request decode step 5.90 -> 5.58 ms against the one-SM kernel's 128-row tiles.
TC_PAIRS = os.environ.get("SNOWLLM_B200_TC_PAIRS", "1") != "0"
PAIRS_MIN_ROWS = 4096             # plain products
PAIRS_MAX_GROUPS = 256            # grouped products always run on pairs (a group's rows are the N side of the MMA)


def _tc(x, w, **kw):
    """The tcgen05 product: on pairs of SMs where there are rows enough."""
    offsets = kw.get("offsets")
    rows = x.shape[0]
    if TC_PAIRS and (rows >= PAIRS_MIN_ROWS if offsets is None else w.shape[0] <= PAIRS_MAX_GROUPS):
        return kernels.gemm_tc2(x, w, **kw)
    return kernels.gemm_tc(x, w, **kw)


SKINNY_MAX_ROWS = 16       # measured crossover: up to here the few-rows kernel reads W faster than 128-row tiles
SKINNY_MAX_GROUP_ROWS = 4  # grouped: mean rows per group up to which the few-rows kernel wins


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K]^T -> [M, N] in ``out_dtype`` (the compute dtype or float32)."""
    if kernels.gemm_skinny_ok(x, w):
        if x.shape[0] <= SKINNY_MAX_ROWS:
            return kernels.gemm_skinny(x, w, out_dtype=out_dtype, out=out)
        return _tc(x, w, out_dtype=out_dtype, out=out)
    return kernels.gemm_simt(x, w, out_dtype=out_dtype, out=out)


def _few_rows_per_group(rows_out: int, groups: int) -> bool:
    return rows_out <= SKINNY_MAX_GROUP_ROWS * groups


def grouped_linear(x, w, offsets, rows_out, max_rows_per_group, a_rows=None, a_div=1, out_dtype=None):
    """Rows sorted by group: row r in [offsets[g], offsets[g+1]) is x[a_rows[r] // a_div] (or x[r])
    times w[g] [N, K]^T.  ``max_rows_per_group`` bounds the rows one group can own."""
    if kernels.gemm_skinny_ok(x, w):
        if _few_rows_per_group(rows_out, w.shape[0]):
            # a pass covers about twice the mean rows of a group; fuller groups take more passes
            hint = min(max_rows_per_group, max(8, 2 * -(-rows_out // w.shape[0])))
            return kernels.gemm_skinny(x, w, out_dtype=out_dtype, a_rows=a_rows, a_div=a_div, offsets=offsets,
                                       rows_out=rows_out, rows_hint=hint)
        # TMA reads whole tiles of contiguous rows: bring the rows into sorted order first
        xs = kernels.gather_rows(x, a_rows, a_div) if a_rows is not None else x
        return _tc(xs, w, out_dtype=out_dtype, offsets=offsets)
    return kernels.gemm_simt(x, w, out_dtype=out_dtype, a_rows=a_rows, a_div=a_div, offsets=offsets,
                             rows_out=rows_out, max_rows_per_group=max_rows_per_group)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[..., I, K] gate and up rows -> [..., 2I, K] in blocks of 8 gate rows followed by the 8 up rows of
    the same features: the layout whose product can apply SwiGLU at its store (I a multiple of 8)."""
    *lead, I, K = gate.shape
    both = torch.stack((gate.reshape(*lead, I // 8, 8, K), up.reshape(*lead, I // 8, 8, K)), dim=-3)
    return both.reshape(*lead, 2 * I, K).contiguous()


def linear_swiglu(x: torch.Tensor, w13: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) -> [M, I] with Wg, Wu held in one matrix w13 [2I, K] (plain halves, or
    interleaved by 8).  With the interleaved layout the bfloat16 products apply SwiGLU at their store."""
    if interleaved and kernels.gemm_skinny_ok(x, w13):
        if x.shape[0] <= SKINNY_MAX_ROWS:
            return kernels.gemm_skinny(x, w13, swiglu=True)
        return _tc(x, w13, swiglu=True)
    return kernels.swiglu(linear(x, w13), interleaved=interleaved)


def grouped_linear_swiglu(x, w13, offsets, rows_out, max_rows_per_group, a_rows, a_div, interleaved: bool):
    """The grouped form of ``linear_swiglu`` over rows sorted by group (w13 [G, 2I, K])."""
    if interleaved and kernels.gemm_skinny_ok(x, w13):
        if _few_rows_per_group(rows_out, w13.shape[0]):
            hint = min(max_rows_per_group, max(8, 2 * -(-rows_out // w13.shape[0])))
            return kernels.gemm_skinny(x, w13, a_rows=a_rows, a_div=a_div, offsets=offsets, rows_out=rows_out,
                                       rows_hint=hint, swiglu=True)
        xs = kernels.gather_rows(x, a_rows, a_div) if a_rows is not None else x
        return _tc(xs, w13, offsets=offsets, swiglu=True)
    h = grouped_linear(x, w13, offsets, rows_out, max_rows_per_group, a_rows=a_rows, a_div=a_div)
    return kernels.swiglu(h, interleaved=interleaved)
