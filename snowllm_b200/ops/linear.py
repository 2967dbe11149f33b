"""Matrix products of the model: the one place that picks a kernel for a shape and dtype.

float32: the CUDA-core kernel of csrc/gemm.cu (true 32-bit, sums in k order).
bfloat16: the same kernel until a tensor-core kernel for the shape is enabled here.
(the role of snowllm/models/projection.py:27-35)
"""
from __future__ import annotations

import torch

from . import kernels


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K]^T -> [M, N] in ``out_dtype`` (the compute dtype or float32)."""
    return kernels.gemm_simt(x, w, out_dtype=out_dtype, out=out)


def grouped_linear(x, w, offsets, rows_out, max_rows_per_group, a_rows=None, a_div=1, out_dtype=None):
    """Rows sorted by group: row r in [offsets[g], offsets[g+1]) is x[a_rows[r] // a_div] (or x[r])
    times w[g] [N, K]^T."""
    return kernels.gemm_simt(x, w, out_dtype=out_dtype, a_rows=a_rows, a_div=a_div, offsets=offsets,
                             rows_out=rows_out, max_rows_per_group=max_rows_per_group)
