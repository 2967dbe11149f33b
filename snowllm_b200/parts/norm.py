"""RMSNorm over the hidden size, fused with the residual sum that precedes it
(snowllm/ops/norm.py:11-30; snowllm/models/lfm2/layers.py:99-104)."""
from __future__ import annotations

from ..ops import kernels
from .base import Part
from .registry import register_norm
from .spec import INIT_ONES, KEEP_SMALL, TensorSpec


class RMSNorm(Part):
    libraries = ("elementwise",)
    fusable_rms = True     # x * rsqrt(mean(x^2) + eps) * weight over the whole width: what a part that fuses
                           # the norm before it into its own first kernel may take over (weight, eps)

    def __init__(self, dtype, names, *, size: int, eps: float):
        super().__init__(dtype, names)
        self.size, self.eps = size, eps
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.size,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, residual, delta=None, rows=None):
        """``residual += delta`` in float, then the norm of the sum in the compute dtype.  With
        ``rows`` (int32 row numbers) only those rows come out and the residual stays untouched."""
        return kernels.add_rmsnorm(residual, delta, self.weight, self.eps, self.dtype, rows=rows)


register_norm("rmsnorm", RMSNorm)
