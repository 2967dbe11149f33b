"""Gated short-convolution mixer with a fixed-size history per request
(snowllm/models/lfm2/layers.py:20-33; snowllm/ops/lfm2.py:8-26): in_proj to (B | C | x), g = B*x,
causal depthwise convolution of ``kernel_size`` taps over the request's history and this step's g,
y = C*conv, out_proj.  The history (the last kernel_size-1 rows of g) lives in the request's slot."""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import Part
from .registry import register_mixer
from .spec import INIT_CONV, KEEP_SMALL, SlotStateSpec, TensorSpec


class ShortConv(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "short_conv")

    def __init__(self, dtype, names, *, hidden_size: int, kernel_size: int):
        super().__init__(dtype, names)
        self.hidden_size, self.kernel_size = hidden_size, kernel_size
        self.in_proj = self.conv = self.out_proj = None

    def cache_spec(self):
        return SlotStateSpec(((max(self.kernel_size - 1, 0), self.hidden_size),), ("compute",))

    def declare(self, has):
        H, L, n = self.hidden_size, self.kernel_size, self.names
        return [TensorSpec("in_proj", n["in_proj"], (3 * H, H)),
                TensorSpec("conv", n["conv"], (H, L), INIT_CONV, KEEP_SMALL, file_shape=(H, 1, L)),
                TensorSpec("out_proj", n["out_proj"], (H, H))]

    def bind(self, tensors):
        self.in_proj, self.out_proj = tensors["in_proj"], tensors["out_proj"]
        self.conv = tensors["conv"].reshape(self.hidden_size, self.kernel_size).contiguous()

    def forward(self, ctx, x, cache, owns_cache=True):
        bcx = linear(x, self.in_proj)
        y = kernels.short_conv(bcx, self.conv, cache.tensors[0], ctx.cu_seqlens, ctx.seg_start,
                               ctx.seg_slot, ctx.row_seg)
        return linear(y, self.out_proj, out_dtype=torch.float32)


register_mixer("short_conv", ShortConv)
