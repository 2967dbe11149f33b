"""Dense SwiGLU feed-forward: down(silu(gate x) * up x)
(snowllm/models/lfm2/layers.py:76-88; snowllm/ops/mlp.py:12-20).  Gate and up are one fused
product [2I, H] (rows interleaved by 8, so that the product's store applies SwiGLU); the down product leaves a float delta for the residual sum."""
from __future__ import annotations

import torch

from ..ops import interleave_gate_up, linear, linear_swiglu
from .base import Part
from .registry import register_ffn
from .spec import TensorSpec


class SwiGLU(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "elementwise")

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int):
        super().__init__(dtype, names)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.w13 = self.w2 = None

    def declare(self, has):
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec("gate", self.names["gate"], (I, H)),
                TensorSpec("up", self.names["up"], (I, H)),
                TensorSpec("down", self.names["down"], (H, I))]

    def bind(self, tensors):
        # gate and up rows interleaved by 8 where the width allows: the product then applies SwiGLU itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w13 = (interleave_gate_up(tensors["gate"], tensors["up"]) if self.interleaved
                    else torch.cat((tensors["gate"], tensors["up"]), 0).contiguous())
        self.w2 = tensors["down"]

    def forward(self, ctx, x):
        act = linear_swiglu(x, self.w13, self.interleaved)
        return linear(act, self.w2, out_dtype=torch.float32)


register_ffn("swiglu", SwiGLU)
