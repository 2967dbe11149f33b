"""Token embedding and output head (snowllm/models/embedding.py:10-19;
snowllm/models/qwen3_5/layers.py:209-228: logits are float whatever the compute dtype)."""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import Part
from .registry import register_embedding, register_head
from .spec import TensorSpec


class Embedding(Part):
    libraries = ("elementwise",)

    def __init__(self, dtype, names, *, vocab_size: int, hidden_size: int):
        super().__init__(dtype, names)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.vocab_size, self.hidden_size))]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def bytes_read(self, bound, picked=None):
        return 0        # a step gathers one row per token: nothing beside the matrices

    def forward(self, ctx):
        """The float residual stream [M, H] of the step's tokens."""
        return kernels.embedding(ctx.token_ids, self.weight, pending=ctx.pending_tokens)


class LinearHead(Part):
    """logits = x . W^T in float.  ``tied``: W is the embedding table, and no tensor is declared."""
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2")

    def __init__(self, dtype, names, *, vocab_size: int, hidden_size: int, tied: bool):
        super().__init__(dtype, names)
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, tied
        self.weight = None

    def declare(self, has):
        if self.tied:
            return []
        return [TensorSpec("weight", self.names["weight"], (self.vocab_size, self.hidden_size))]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def bytes_read(self, bound, picked=None):
        # tied: nothing was declared here, yet the whole table is read as the head
        return self.weight.numel() * self.weight.element_size() if self.weight is not None else 0

    def forward(self, ctx, x):
        return linear(x, self.weight, out_dtype=torch.float32)


register_embedding("embedding", Embedding)
register_head("linear_head", LinearHead)
