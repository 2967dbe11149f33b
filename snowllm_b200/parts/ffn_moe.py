"""Sigmoid-routed top-k experts, each a SwiGLU feed-forward, no shared expert
(snowllm/models/qwen3_5/layers.py:166-188; router formula tests/test_lfm2_reference.py:113-119;
tensor names and the fused / per-expert spellings snowllm/models/lfm2/weights.py:79-92).

Steps: router in float -> sort the (token, pick) pairs by expert -> grouped gate|up product over
the sorted rows (rows gathered from x) with SwiGLU at its store -> grouped down product (float) ->
weighted sum per token in pick order (left to the norm that follows: `kernels.ExpertSum`).  Only experts that own rows are read."""
from __future__ import annotations

import torch

from ..ops import grouped_linear, grouped_linear_swiglu, interleave_gate_up, kernels
from .base import Part
from .registry import register_ffn
from .spec import INIT_BIAS, KEEP_F32, KEEP_SMALL, TensorSpec


class SigmoidMoE(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "moe", "elementwise")

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int, num_experts: int,
                 top_k: int, norm_topk_prob: bool, use_expert_bias: bool, routed_scaling_factor: float):
        super().__init__(dtype, names)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top_k = num_experts, top_k
        self.norm_topk_prob, self.use_expert_bias = norm_topk_prob, use_expert_bias
        self.routed_scaling_factor = routed_scaling_factor
        self.router = self.bias = self.w13 = self.w2 = None
        self._fused = False
        self._ticket = None            # the counter of the one-launch front end (zero between launches)

    def declare(self, has):
        H, I, E = self.hidden_size, self.intermediate_size, self.num_experts
        n = self.names
        specs = [TensorSpec("router", n["router"], (E, H), keep=KEEP_SMALL)]
        if self.use_expert_bias:
            specs.append(TensorSpec("expert_bias", n["expert_bias"], (E,), INIT_BIAS, KEEP_F32))
        self._fused = has(n["fused_gate_up"])
        if self._fused:
            specs += [TensorSpec("gate_up", n["fused_gate_up"], (E, 2 * I, H)),
                      TensorSpec("down", n["fused_down"], (E, H, I))]
        else:
            for e in range(E):
                p = f"{n['experts']}{e}."
                specs += [TensorSpec(f"gate.{e}", p + n["expert_gate"], (I, H)),
                          TensorSpec(f"up.{e}", p + n["expert_up"], (I, H)),
                          TensorSpec(f"down.{e}", p + n["expert_down"], (H, I))]
        return specs

    def bind(self, tensors):
        E = self.num_experts
        self.router = tensors["router"]
        self.bias = tensors.get("expert_bias") if self.use_expert_bias else None
        if self._fused:
            gate, up = tensors["gate_up"].chunk(2, dim=1)
            self.w2 = tensors["down"].contiguous()
        else:
            gate = torch.stack([tensors[f"gate.{e}"] for e in range(E)])
            up = torch.stack([tensors[f"up.{e}"] for e in range(E)])
            self.w2 = torch.stack([tensors[f"down.{e}"] for e in range(E)]).contiguous()
        # gate and up rows interleaved by 8 where the width allows: the product then applies SwiGLU itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w13 = interleave_gate_up(gate, up) if self.interleaved else torch.cat((gate, up), 1).contiguous()

    def bytes_read(self, bound, picked=None):
        """Router and bias whole; of the experts only those that were picked (``picked`` None: all)."""
        experts = sum(n for name, n in bound.items() if name.split(".")[0] in ("gate", "up", "down", "gate_up"))
        rest = sum(bound.values()) - experts
        share = 1.0 if picked is None else min(picked, self.num_experts) / self.num_experts
        return rest + int(experts * share)

    def route(self, x):
        return kernels.moe_route(x, self.router, self.bias, self.top_k, self.norm_topk_prob,
                                 self.routed_scaling_factor)

    def forward_from_residual(self, ctx, residual, delta, norm):
        """The norm that precedes this feed-forward, the router and the sort in one launch, for the few rows
        of a decode step (csrc/moe.cu: norm_route_sort_kernel); None when this step or this norm is not
        one it takes, and the block then runs the norm and ``forward`` one after the other."""
        weight, eps = getattr(norm, "weight", None), getattr(norm, "eps", None)
        if getattr(norm, "fusable_rms", False) is not True or weight is None or eps is None:
            return None
        if not kernels.FUSE_ROUTER or not kernels.norm_route_sort_ok(residual, delta, weight, self.router, self.top_k):
            return None
        if self._ticket is None or self._ticket.device != residual.device:
            self._ticket = torch.zeros(1, dtype=torch.int32, device=residual.device)
        x, *routed = kernels.norm_route_sort(residual, delta, weight, eps, self.dtype, self.router, self.bias,
                                             self.top_k, self.norm_topk_prob, self.routed_scaling_factor,
                                             self._ticket)
        if ctx is not None:
            ctx.tap("ffn_in", x)
        return self._experts(ctx, x, *routed)

    def forward(self, ctx, x):
        return self._experts(ctx, x, *kernels.moe_route_sort(
            x, self.router, self.bias, self.top_k, self.norm_topk_prob, self.routed_scaling_factor))

    def _experts(self, ctx, x, ids, weights, offsets, pair_pos, sorted_pair):
        M, k = x.shape[0], self.top_k
        if ctx is not None:
            ctx.tap("moe_route", ids)
            ctx.tap("moe_route_input", x)
        cap = min(M, M * k)          # an expert gets a token at most once
        act = grouped_linear_swiglu(x, self.w13, offsets, M * k, cap, sorted_pair, k, self.interleaved)
        y = grouped_linear(act, self.w2, offsets, M * k, cap, out_dtype=torch.float32)
        return kernels.ExpertSum(y, pair_pos, weights)     # the norm that follows adds it into the residual


register_ffn("sigmoid_moe", SigmoidMoE)
