"""Grouped-query attention mixer over the paged cache
(snowllm/models/lfm2/layers.py:36-70; snowllm/models/qwen3_5/layers.py:122-135).

q, k, v are one fused product; a second kernel applies the per-head RMSNorm of q and k, the
position encoding, and writes k and v into the cache pages; then the rows attend over the pages:
prompt portions (bfloat16, head sizes 64 and 128) in 64-row tiles on the tensor cores, all other
rows one by one with their keys split into chunks.
``window`` keeps the last ``window`` keys only (None: all).  A layer that reads another layer's
cache (``owns_cache`` False) projects q alone and writes nothing."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import kernels, linear
from . import attention_plan as plan
from .base import Part
from .registry import lookup, register_mixer
from .spec import INIT_ONES, KEEP_SMALL, PagedKVSpec, TensorSpec


class Attention(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "rope_cache", "attention", "attention_mma", "attention_tc")

    def __init__(self, dtype, names, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qk_norm_eps: float | None, position: dict, window: int | None = None,
                 scale: float | None = None):
        super().__init__(dtype, names)
        if num_heads % num_kv_heads:
            raise ConfigError(f"num_heads={num_heads} is no multiple of num_kv_heads={num_kv_heads}")
        vector = 8 if dtype == torch.bfloat16 else 4      # cache rows are copied in 16-byte vectors
        if head_dim % vector or head_dim > 512:
            raise ConfigError(f"head_dim={head_dim}: the attention kernels take multiples of {vector} up to 512 "
                              f"in {dtype}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.qk_norm_eps, self.window = head_dim, qk_norm_eps, window
        self.scale = head_dim ** -0.5 if scale is None else scale
        pos = dict(position)
        self.position = lookup("position", pos.pop("kind"))(**pos)
        self.wqkv = self.wq = self.wo = self.q_norm = self.k_norm = None

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def declare(self, has):
        H, hd, n = self.hidden_size, self.head_dim, self.names
        specs = [TensorSpec("q_proj", n["q_proj"], (self.num_heads * hd, H)),
                 TensorSpec("k_proj", n["k_proj"], (self.num_kv_heads * hd, H)),
                 TensorSpec("v_proj", n["v_proj"], (self.num_kv_heads * hd, H)),
                 TensorSpec("out_proj", n["out_proj"], (H, self.num_heads * hd))]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec("q_norm", n["q_norm"], (hd,), INIT_ONES, KEEP_SMALL),
                      TensorSpec("k_norm", n["k_norm"], (hd,), INIT_ONES, KEEP_SMALL)]
        return specs

    def bind(self, tensors):
        self.wqkv = torch.cat((tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]), 0).contiguous()
        self.wq = self.wqkv[: self.num_heads * self.head_dim]
        self.wo = tensors["out_proj"]
        self.q_norm, self.k_norm = tensors.get("q_norm"), tensors.get("k_norm")
        if self.q_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def forward(self, ctx, x, cache, owns_cache=True):
        qkv = linear(x, self.wqkv if owns_cache else self.wq)
        inv_freq, rot_dim = self.position.rotary(x.device)
        q = kernels.qk_norm_rope_cache(
            qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, inv_freq, rot_dim, ctx.positions,
            ctx.row_seg, cache.block_table, cache.page_size, cache.pool, self.num_heads,
            self.num_kv_heads, self.head_dim, write_kv=owns_cache)
        ctx.tap("attention_q", q)
        o = torch.empty(ctx.M, self.num_heads * self.head_dim, dtype=q.dtype, device=q.device)
        ctx.tap("attention_o", o)            # filled by the launches below
        rows = rows_host = None
        if kernels.attention_prefill_ok(q) and max(ctx.host_seg_len) >= plan.PREFILL_MIN_ROWS:
            # prompt portions on the tensor cores; rows of short segments (decoded tokens) row by row
            if kernels.attention_prefill_tc_ok(q, cache.page_size):
                tiles, rows, rows_host = plan.split(ctx, kernels.PREFILL_TC_TILE_ROWS)
                kernels.attention_prefill_tc(q, cache.pool, cache.block_table, cache.page_size, tiles, self.scale,
                                             o, window=self.window)
            else:
                tiles, rows, rows_host = plan.split(ctx, kernels.PREFILL_TILE_ROWS)
                kernels.attention_prefill(q, cache.pool, cache.block_table, cache.page_size, tiles, self.scale, o,
                                          window=self.window)
            if not rows_host:
                return linear(o, self.wo, out_dtype=torch.float32)
        served = ctx.M if rows_host is None else len(rows_host)
        if kernels.attention_decode_mma_ok(q, self.num_kv_heads):
            # rows of decoded tokens on the tensor cores: keys in chunks of 256, merged in order
            num_chunks = plan.chunks(ctx, self.window, rows_host, kernels.DECODE_MMA_CHUNK)
            scratch = ctx.scratch(kernels.attention_scratch_bytes(
                served, self.num_heads, self.head_dim, num_chunks)) if num_chunks > 1 else None
            kernels.attention_decode_mma(q, cache.pool, cache.block_table, cache.page_size, ctx.positions,
                                         ctx.row_seg, self.scale, num_chunks, o, window=self.window,
                                         scratch=scratch, rows=rows)
            return linear(o, self.wo, out_dtype=torch.float32)
        chunk, num_chunks = plan.plan(ctx, self.window, rows_host)
        scratch = ctx.scratch(kernels.attention_scratch_bytes(
            served, self.num_heads, self.head_dim, num_chunks)) if num_chunks > 1 else None
        kernels.paged_attention(q, cache.pool, cache.block_table, cache.page_size, ctx.positions,
                                ctx.row_seg, self.scale, window=self.window, chunk=chunk,
                                num_chunks=num_chunks, scratch=scratch, out=o, rows=rows)
        return linear(o, self.wo, out_dtype=torch.float32)


register_mixer("attention", Attention)
