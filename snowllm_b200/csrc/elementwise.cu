// Embedding gather, fused residual-add + RMSNorm, SwiGLU activation.
//
// Embedding: h[m,:] = E[ids[m],:]                      (snowllm/ops/embedding.py:12-25)
// RMSNorm:   y = x * rsqrt(mean(x^2) + eps) * weight    (snowllm/ops/norm.py:11-30)
// SwiGLU:    out = silu(gate) * up                      (snowllm/ops/mlp.py:12-20)
// Both are evaluated in float and rounded to the compute dtype once, at the store (SnowLLM's
// bf16 kernels also round the normalised value before the weight, and silu before the product;
// those extra roundings are left out).  The residual stream is float, so the residual sum is a
// 32-bit sum.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// A negative id -(i + 1) stands for pending[i]: a token that an earlier launch sampled and that the host
// has not read yet (the step that follows a sampled token can then be launched before the token is known).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ pending, int num_pending,
                                 const T* __restrict__ table, float* __restrict__ out, int H, int V) {
  pdl_begin();
  const int m = blockIdx.x;
  int id = ids[m];
  if (id < 0 && pending != nullptr && -(id + 1) < num_pending) id = pending[-(id + 1)];
  const bool ok = id >= 0 && id < V;     // the host checks ids; a bad one reads nothing
  const T* row = table + (size_t)(ok ? id : 0) * H;
  float* o = out + (size_t)m * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_f<T>(row[i]) : 0.f;
}

SNK_API int snk_embedding(const int* ids, const int* pending, int num_pending, const void* table, float* out,
                          int M, int H, int V, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  SNK_DISPATCH(dtype, snk_launch(embedding_kernel<T>, dim3(M), dim3(threads), 0, stream,
                          ids, pending, num_pending, static_cast<const T*>(table), out, H, V));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// One block per output row.  rows == nullptr: row r is residual row r; delta (if any) is
// added into the residual and the sum is written back.  rows != nullptr: output row r
// normalises residual[rows[r]] + delta[rows[r]] and nothing is written back.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                   SmallVec gamma, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int vec4,
                                   const float* __restrict__ moe_y, const int* __restrict__ pair_pos,
                                   const float* __restrict__ topk_w, int k) {
  pdl_begin();
  extern __shared__ __align__(16) float xs[];   // H floats + 33 for the reduction
  float* red = xs + ((H + 3) & ~3);
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* res = residual + src * H;
  const float* d = delta ? delta + src * H : nullptr;
  float ss = 0.f;
  T* o = out + (size_t)r * H;
  if (moe_y) {
    // The delta is the routed experts' weighted sum, formed here instead of by a kernel of its own:
    // sum_j w[src, j] * y[pair_pos[src*k + j], :], j in order (the rows are 16-byte aligned).
    float4* xs4 = reinterpret_cast<float4*>(xs);
    float4* res4 = reinterpret_cast<float4*>(res);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < k; ++j) {
        const float w = topk_w[src * k + j];
        const float4 y = reinterpret_cast<const float4*>(moe_y + (size_t)pair_pos[src * k + j] * H)[i];
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
      }
      float4 v = res4[i];
      v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
      if (!rows) res4[i] = v;
      xs4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);      // one fixed order of the squares in every path
      ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      const float4 v = xs4[i];
      store4<T>(o + 4 * i, v.x * inv * gamma[4 * i], v.y * inv * gamma[4 * i + 1], v.z * inv * gamma[4 * i + 2],
                v.w * inv * gamma[4 * i + 3]);
    }
    return;
  }
  if (vec4) {                                   // H a multiple of 4 and 16-byte aligned rows
    float4* xs4 = reinterpret_cast<float4*>(xs);
    float4* res4 = reinterpret_cast<float4*>(res);
    const float4* d4 = reinterpret_cast<const float4*>(d);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 v = res4[i];
      if (d) {
        const float4 e = d4[i];
        v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
        if (!rows) res4[i] = v;
      }
      xs4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);      // one fixed order of the squares in every path
      ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      const float4 v = xs4[i];
      store4<T>(o + 4 * i, v.x * inv * gamma[4 * i], v.y * inv * gamma[4 * i + 1], v.z * inv * gamma[4 * i + 2],
                v.w * inv * gamma[4 * i + 3]);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = res[i];
    if (d) {
      v += d[i];
      if (!rows) res[i] = v;
    }
    xs[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = from_f<T>(xs[i] * inv * gamma[i]);
}

#define NORM_REG_MIN_ROWS 160   // up to here every row's wide block finds an SM of its own at once (measured at 64 rows,
                                // the 64-request decode step: 4.5 -> 3.7 us a launch, 5.61 -> 5.57 ms a step)

// The same for rows of 16-byte vectors that fit the block's registers: a thread holds ITERS vectors of
// its row, all of their loads are in flight together, and nothing but the sum of squares passes through
// shared memory.  Small blocks (128 threads for H up to 4096), so that many rows are in flight on an SM.
__device__ __forceinline__ float4 gamma4(const SmallVec& g, int i) {
  if (g.is_f32) return __ldg(reinterpret_cast<const float4*>(g.p) + i);
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(g.p) + i);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}

template <typename T, int ITERS>
__global__ void add_rmsnorm_reg_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                       SmallVec gamma, T* __restrict__ out, const int* __restrict__ rows,
                                       int H, float eps, const float* __restrict__ moe_y,
                                       const int* __restrict__ pair_pos, const float* __restrict__ topk_w, int k) {
  pdl_begin();
  __shared__ float red[33];
  const int r = blockIdx.x, n4 = H / 4;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float4* res4 = reinterpret_cast<float4*>(residual + src * H);
  float4 v[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    v[it] = i < n4 ? res4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (moe_y) {
    // the routed experts' weighted sum, j in order, then the residual sum: as the kernel above forms it
    float4 acc[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) acc[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int JU = ITERS <= 2 ? 4 : 2;                  // picks whose rows are in flight together
    for (int j0 = 0; j0 < k; j0 += JU) {
      float w[JU];
      const float4* y4[JU];
#pragma unroll
      for (int u = 0; u < JU; ++u) {
        const int j = min(j0 + u, k - 1);
        w[u] = topk_w[src * k + j];
        y4[u] = reinterpret_cast<const float4*>(moe_y + (size_t)pair_pos[src * k + j] * H);
      }
      float4 y[JU][ITERS];
#pragma unroll
      for (int u = 0; u < JU; ++u)
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          const int i = threadIdx.x + it * blockDim.x;
          y[u][it] = (i < n4 && j0 + u < k) ? y4[u][i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int u = 0; u < JU; ++u) {
        if (j0 + u < k) {
#pragma unroll
          for (int it = 0; it < ITERS; ++it) {
            acc[it].x = fmaf(w[u], y[u][it].x, acc[it].x); acc[it].y = fmaf(w[u], y[u][it].y, acc[it].y);
            acc[it].z = fmaf(w[u], y[u][it].z, acc[it].z); acc[it].w = fmaf(w[u], y[u][it].w, acc[it].w);
          }
        }
      }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      v[it].x += acc[it].x; v[it].y += acc[it].y; v[it].z += acc[it].z; v[it].w += acc[it].w;
    }
  } else if (delta) {
    const float4* d4 = reinterpret_cast<const float4*>(delta + src * H);
    float4 e[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = threadIdx.x + it * blockDim.x;
      e[it] = i < n4 ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      v[it].x += e[it].x; v[it].y += e[it].y; v[it].z += e[it].z; v[it].w += e[it].w;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < n4) {
      if (!rows && (moe_y || delta)) res4[i] = v[it];
      ss = fmaf(v[it].x, v[it].x, ss); ss = fmaf(v[it].y, v[it].y, ss);
      ss = fmaf(v[it].z, v[it].z, ss); ss = fmaf(v[it].w, v[it].w, ss);
    }
  }
  float4 g[ITERS];                                          // the weights are on their way while the sum is formed
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    g[it] = i < n4 ? gamma4(gamma, i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = out + (size_t)r * H;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < n4)
      store4<T>(o + 4 * i, v[it].x * inv * g[it].x, v[it].y * inv * g[it].y, v[it].z * inv * g[it].z,
                v[it].w * inv * g[it].w);
  }
}

// moe_y (may be null): instead of delta, add sum_j topk_w[row, j] * moe_y[pair_pos[row*k + j], :].
SNK_API int snk_add_rmsnorm(float* residual, const float* delta, const void* gamma,
                            int gamma_is_f32, void* out, const int* rows, int R, int H,
                            float eps, int dtype, const float* moe_y, const int* pair_pos,
                            const float* topk_w, int k, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || H > 65536) return SNK_ERR_SIZE;
  if (moe_y && (H % 4 || (uintptr_t)moe_y % 16 || (uintptr_t)residual % 16 || (uintptr_t)out % 16 || k <= 0))
    return SNK_ERR_ALIGN;
  // The block size depends on H alone, so a row's statistics never depend on the batch.
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
  SmallVec g{gamma, gamma_is_f32};
  const int vec4 = H % 4 == 0 && (uintptr_t)residual % 16 == 0 && (uintptr_t)delta % 16 == 0 &&
                   (uintptr_t)out % 16 == 0;
  // Many rows (prompt portions): rows of vectors that fit the registers of a small block, many blocks
  // on an SM (measured at 2048 x 2048: the experts' sum 26 -> 21 us).  The few rows of a decode step keep
  // the wide block below, whose single round of loads has the shorter latency (3.2 against 4.5 us).
  // Either block's size depends on H alone; which of the two sums a row's squares depends on R only
  // through this threshold.
  const int reg_threads = H <= 4096 ? 128 : 256;
  if (R >= NORM_REG_MIN_ROWS && vec4 && (uintptr_t)gamma % 16 == 0 && H / 4 <= reg_threads * 8) {
    const int iters = (H / 4 + reg_threads - 1) / reg_threads;
#define NORM_REG(I_)                                                                                      \
  snk_launch(add_rmsnorm_reg_kernel<T, I_>, dim3(R), dim3(reg_threads), 0, stream, residual, delta, g,    \
             static_cast<T*>(out), rows, H, eps, moe_y, pair_pos, topk_w, k)
    SNK_DISPATCH(dtype, {
      if (iters <= 1) NORM_REG(1);
      else if (iters <= 2) NORM_REG(2);
      else if (iters <= 4) NORM_REG(4);
      else NORM_REG(8);
    });
#undef NORM_REG
    SNK_LAUNCH_CHECK();
    return 0;
  }
  SNK_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    snk_launch(add_rmsnorm_kernel<T>, dim3(R), dim3(threads), smem, stream, residual, delta, g,
                                                        static_cast<T*>(out), rows, H, eps, vec4, moe_y, pair_pos,
                                                        topk_w, k);
  });
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// Residual update without a norm: residual += delta (used where no norm follows).
__global__ void add_kernel(float* __restrict__ residual, const float* __restrict__ delta, size_t n) {
  pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) residual[i] += delta[i];
}

SNK_API int snk_residual_add(float* residual, const float* delta, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  snk_launch(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, residual, delta, (size_t)n);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// gu: [M, 2I].  Plain: the gate in columns [0, I), the up projection in [I, 2I).  Interleaved: blocks of
// 16 columns, 8 gate columns then the 8 up columns of the same features (what the fused products use).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int interleaved) {
  pdl_begin();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t m = idx / I;
  const int i = (int)(idx - m * I);
  const size_t gcol = interleaved ? (size_t)(i / 8) * 16 + i % 8 : (size_t)i;
  const size_t ucol = interleaved ? gcol + 8 : (size_t)I + i;
  const float g = to_f<T>(gu[m * 2 * I + gcol]);
  const float u = to_f<T>(gu[m * 2 * I + ucol]);
  const float s = g / (1.f + expf(-g));
  out[idx] = from_f<T>(s * u);
}

SNK_API int snk_swiglu(const void* gu, void* out, int M, int I, int interleaved, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)M * I;
  if (total == 0) return 0;
  if (interleaved && I % 8) return SNK_ERR_SIZE;
  SNK_DISPATCH(dtype, snk_launch(swiglu_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 
                          static_cast<const T*>(gu), static_cast<T*>(out), I, total, interleaved));
  SNK_LAUNCH_CHECK();
  return 0;
}
