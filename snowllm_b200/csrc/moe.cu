// Routed feed-forward: sigmoid router with top-k, token -> expert sort, weighted combine.
//
//   logits = u_f32 . Wr^T (float);  p = sigmoid(logits);  the k largest of p + bias select
//   (the bias only selects; equal scores go to the lower expert index);  w = p[sel];
//   w /= (sum w + 1e-6) when norm_topk_prob;  w *= routed_scaling_factor
//   (tests/test_lfm2_reference.py:113-119; snowllm/models/lfm2/weights.py:79-81)
//   out[m] = sum_j w[m,j] * expert_{sel[m,j]}(u[m])      (snowllm/models/qwen3_5/layers.py:176-188)
//
// The expert products themselves are grouped matrix products over rows sorted by expert;
// this file makes the sort (offsets per expert, position of each (token, j) pair) and the
// final weighted sum, which walks j = 0..k-1 in order and uses no atomics.
#include "common.cuh"

#define ROUTE_THREADS 128
#define ROUTE_MAX_EXPERTS 1024

// The k largest of score[] (ties to the lower index, NaN never wins) by one warp; weights from prob[],
// normalised by (sum + 1e-6) when asked, times the scaling factor.  score[] is consumed.
__device__ __forceinline__ void select_topk(float* prob, float* score, int* ids, float* wts, int E, int k,
                                            int norm_topk, float scaling, int lane) {
  float wsum = 0.f;
  float my_w = 0.f;              // lane j keeps the weight of pick j (k <= 32 per round)
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = score[e];
      // NaN never wins; ties keep the lower index
      if (s > best || (s == best && e < best_e)) { best = s; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (best_e == 0x7fffffff) best_e = j < E ? j : 0;   // every score NaN: fall back to index order
    const float p = prob[best_e];
    wsum += p;
    if (lane == 0) score[best_e] = -INFINITY;
    __syncwarp();
    if (lane == (j & 31)) { my_w = p; my_id = best_e; }
    if ((j & 31) == 31 || j == k - 1) {
      // flush this round of up to 32 picks; the normaliser is applied in a second pass
      const int base = j & ~31;
      if (base + lane <= j) {
        ids[base + lane] = my_id;
        wts[base + lane] = my_w;
      }
    }
  }
  __syncwarp();
  const float mul = (norm_topk ? 1.f / (wsum + 1e-6f) : 1.f);
  for (int j = lane; j < k; j += 32) {
    float w = wts[j];
    w = norm_topk ? w * mul : w;
    wts[j] = w * scaling;
  }
}

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, SmallVec wr, const float* __restrict__ bias,
                                 int* __restrict__ topk_ids, float* __restrict__ topk_w, int H, int E,
                                 int k, int norm_topk, float scaling) {
  pdl_begin();
  extern __shared__ float sh[];
  float* xs = sh;                // H
  float* prob = xs + H;          // E
  float* score = prob + E;       // E
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const T* xr = x + (size_t)m * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) xs[i] = to_f<T>(xr[i]);
  __syncthreads();
  for (int e = warp; e < E; e += nwarp) {
    float acc = 0.f;
    for (int i = lane; i < H; i += 32) acc = fmaf(xs[i], wr[(size_t)e * H + i], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      const float p = 1.f / (1.f + expf(-acc));
      prob[e] = p;
      score[e] = bias ? p + bias[e] : p;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  select_topk(prob, score, topk_ids + (size_t)m * k, topk_w + (size_t)m * k, E, k, norm_topk, scaling, lane);
}

// One warp per token: probabilities and selection from float logits [M, E] that a matrix product left.
__global__ void moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                int* __restrict__ topk_ids, float* __restrict__ topk_w, int M, int E, int k,
                                int norm_topk, float scaling) {
  pdl_begin();
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int m = blockIdx.x * nwarp + warp;
  if (m >= M) return;
  float* prob = sh + (size_t)warp * 2 * E;
  float* score = prob + E;
  for (int e = lane; e < E; e += 32) {
    const float p = 1.f / (1.f + expf(-logits[(size_t)m * E + e]));
    prob[e] = p;
    score[e] = bias ? p + bias[e] : p;
  }
  __syncwarp();
  select_topk(prob, score, topk_ids + (size_t)m * k, topk_w + (size_t)m * k, E, k, norm_topk, scaling, lane);
}

SNK_API int snk_moe_topk(const float* logits, const float* bias, int* topk_ids, float* topk_w, int M, int E,
                         int k, int norm_topk, float scaling, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E) return SNK_ERR_SIZE;
  const int warps = 4;
  snk_launch(moe_topk_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), (size_t)warps * 2 * E * sizeof(float), stream, 
      logits, bias, topk_ids, topk_w, M, E, k, norm_topk, scaling);
  SNK_LAUNCH_CHECK();
  return 0;
}

SNK_API int snk_moe_route(const void* x, const void* wr, int wr_is_f32, const float* bias,
                          int* topk_ids, float* topk_w, int M, int H, int E, int k, int norm_topk,
                          float scaling, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(H + 2 * E) * sizeof(float);
  if (smem > 200 * 1024) return SNK_ERR_SIZE;
  SmallVec w{wr, wr_is_f32};
  SNK_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // one warp per expert where it fits: the few rows of a decode step would otherwise leave most
    // of the GPU idle.  A dot product's order does not depend on the number of warps.
    const int threads = E >= 32 ? 1024 : (E >= 16 ? 512 : (E >= 8 ? 256 : ROUTE_THREADS));
    snk_launch(moe_route_kernel<T>, dim3(M), dim3(threads), smem, stream, static_cast<const T*>(x), w, bias, topk_ids,
                                                            topk_w, H, E, k, norm_topk, scaling);
  });
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// One block sorts all (token, j) pairs by expert.  offsets[E+1]: first sorted row of each
// expert; pair_pos[p]: sorted row of pair p = m*k + j; sorted_pair[r]: the pair at row r.
// Where a pair lands inside its expert's rows may vary from run to run; no value depends
// on it, since each row is computed on its own.
__global__ void moe_sort_kernel(const int* __restrict__ topk_ids, int* __restrict__ offsets,
                                int* __restrict__ pair_pos, int* __restrict__ sorted_pair, int pairs,
                                int E) {
  pdl_begin();
  extern __shared__ int cnt[];   // E counts, then E+1 offsets
  int* off = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    int e = topk_ids[p];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    pair_pos[p] = atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { off[e] = run; run += cnt[e]; }
    off[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    int e = topk_ids[p];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    const int r = off[e] + pair_pos[p];
    pair_pos[p] = r;
    sorted_pair[r] = p;
  }
}

SNK_API int snk_moe_sort(const int* topk_ids, int* offsets, int* pair_pos, int* sorted_pair,
                         int pairs, int E, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (E <= 0 || E > 4096) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(2 * E + 1) * sizeof(int);
  snk_launch(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, topk_ids, offsets, pair_pos, sorted_pair, pairs, E);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// out[m,:] = sum_j w[m,j] * y[pair_pos[m*k+j], :]   (float in, float out)
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_pos,
                                   const float* __restrict__ topk_w, float* __restrict__ out, int H,
                                   int k) {
  pdl_begin();
  const int m = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j)
      acc = fmaf(topk_w[(size_t)m * k + j], y[(size_t)pair_pos[(size_t)m * k + j] * H + i], acc);
    out[(size_t)m * H + i] = acc;
  }
}

SNK_API int snk_moe_combine(const float* y, const int* pair_pos, const float* topk_w, float* out,
                            int M, int H, int k, cudaStream_t stream) {
  if (M <= 0) return 0;
  snk_launch(moe_combine_kernel, dim3(M), dim3(H >= 1024 ? 256 : 128), 0, stream, y, pair_pos, topk_w, out, H, k);
  SNK_LAUNCH_CHECK();
  return 0;
}
