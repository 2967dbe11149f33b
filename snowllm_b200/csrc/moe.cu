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
    if (k > 32 && ((j & 31) == 31 || j == k - 1)) {
      // flush this round of up to 32 picks; the normaliser is applied in a second pass
      const int base = j & ~31;
      if (base + lane <= j) {
        ids[base + lane] = my_id;
        wts[base + lane] = my_w;
      }
    }
  }
  const float mul = (norm_topk ? 1.f / (wsum + 1e-6f) : 1.f);
  if (k <= 32) {                   // one round: every pick is in a lane's registers; written once, normalised
    if (lane < k) {
      ids[lane] = my_id;
      wts[lane] = (norm_topk ? my_w * mul : my_w) * scaling;
    }
    return;
  }
  __syncwarp();
  for (int j = lane; j < k; j += 32) {
    float w = wts[j];
    w = norm_topk ? w * mul : w;
    wts[j] = w * scaling;
  }
}

// Eight consecutive elements as floats, by 16-byte loads.
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// x . w over H elements by one warp; every lane gets the sum.  Lane l owns the elements
// [8l, 8l + 8) of every run of 256 and adds them in ascending order, then the lanes' sums meet in a
// butterfly: the order depends on H alone, never on the launch.  vec: both rows are 16-byte aligned.
template <typename T, typename W>
__device__ __forceinline__ float warp_dot(const T* __restrict__ x, const W* __restrict__ w, int H, int lane,
                                          bool vec) {
  float acc = 0.f;
  int done = 0;
  if (vec) {
    done = H & ~7;
#pragma unroll 4
    for (int i = lane * 8; i < done; i += 256) {
      float xv[8], wv[8];
      load8<T>(x + i, xv);
      load8<W>(w + i, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(xv[j], wv[j], acc);
    }
  }
  for (int i = done + lane; i < H; i += 32) acc = fmaf(to_f<T>(x[i]), to_f<W>(w[i]), acc);
  return warp_sum(acc);
}

// One block per token, one warp per expert (in turns when there are more experts than warps).
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, SmallVec wr, const float* __restrict__ bias,
                                 int* __restrict__ topk_ids, float* __restrict__ topk_w, int H, int E,
                                 int k, int norm_topk, float scaling, int vec) {
  pdl_begin();
  extern __shared__ float sh[];
  float* prob = sh;              // E
  float* score = prob + E;       // E
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const T* xr = x + (size_t)m * H;
  for (int e = warp; e < E; e += nwarp) {
    const float acc = wr.is_f32
        ? warp_dot<T, float>(xr, static_cast<const float*>(wr.p) + (size_t)e * H, H, lane, vec)
        : warp_dot<T, bf16>(xr, static_cast<const bf16*>(wr.p) + (size_t)e * H, H, lane, vec);
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

// logits[m, e] = x[m] . wr[e], one warp per (token, expert): the few tokens of a decode step spread
// over many blocks, where one block per token would pull the whole router matrix through one SM.
// The same dot product as moe_route_kernel's, so a token's logits do not depend on the path.
template <typename T>
__global__ void moe_logits_kernel(const T* __restrict__ x, SmallVec wr, float* __restrict__ logits, int H,
                                  int E, int vec) {
  pdl_begin();
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * (blockDim.x >> 5) + warp;
  if (e >= E) return;
  const T* xr = x + (size_t)m * H;
  const float acc = wr.is_f32
      ? warp_dot<T, float>(xr, static_cast<const float*>(wr.p) + (size_t)e * H, H, lane, vec)
      : warp_dot<T, bf16>(xr, static_cast<const bf16*>(wr.p) + (size_t)e * H, H, lane, vec);
  if (lane == 0) logits[(size_t)m * E + e] = acc;
}

// One warp per token: probabilities and selection from float logits that a matrix product left, [M, E]
// or (transposed) [E, M].
// planes > 1: the logits are the sum of that many planes of [M, E] (a product split along K), added here in
// plane order.
__global__ void moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                int* __restrict__ topk_ids, float* __restrict__ topk_w, int M, int E, int k,
                                int norm_topk, float scaling, int transposed, int planes) {
  pdl_begin();
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int m = blockIdx.x * nwarp + warp;
  if (m >= M) return;
  float* prob = sh + (size_t)warp * 2 * E;
  float* score = prob + E;
  for (int e = lane; e < E; e += 32) {
    float x = transposed ? logits[(size_t)e * M + m] : logits[(size_t)m * E + e];
    if (planes > 1) {
      x += 0.f;                                          // the sum starts from zero, as the product's own sum does
      for (int q = 1; q < planes; ++q) x += logits[(size_t)q * M * E + (size_t)m * E + e];
    }
    const float p = 1.f / (1.f + expf(-x));
    prob[e] = p;
    score[e] = bias ? p + bias[e] : p;
  }
  __syncwarp();
  select_topk(prob, score, topk_ids + (size_t)m * k, topk_w + (size_t)m * k, E, k, norm_topk, scaling, lane);
}

SNK_API int snk_moe_topk(const float* logits, const float* bias, int* topk_ids, float* topk_w, int M, int E,
                         int k, int norm_topk, float scaling, int transposed, int planes, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E || planes < 1 || (planes > 1 && transposed)) return SNK_ERR_SIZE;
  const int warps = 4;
  snk_launch(moe_topk_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), (size_t)warps * 2 * E * sizeof(float), stream, 
      logits, bias, topk_ids, topk_w, M, E, k, norm_topk, scaling, transposed, planes);
  SNK_LAUNCH_CHECK();
  return 0;
}

SNK_API int snk_moe_route(const void* x, const void* wr, int wr_is_f32, const float* bias,
                          int* topk_ids, float* topk_w, int M, int H, int E, int k, int norm_topk,
                          float scaling, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(2 * E) * sizeof(float);
  SmallVec w{wr, wr_is_f32};
  const size_t xsz = dtype == SNK_F32 ? 4 : 2, wsz = wr_is_f32 ? 4 : 2;
  const int vec = ((uintptr_t)x % 16 == 0) && ((uintptr_t)wr % 16 == 0) && ((H * xsz) % 16 == 0) &&
                  ((H * wsz) % 16 == 0);
  SNK_DISPATCH(dtype, {
    // one warp per expert where it fits: the few rows of a decode step would otherwise leave most
    // of the GPU idle.  A dot product's order does not depend on the number of warps.
    const int threads = E >= 32 ? 1024 : (E >= 16 ? 512 : (E >= 8 ? 256 : ROUTE_THREADS));
    snk_launch(moe_route_kernel<T>, dim3(M), dim3(threads), smem, stream, static_cast<const T*>(x), w, bias, topk_ids,
                                                            topk_w, H, E, k, norm_topk, scaling, vec);
  });
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
// One block sorts all (token, j) pairs by expert.  offsets[E+1]: first sorted row of each
// expert; pair_pos[p]: sorted row of pair p = m*k + j; sorted_pair[r]: the pair at row r.
// Where a pair lands inside its expert's rows may vary from run to run; no value depends
// on it, since each row is computed on its own.
__device__ __forceinline__ void sort_pairs(const int* __restrict__ topk_ids, int* __restrict__ offsets,
                                           int* __restrict__ pair_pos, int* __restrict__ sorted_pair, int pairs,
                                           int E, int* cnt) {
  int* off = cnt + E;            // cnt: E counts, then E+1 offsets
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  // Up to SORT_KEEP pairs per thread stay in registers between the two passes, and their ids are all asked
  // for before the first is used: one trip to memory instead of one per pair and pass.
  constexpr int SORT_KEEP = 8;
  int ids[SORT_KEEP], place[SORT_KEEP];
  const bool keep = pairs <= SORT_KEEP * (int)blockDim.x;
  if (keep) {
#pragma unroll
    for (int i = 0; i < SORT_KEEP; ++i) {
      const int p = threadIdx.x + i * blockDim.x;
      int e = p < pairs ? topk_ids[p] : 0;
      ids[i] = e < 0 ? 0 : (e >= E ? E - 1 : e);
    }
#pragma unroll
    for (int i = 0; i < SORT_KEEP; ++i)
      if ((int)(threadIdx.x + i * blockDim.x) < pairs) place[i] = atomicAdd(&cnt[ids[i]], 1);
  } else {
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      int e = topk_ids[p];
      e = e < 0 ? 0 : (e >= E ? E - 1 : e);
      pair_pos[p] = atomicAdd(&cnt[e], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { off[e] = run; run += cnt[e]; }
    off[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  if (keep) {
#pragma unroll
    for (int i = 0; i < SORT_KEEP; ++i) {
      const int p = threadIdx.x + i * blockDim.x;
      if (p < pairs) {
        const int r = off[ids[i]] + place[i];
        pair_pos[p] = r;
        sorted_pair[r] = p;
      }
    }
    return;
  }
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    int e = topk_ids[p];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    const int r = off[e] + pair_pos[p];
    pair_pos[p] = r;
    sorted_pair[r] = p;
  }
}

__global__ void moe_sort_kernel(const int* __restrict__ topk_ids, int* __restrict__ offsets,
                                int* __restrict__ pair_pos, int* __restrict__ sorted_pair, int pairs,
                                int E) {
  pdl_begin();
  extern __shared__ int cnt[];
  sort_pairs(topk_ids, offsets, pair_pos, sorted_pair, pairs, E, cnt);
}

// Selection and sort in one block, for the few tokens of a decode step: a warp per token selects from
// the logits, then the block sorts the pairs.  The picks and their places stay in shared memory until
// the end (each trip through global memory would cost more than the arithmetic between two of them).
__global__ void moe_topk_sort_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                     int* __restrict__ topk_ids, float* __restrict__ topk_w,
                                     int* __restrict__ offsets, int* __restrict__ pair_pos,
                                     int* __restrict__ sorted_pair, int M, int E, int k, int norm_topk,
                                     float scaling) {
  pdl_begin();
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int pairs = M * k;
  int* ids_s = reinterpret_cast<int*>(sh);              // [pairs]
  int* pos_s = ids_s + pairs;                           // [pairs]
  float* work = reinterpret_cast<float*>(pos_s + pairs);
  float* prob = work + (size_t)warp * 2 * E;
  float* score = prob + E;
  for (int m = warp; m < M; m += nwarp) {
    for (int e = lane; e < E; e += 32) {
      const float p = 1.f / (1.f + expf(-logits[(size_t)m * E + e]));
      prob[e] = p;
      score[e] = bias ? p + bias[e] : p;
    }
    __syncwarp();
    select_topk(prob, score, ids_s + (size_t)m * k, topk_w + (size_t)m * k, E, k, norm_topk, scaling, lane);
    __syncwarp();
  }
  __syncthreads();
  sort_pairs(ids_s, offsets, pos_s, sorted_pair, pairs, E, reinterpret_cast<int*>(work));
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    topk_ids[p] = ids_s[p];
    pair_pos[p] = pos_s[p];
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

// Few rows: logits by one warp per (token, expert), then selection and sort in one block.
// logits: float scratch [M, E].  Refuses (SNK_ERR_SIZE) what does not fit one block's shared memory;
// the caller then takes snk_moe_route and snk_moe_sort.
SNK_API int snk_moe_route_sort(const void* x, const void* wr, int wr_is_f32, const float* bias, float* logits,
                               int* topk_ids, float* topk_w, int* offsets, int* pair_pos, int* sorted_pair,
                               int M, int H, int E, int k, int norm_topk, float scaling, int dtype,
                               cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E || M > 1024) return SNK_ERR_SIZE;
  const int warps = M < 32 ? M : 32;
  size_t smem = (size_t)warps * 2 * E * sizeof(float);
  const size_t sort_smem = (size_t)(2 * E + 1) * sizeof(int);
  if (smem < sort_smem) smem = sort_smem;
  smem += (size_t)2 * M * k * sizeof(int);               // the picks and their places
  if (smem > 48 * 1024) return SNK_ERR_SIZE;
  SmallVec w{wr, wr_is_f32};
  const size_t xsz = dtype == SNK_F32 ? 4 : 2, wsz = wr_is_f32 ? 4 : 2;
  const int vec = ((uintptr_t)x % 16 == 0) && ((uintptr_t)wr % 16 == 0) && ((H * xsz) % 16 == 0) &&
                  ((H * wsz) % 16 == 0);
  const int lw = 4;              // experts per block of the logits kernel
  SNK_DISPATCH(dtype, snk_launch(moe_logits_kernel<T>, dim3(M, (E + lw - 1) / lw), dim3(lw * 32), 0, stream,
                                 static_cast<const T*>(x), w, logits, H, E, vec));
  SNK_LAUNCH_CHECK();
  snk_launch(moe_topk_sort_kernel, dim3(1), dim3(warps * 32), smem, stream, logits, bias, topk_ids, topk_w,
             offsets, pair_pos, sorted_pair, M, E, k, norm_topk, scaling);
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
