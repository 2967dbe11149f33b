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
#include <algorithm>

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
// GLOBAL_IDS: the ids lie in global memory and may have been written by other blocks of this launch, so they
// are read through L2 (ld.global.cg; never to be used on the shared-memory ids of moe_topk_sort_kernel).
template <bool GLOBAL_IDS = false>
__device__ __forceinline__ int pair_id(const int* p) {
  if constexpr (GLOBAL_IDS) return __ldcg(p);
  else return *p;
}

template <bool GLOBAL_IDS = false>
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
      int e = p < pairs ? pair_id<GLOBAL_IDS>(topk_ids + p) : 0;
      ids[i] = e < 0 ? 0 : (e >= E ? E - 1 : e);
    }
#pragma unroll
    for (int i = 0; i < SORT_KEEP; ++i)
      if ((int)(threadIdx.x + i * blockDim.x) < pairs) place[i] = atomicAdd(&cnt[ids[i]], 1);
  } else {
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      int e = pair_id<GLOBAL_IDS>(topk_ids + p);
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
    int e = pair_id<GLOBAL_IDS>(topk_ids + p);
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
// The front of a routed feed-forward for the few rows of a decode step, in ONE launch instead of three
// (norm, logits, selection + sort): a block per row
//   1. adds the delta into the float residual (a tensor, or the experts' outputs of the layer before, still
//      in pieces: sum_j w[m, j] * y[pos[m*k + j]], j in order), normalises, stores x in the compute dtype
//      (the arithmetic and its order are add_rmsnorm_kernel's, csrc/elementwise.cu);
//   2. forms the router's logits from x as stored, a warp per expert in turns, each dot product in
//      warp_dot's order (a row's logits are the same numbers as on the other paths);
//   3. selects (warp 0), and
//   4. takes a ticket; the block that draws the last one sorts all rows' pairs by expert and puts the
//      ticket counter back to zero.  Nobody waits for anybody.
// x . w as warp_dot forms it, with x as floats in shared memory.
// Eight consecutive elements as floats from shared memory (load8 reads through the read-only global path).
template <typename T> __device__ __forceinline__ void load8_shared(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8_shared<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8_shared<bf16>(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// SHARED_W: the weight row lies in shared memory (brought there ahead of time), else in global memory.
template <typename W, bool SHARED_W>
__device__ __forceinline__ float warp_dot_shared(const float* __restrict__ xs, const W* __restrict__ w, int H,
                                                 int lane, bool vec) {
  float acc = 0.f;
  int done = 0;
  if (vec) {
    done = H & ~7;
#pragma unroll 4
    for (int i = lane * 8; i < done; i += 256) {
      float wv[8];
      if constexpr (SHARED_W) load8_shared<W>(w + i, wv);
      else load8<W>(w + i, wv);
      const float4 a = *reinterpret_cast<const float4*>(xs + i), b = *reinterpret_cast<const float4*>(xs + i + 4);
      acc = fmaf(a.x, wv[0], acc); acc = fmaf(a.y, wv[1], acc); acc = fmaf(a.z, wv[2], acc); acc = fmaf(a.w, wv[3], acc);
      acc = fmaf(b.x, wv[4], acc); acc = fmaf(b.y, wv[5], acc); acc = fmaf(b.z, wv[6], acc); acc = fmaf(b.w, wv[7], acc);
    }
  }
  for (int i = done + lane; i < H; i += 32) acc = fmaf(xs[i], to_f<W>(w[i]), acc);
  return warp_sum(acc);
}

template <typename T>
__global__ void __launch_bounds__(512)
norm_route_sort_kernel(float* __restrict__ residual, const float* __restrict__ delta, SmallVec gamma,
                       T* __restrict__ x_out, int H, float eps, const float* __restrict__ moe_y,
                       const int* __restrict__ prev_pos, const float* __restrict__ prev_w, int prev_k,
                       SmallVec wr, const float* __restrict__ bias, int* __restrict__ topk_ids,
                       float* __restrict__ topk_w, int* __restrict__ offsets, int* __restrict__ pair_pos,
                       int* __restrict__ sorted_pair, int M, int E, int k, int norm_topk, float scaling, int vec,
                       unsigned int* __restrict__ ticket, int stage_w) {
  extern __shared__ __align__(16) float xs[];            // max(H, 2E + 1) floats, then 33, then prob[E], score[E]
  const int span = max((H + 3) & ~3, (2 * E + 4) & ~3);
  float* red = xs + span;
  float* prob = red + 36;
  float* score = prob + ((E + 3) & ~3);                  // every piece starts on a 16-byte boundary
  unsigned char* w_stage = reinterpret_cast<unsigned char*>(score + ((E + 3) & ~3));   // stage_w: the router matrix
  if (stage_w) {
    // The router matrix is a constant: it is fetched into shared memory before the wait for the kernel
    // before this one, so the fetch runs while that kernel ends.
    const size_t bytes = (size_t)E * H * (wr.is_f32 ? 4 : 2);
    const unsigned char* src = static_cast<const unsigned char*>(wr.p);
    const unsigned dst0 = (unsigned)__cvta_generic_to_shared(w_stage);
    for (size_t off = (size_t)threadIdx.x * 16; off < bytes; off += (size_t)blockDim.x * 16)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + (unsigned)off), "l"(src + off));
    asm volatile("cp.async.commit_group;");
  }
  pdl_begin();
  __shared__ int is_last;
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  float4* xs4 = reinterpret_cast<float4*>(xs);
  float4* res4 = reinterpret_cast<float4*>(residual + (size_t)m * H);
  float ss = 0.f;
  if (moe_y) {
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < prev_k; ++j) {
        const float w = prev_w[(size_t)m * prev_k + j];
        const float4 y = reinterpret_cast<const float4*>(moe_y + (size_t)prev_pos[(size_t)m * prev_k + j] * H)[i];
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
      }
      float4 v = res4[i];
      v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
      res4[i] = v;
      xs4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  } else {
    const float4* d4 = delta ? reinterpret_cast<const float4*>(delta + (size_t)m * H) : nullptr;
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 v = res4[i];
      if (d4) {
        const float4 e = d4[i];
        v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
        res4[i] = v;
      }
      xs4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = x_out + (size_t)m * H;
  for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
    const float4 v = xs4[i];
    const float a = v.x * inv * gamma[4 * i], b = v.y * inv * gamma[4 * i + 1], c = v.z * inv * gamma[4 * i + 2],
                d = v.w * inv * gamma[4 * i + 3];
    store4<T>(o + 4 * i, a, b, c, d);
    // the router reads x as it was stored
    xs4[i] = make_float4(to_f<T>(from_f<T>(a)), to_f<T>(from_f<T>(b)), to_f<T>(from_f<T>(c)), to_f<T>(from_f<T>(d)));
  }
  if (stage_w) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int e = warp; e < E; e += nwarp) {
    float acc;
    if (stage_w)
      acc = wr.is_f32
          ? warp_dot_shared<float, true>(xs, reinterpret_cast<const float*>(w_stage) + (size_t)e * H, H, lane, true)
          : warp_dot_shared<bf16, true>(xs, reinterpret_cast<const bf16*>(w_stage) + (size_t)e * H, H, lane, true);
    else
      acc = wr.is_f32
          ? warp_dot_shared<float, false>(xs, static_cast<const float*>(wr.p) + (size_t)e * H, H, lane, vec)
          : warp_dot_shared<bf16, false>(xs, static_cast<const bf16*>(wr.p) + (size_t)e * H, H, lane, vec);
    if (lane == 0) {
      const float p = 1.f / (1.f + expf(-acc));
      prob[e] = p;
      score[e] = bias ? p + bias[e] : p;
    }
  }
  __syncthreads();
  if (warp == 0) {
    select_topk(prob, score, topk_ids + (size_t)m * k, topk_w + (size_t)m * k, E, k, norm_topk, scaling, lane);
    __syncwarp();
    if (lane == 0) {
      __threadfence();                                   // this row's picks before its ticket
      is_last = atomicAdd(ticket, 1u) == (unsigned int)(M - 1);
    }
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();                                       // the other rows' picks after their tickets
  sort_pairs<true>(topk_ids, offsets, pair_pos, sorted_pair, M * k, E, reinterpret_cast<int*>(xs));
  if (threadIdx.x == 0) *ticket = 0u;                    // ready for the next launch
}

// ticket: one unsigned int of device memory that is zero before the first launch (the kernel leaves it zero).
// Refuses (SNK_ERR_SIZE / SNK_ERR_ALIGN) what it does not take; the caller then runs the three kernels.
SNK_API int snk_norm_route_sort(float* residual, const float* delta, const void* gamma, int gamma_is_f32,
                                void* x_out, int H, float eps, const float* moe_y, const int* prev_pos,
                                const float* prev_w, int prev_k, const void* wr, int wr_is_f32, const float* bias,
                                int* topk_ids, float* topk_w, int* offsets, int* pair_pos, int* sorted_pair,
                                int M, int E, int k, int norm_topk, float scaling, int dtype, unsigned int* ticket,
                                cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_EXPERTS || k <= 0 || k > E || k > 32 || H <= 0 || H % 4 || H > 32768 || M > 1024)
    return SNK_ERR_SIZE;
  if (M * k > 8 * 512 || (moe_y && prev_k <= 0)) return SNK_ERR_SIZE;
  if ((uintptr_t)residual % 16 || (uintptr_t)delta % 16 || (uintptr_t)x_out % 16 || (uintptr_t)moe_y % 16 ||
      (uintptr_t)gamma % 4)
    return SNK_ERR_ALIGN;
  const size_t wsz = wr_is_f32 ? 4 : 2;
  const int vec = ((uintptr_t)wr % 16 == 0) && ((H * wsz) % 16 == 0);
  const int span = std::max((H + 3) & ~3, (2 * E + 4) & ~3);
  size_t smem = (size_t)(span + 36 + 2 * ((E + 3) & ~3)) * sizeof(float);
  if (smem > 200 * 1024) return SNK_ERR_SIZE;
  // the router matrix in shared memory when it fits beside the rest (16-byte rows, so that a row's dot product
  // keeps the vector path's order)
  const size_t w_bytes = (size_t)E * H * wsz;
  const int stage_w = vec && smem + w_bytes <= 200 * 1024;
  if (stage_w) smem += w_bytes;
  SmallVec g{gamma, gamma_is_f32}, w{wr, wr_is_f32};
  SNK_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_route_sort_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // the block size of add_rmsnorm_kernel for this H, so that a row's sum of squares is formed the same way
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    snk_launch(norm_route_sort_kernel<T>, dim3(M), dim3(threads), smem, stream, residual, delta, g,
               static_cast<T*>(x_out), H, eps, moe_y, prev_pos, prev_w, prev_k, w, bias, topk_ids, topk_w, offsets,
               pair_pos, sorted_pair, M, E, k, norm_topk, scaling, vec, ticket, stage_w);
  });
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
