// Per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into the
// paged cache, in one pass over the fused qkv rows.
//
//   q, k: x * rsqrt(mean_hd(x^2) + eps) * weight   (snowllm/models/lfm2/layers.py:55-59)
//   rope: ang = pos * inv_freq[i] in float; split-half rotation over the first rot_dim
//         elements of the head: x'[i] = x[i] cos - x[i+h] sin; x'[i+h] = x[i+h] cos + x[i] sin
//         (snowllm/ops/rope.py:11-24; tests/test_lfm2.py:108-118); norm and rotation run in
//         float and the result is rounded to the compute dtype once, at the store
//   cache: k and v rows go to page block_table[seg][pos / P], offset pos % P
//         (snowllm/ops/cache.py:12-20).  Pool layout: [page, 2 (k, v), kv head, P, hd].
#include "common.cuh"

#define ROPE_MAX_PER_LANE 16   // head_dim <= 512

// PER: elements per lane, head_dim <= 32 * PER (a compile-time bound keeps the loops free of dead
// iterations).
template <typename T, int PER>
__global__ void qk_norm_rope_cache_kernel(
    const T* __restrict__ qkv, SmallVec q_gamma, SmallVec k_gamma, int has_norm, float eps,
    const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ block_table, int max_pages,
    int page_size, T* __restrict__ pool, T* __restrict__ q_out, int nh, int nkv, int hd,
    int write_kv) {
  pdl_begin();
  extern __shared__ float sh[];            // one head per warp: hd floats each; then cos, sin of the row
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int total_heads = write_kv ? nh + 2 * nkv : nh;
  float* cs_tab = sh + (size_t)warps * hd;
  float* sn_tab = cs_tab + (rot_dim >> 1);
  if (inv_freq != nullptr) {               // the row's angles once, for all of its heads
    const float posf = (float)positions[m];
    for (int i = threadIdx.x; i < (rot_dim >> 1); i += blockDim.x) sincosf(posf * inv_freq[i], &sn_tab[i], &cs_tab[i]);
  }
  __syncthreads();
  for (int head = blockIdx.y * warps + warp; head < total_heads; head += warps * gridDim.y) {
  float* buf = sh + (size_t)warp * hd;
  // A layer that reads another layer's cache projects q only: its rows hold no k, v.
  const int row_width = (write_kv ? nh + 2 * nkv : nh) * hd;
  const T* src = qkv + (size_t)m * row_width + (size_t)head * hd;

  const bool is_q = head < nh;
  const bool is_k = !is_q && head < nh + nkv;
  float x[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int d = lane + 32 * j;
    x[j] = d < hd ? to_f<T>(src[d]) : 0.f;
    ss += x[j] * x[j];
  }
  if (is_q || is_k) {
    if (has_norm) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)hd + eps);
      const SmallVec& g = is_q ? q_gamma : k_gamma;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) x[j] = x[j] * inv * g[d];
      }
    }
    if (inv_freq != nullptr && rot_dim > 0) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) buf[d] = x[j];
      }
      __syncwarp();
      const int half = rot_dim >> 1;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int d = lane + 32 * j;
        if (d < rot_dim) {
          const int i = d < half ? d : d - half;
          const float sn = sn_tab[i], cs = cs_tab[i];
          const float other = d < half ? -buf[d + half] : buf[d - half];
          x[j] = x[j] * cs + other * sn;
        }
      }
    }
  }
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)m * nh + head) * hd;
  } else {
    const int kvh = is_k ? head - nh : head - nh - nkv;
    const int pos = positions[m];
    const int page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
    dst = pool + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + pos % page_size) * hd;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int d = lane + 32 * j;
    if (d < hd) dst[d] = from_f<T>(x[j]);
  }
  __syncwarp();                              // buf is reused by the warp's next head
  }
}

SNK_API int snk_qk_norm_rope_cache(
    const void* qkv, const void* q_gamma, const void* k_gamma, int gamma_is_f32, int has_norm,
    float eps, const float* inv_freq, int rot_dim, const int* positions, const int* row_seg,
    const int* block_table, int max_pages, int page_size, void* pool, void* q_out, int M, int nh,
    int nkv, int hd, int write_kv, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (hd <= 0 || hd > 32 * ROPE_MAX_PER_LANE || rot_dim > hd || (rot_dim & 1)) return SNK_ERR_SIZE;
  const int total_heads = write_kv ? nh + 2 * nkv : nh;
  const int warps = total_heads >= 8 ? 8 : (total_heads >= 4 ? 4 : 2);
  // few rows (decode): the heads of a row spread over several blocks, one head per warp
  dim3 grid(M, M < 64 ? (total_heads + warps - 1) / warps : 1);
  const size_t smem = ((size_t)warps * hd + rot_dim) * sizeof(float);
  SmallVec qg{q_gamma, gamma_is_f32}, kg{k_gamma, gamma_is_f32};
#define ROPE_LAUNCH(PER_)                                                                            \
  snk_launch(qk_norm_rope_cache_kernel<T, PER_>, dim3(grid), dim3(warps * 32), smem, stream,                             \
      static_cast<const T*>(qkv), qg, kg, has_norm, eps, inv_freq, rot_dim, positions, row_seg,      \
      block_table, max_pages, page_size, static_cast<T*>(pool), static_cast<T*>(q_out), nh, nkv, hd, \
      write_kv)
  SNK_DISPATCH(dtype, {
    if (hd <= 32) ROPE_LAUNCH(1);
    else if (hd <= 64) ROPE_LAUNCH(2);
    else if (hd <= 128) ROPE_LAUNCH(4);
    else if (hd <= 256) ROPE_LAUNCH(8);
    else ROPE_LAUNCH(16);
  });
#undef ROPE_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
