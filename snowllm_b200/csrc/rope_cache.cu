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

// The same work with 16-byte accesses, for head sizes of 16 bytes times a power of two and a rotation
// over the whole head: a lane owns VEC consecutive elements, LPH = hd / VEC lanes share a head, and a
// warp serves 32 / LPH heads at once.  The partner of element d (d +- hd/2) lies LPH/2 lanes away at the
// same place, so the rotation needs a shuffle and no shared memory.  A warp loads ROPE_UNROLL groups of
// heads before it uses the first.  Sums of squares: a lane's VEC elements in order, then a butterfly
// over the head's lanes; one order for every batch size, as this kernel serves all of them.
#define ROPE_UNROLL 3

template <typename T> struct RopeVec;
template <> struct RopeVec<float> {
  static constexpr int N = 4;
  using Raw = float4;
  static __device__ __forceinline__ void unpack(const Raw& t, float (&v)[4]) { v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  static __device__ __forceinline__ Raw pack(const float (&v)[4]) { return make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct RopeVec<bf16> {
  static constexpr int N = 8;
  using Raw = uint4;
  static __device__ __forceinline__ void unpack(const Raw& t, float (&v)[8]) {
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ Raw pack(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T>
__global__ void qk_norm_rope_cache_vec_kernel(
    const T* __restrict__ qkv, SmallVec q_gamma, SmallVec k_gamma, int has_norm, float eps,
    const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ block_table, int max_pages,
    int page_size, T* __restrict__ pool, T* __restrict__ q_out, int nh, int nkv, int hd,
    int write_kv) {
  pdl_begin();
  constexpr int VEC = RopeVec<T>::N;
  using Raw = typename RopeVec<T>::Raw;
  extern __shared__ float sh[];            // cos, then sin, of the row's hd / 2 angles
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int half = hd >> 1;
  float* cs_tab = sh;
  float* sn_tab = sh + half;
  const int lph = hd / VEC, hpw = 32 / lph;          // lanes per head, heads per warp
  const int total_heads = write_kv ? nh + 2 * nkv : nh;
  const int groups = (total_heads + hpw - 1) / hpw;
  const int sub = lane % lph, d0 = sub * VEC;
  const bool first_half = d0 < half;
  const int stride = warps * gridDim.y;
  const T* row = qkv + (size_t)m * total_heads * hd;
  Raw raw[ROPE_UNROLL];
  auto load = [&](int g0) {
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int head = (g0 + u * stride) * hpw + lane / lph;
      raw[u] = Raw{};
      if (g0 + u * stride < groups && head < total_heads)
        raw[u] = *reinterpret_cast<const Raw*>(row + (size_t)head * hd + d0);
    }
  };
  int g0 = blockIdx.y * warps + warp;
  load(g0);                                          // in flight while the row's angles are computed
  const int pos = positions[m];
  if (inv_freq != nullptr) {
    const float posf = (float)pos;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(posf * inv_freq[i], &sn_tab[i], &cs_tab[i]);
  }
  __syncthreads();
  for (; g0 < groups; g0 += ROPE_UNROLL * stride, load(g0)) {
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      if (g0 + u * stride >= groups) break;          // the same for every lane of the warp
      const int head = (g0 + u * stride) * hpw + lane / lph;
      const bool is_q = head < nh;
      const bool is_k = !is_q && head < nh + nkv;
      float x[VEC];
      RopeVec<T>::unpack(raw[u], x);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss += x[e] * x[e];
      if (has_norm) {
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (is_q || is_k) {
          const float inv = rsqrtf(ss / (float)hd + eps);
          const SmallVec& g = is_q ? q_gamma : k_gamma;
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[e] = x[e] * inv * g[d0 + e];
        }
      }
      if (inv_freq != nullptr) {
        const int i0 = first_half ? d0 : d0 - half;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float partner = __shfl_xor_sync(0xffffffffu, x[e], lph >> 1);
          if (is_q || is_k) {
            const float other = first_half ? -partner : partner;
            x[e] = x[e] * cs_tab[i0 + e] + other * sn_tab[i0 + e];
          }
        }
      }
      if (head < total_heads) {
        T* dst;
        if (is_q) {
          dst = q_out + ((size_t)m * nh + head) * hd;
        } else {
          const int kvh = is_k ? head - nh : head - nh - nkv;
          const int page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
          dst = pool + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + pos % page_size) * hd;
        }
        *reinterpret_cast<Raw*>(dst + d0) = RopeVec<T>::pack(x);
      }
    }
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
  {
    const int vec = dtype == SNK_F32 ? 4 : 8;
    const int lph = hd / vec;
    const bool pow2 = lph >= 2 && lph <= 32 && (lph & (lph - 1)) == 0 && lph * vec == hd;
    const bool aligned = (uintptr_t)qkv % 16 == 0 && (uintptr_t)pool % 16 == 0 && (uintptr_t)q_out % 16 == 0;
    if (pow2 && aligned && (inv_freq == nullptr || rot_dim == hd)) {
      const int vwarps = 4, hpw = 32 / lph, groups = (total_heads + hpw - 1) / hpw;
      // few rows (decode): a row's groups of heads spread over several blocks, one group per warp
      dim3 vgrid(M, M < 64 ? (groups + vwarps - 1) / vwarps : 1);
      SmallVec vq{q_gamma, gamma_is_f32}, vk{k_gamma, gamma_is_f32};
      SNK_DISPATCH(dtype, snk_launch(qk_norm_rope_cache_vec_kernel<T>, dim3(vgrid), dim3(vwarps * 32),
                                     (size_t)hd * sizeof(float), stream, static_cast<const T*>(qkv), vq, vk,
                                     has_norm, eps, inv_freq, positions, row_seg, block_table, max_pages,
                                     page_size, static_cast<T*>(pool), static_cast<T*>(q_out), nh, nkv, hd,
                                     write_kv));
      SNK_LAUNCH_CHECK();
      return 0;
    }
  }
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
