// Causal grouped-query attention over the paged cache, for any mix of prompt portions and
// single decoded tokens in one launch.
//
//   s = (q . k) * scale over the request's cached keys with  lo <= key position <= query
//   position, lo = max(0, pos - window + 1) with a window, else 0; q head i reads kv head
//   i / (nh / nkv); softmax in float; o = softmax(s) v
//   (snowllm/models/lfm2/layers.py:36-70; tests/test_lfm2_long_attention.py:36-47)
//
// Work split: one block per (query row, kv head, key chunk); its warps are the q heads of
// that kv head, which share each tile of keys and values through shared memory.  Tiles of 32
// keys come in by 16-byte cp.async copies, three tiles in flight per block, straight from the
// pages in the cache dtype; keys outside the row's range are zero-filled, never read.  Key
// chunks are aligned to absolute positions, so what a row computes depends on its own
// position and on the chunk length only, never on the rest of the batch.  With more than
// one chunk the blocks write partial (o, max, sum) to scratch and a second kernel merges
// them in chunk order.
//
// Pool layout: [page, 2 (k, v), kv head, page_size, head_dim].
#include "common.cuh"

#define ATT_TILE 32            // keys per tile: one per lane
#define ATT_MAX_WARPS 8        // q heads handled by one block
#define ATT_MAX_DPL 16         // head_dim <= 512
#define ATT_STAGES 3           // tiles in flight per block (cp.async ring)

// 16-byte vectors of the cache dtype, unpacked to float.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    // a bfloat16 is the upper half of a float
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;                // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// DPL: output elements per lane, head_dim <= 32 * DPL (a compile-time bound keeps the inner loops
// free of dead iterations).
template <typename T, int DPL>
__global__ void paged_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ pool, const int* __restrict__ block_table,
    int max_pages, int page_size, const int* __restrict__ positions, const int* __restrict__ row_seg,
    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
    int hd, int window, int chunk, int num_chunks, float scale, const int* __restrict__ row_list) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char sh_raw[];
  constexpr int VEC = Vec16<T>::N;
  const int group = nh / nkv;
  const int heads_per_block = blockDim.x >> 5;
  const int blocks_per_kv = (group + heads_per_block - 1) / heads_per_block;
  const int m = row_list ? row_list[blockIdx.x] : blockIdx.x;    // the row of the batch this block serves
  const int kvh = blockIdx.y / blocks_per_kv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head_in_group = (blockIdx.y % blocks_per_kv) * heads_per_block + warp;
  const bool active = head_in_group < group;
  const int head = kvh * group + head_in_group;

  const int pos = positions[m];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_chunk = lo / chunk;
  const int c = first_chunk + blockIdx.z;
  if ((long long)c * chunk > pos) return;                  // no key of this row in this chunk
  const int k_begin = max(lo, c * chunk);
  const int k_end = min(pos + 1, (c + 1) * chunk);         // exclusive

  // shared memory: [stages][k | v][ATT_TILE rows of hd*sizeof(T) + 16 bytes], then q as float
  const int row_bytes = hd * (int)sizeof(T);
  const int rstride = row_bytes + 16;                      // the pad keeps 16-byte row reads off one bank
  const int vecs_per_row = row_bytes / 16;
  const int tile_bytes = ATT_TILE * rstride;
  unsigned char* kv_smem = sh_raw;
  float* qs = reinterpret_cast<float*>(sh_raw + (size_t)ATT_STAGES * 2 * tile_bytes);

  if (active) {
    const T* qrow = q + ((size_t)m * nh + head) * hd;
    for (int d = lane; d < hd; d += 32) qs[warp * hd + d] = to_f<T>(qrow[d]) * scale;
  }
  const int* bt = block_table + (size_t)row_seg[m] * max_pages;
  const size_t page_stride = (size_t)2 * nkv * page_size * hd;
  const size_t v_off = (size_t)nkv * page_size * hd;

  // Tiles start at multiples of ATT_TILE counted from the chunk's absolute start.
  const int t_first = c * chunk + ((k_begin - c * chunk) / ATT_TILE) * ATT_TILE;
  const int ntiles = (k_end - t_first + ATT_TILE - 1) / ATT_TILE;

  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = t_first + tile * ATT_TILE;
      unsigned char* ks = kv_smem + (size_t)(tile % ATT_STAGES) * 2 * tile_bytes;
      unsigned char* vs = ks + tile_bytes;
      for (int v = threadIdx.x; v < ATT_TILE * vecs_per_row; v += blockDim.x) {
        const int j = v / vecs_per_row, cv = v - j * vecs_per_row;
        const int kp = t0 + j;
        const bool valid = kp >= k_begin && kp < k_end;
        const T* src = pool;
        if (valid) {
          const int page = bt[kp / page_size];
          src = pool + (size_t)page * page_stride + ((size_t)kvh * page_size + kp % page_size) * hd + cv * VEC;
        }
        cp_async16(ks + j * rstride + cv * 16, src, valid);
        cp_async16(vs + j * rstride + cv * 16, valid ? src + v_off : src, valid);
      }
    }
    cp_async_commit();
  };

  float mx = -INFINITY, l = 0.f;
  float o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;

#pragma unroll
  for (int s = 0; s < ATT_STAGES - 1; ++s) issue(s);
  for (int tile = 0; tile < ntiles; ++tile) {
    cp_async_wait<ATT_STAGES - 2>();
    __syncthreads();                                       // tile is in; everyone is done with tile - 1
    issue(tile + ATT_STAGES - 1);
    if (!active) continue;
    const int t0 = t_first + tile * ATT_TILE;
    const unsigned char* ks = kv_smem + (size_t)(tile % ATT_STAGES) * 2 * tile_bytes;
    const unsigned char* vs = ks + tile_bytes;
    const int kp = t0 + lane;
    const bool valid = kp >= k_begin && kp < k_end;
    float s = 0.f;
    const float* qw = qs + warp * hd;
    const unsigned char* kr = ks + lane * rstride;
    for (int cv = 0; cv < vecs_per_row; ++cv) {
      float f[VEC];
      Vec16<T>::unpack(*reinterpret_cast<const uint4*>(kr + cv * 16), f);
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qw + cv * VEC + e);
        s = fmaf(q4.x, f[e], s);
        s = fmaf(q4.y, f[e + 1], s);
        s = fmaf(q4.z, f[e + 2], s);
        s = fmaf(q4.w, f[e + 3], s);
      }
    }
    s = valid ? s : -INFINITY;
    float p, corr;
    if constexpr (sizeof(T) == 2) {
      // bfloat16: base-2 exponents against a whole-number reference, P rounded to bfloat16 for P V as the
      // tensor-core kernels do (csrc/attention_mma.cu, "Rounding of P"); the row sum keeps the unrounded values
      s *= 1.4426950408889634f;
      const float m_new = fmaxf(mx, ceilf(warp_max(s)));   // finite: each tile run has a valid key
      corr = exp2f(mx - m_new);                            // a power of two; 0 on the first tile
      p = valid ? exp2f(s - m_new) : 0.f;
      l = l * corr + warp_sum(p);
      p = __bfloat162float(__float2bfloat16_rn(p));
      mx = m_new;
    } else {
      const float tmax = warp_max(s);
      const float m_new = fmaxf(mx, tmax);                 // finite: each tile run has a valid key
      corr = expf(mx - m_new);                             // exp(-inf) = 0 on the first tile
      p = valid ? expf(s - m_new) : 0.f;
      l = l * corr + warp_sum(p);
      mx = m_new;
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] *= corr;
    const T* vrow = reinterpret_cast<const T*>(vs);
    const int vstride = rstride / (int)sizeof(T);
    for (int j = 0; j < ATT_TILE; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[i] = fmaf(pj, to_f<T>(vrow[j * vstride + d]), o[i]);
      }
    }
  }
  cp_async_wait<0>();
  if (!active) return;
  if (num_chunks == 1) {
    const float inv = 1.f / l;
    T* orow = out + ((size_t)m * nh + head) * hd;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) orow[d] = from_f<T>(o[i] * inv);
    }
  } else {
    const size_t slot = ((size_t)blockIdx.x * nh + head) * num_chunks + blockIdx.z;
    float* po = part_o + slot * hd;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) po[d] = o[i];
    }
    if (lane == 0) {
      part_ml[slot * 2] = sizeof(T) == 2 ? mx * 0.6931471805599453f : mx;   // the merge works with natural exponents
      part_ml[slot * 2 + 1] = l;
    }
  }
}

// Merge the chunks of one (row, head).  The first warp finds the running maximum and the normaliser
// over the chunks (lanes take chunks in turns, then a butterfly).  The chunks are then cut into
// MERGE_ZG runs; a thread sums one element of the output over one run in chunk order, and the runs'
// sums are added in run order: many short chains of loads instead of one long one.
#define MERGE_ZG 4

template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       const int* __restrict__ positions, T* __restrict__ out, int nh,
                                       int hd, int window, int chunk, int num_chunks,
                                       const int* __restrict__ row_list) {
  pdl_begin();
  extern __shared__ float merge_sh[];                      // [MERGE_ZG][hd]
  __shared__ float s_mx, s_inv;
  const int m = row_list ? row_list[blockIdx.x] : blockIdx.x, head = blockIdx.y;
  const int pos = positions[m];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos / chunk - lo / chunk + 1;              // chunks this row really has
  const size_t base = ((size_t)blockIdx.x * nh + head) * num_chunks;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mx = -INFINITY;
    for (int z = lane; z < n; z += 32) mx = fmaxf(mx, part_ml[(base + z) * 2]);
    mx = warp_max(mx);
    float l = 0.f;
    for (int z = lane; z < n; z += 32) l += part_ml[(base + z) * 2 + 1] * expf(part_ml[(base + z) * 2] - mx);
    l = warp_sum(l);
    if (lane == 0) { s_mx = mx; s_inv = 1.f / l; }
  }
  __syncthreads();
  const float mx = s_mx, inv = s_inv;
  const int dthreads = blockDim.x / MERGE_ZG, zg = threadIdx.x / dthreads, dt = threadIdx.x % dthreads;
  const int per = (n + MERGE_ZG - 1) / MERGE_ZG;
  const int z0 = min(n, zg * per), z1 = min(n, z0 + per);
  for (int d = dt; d < hd; d += dthreads) {
    float acc = 0.f;
#pragma unroll 8
    for (int z = z0; z < z1; ++z)
      acc = fmaf(part_o[(base + z) * hd + d], expf(part_ml[(base + z) * 2] - mx), acc);
    merge_sh[zg * hd + d] = acc;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = merge_sh[d];
#pragma unroll
    for (int r = 1; r < MERGE_ZG; ++r) acc += merge_sh[r * hd + d];
    out[((size_t)m * nh + head) * hd + d] = from_f<T>(acc * inv);
  }
}

// Bytes of scratch the launch below needs for `num_chunks` > 1 (0 for one chunk).
SNK_API long long snk_paged_attention_scratch_bytes(int M, int nh, int hd, int num_chunks) {
  if (num_chunks <= 1) return 0;
  return (long long)M * nh * num_chunks * (hd + 2) * (long long)sizeof(float);
}

// row_list (may be null): the M rows of the batch to serve, when not all of them.
SNK_API int snk_paged_attention_rows(const void* q, const void* pool, const int* block_table,
                                     int max_pages, int page_size, const int* positions,
                                     const int* row_seg, void* out, void* scratch, int M, int nh,
                                     int nkv, int hd, int window, int chunk, int num_chunks,
                                     float scale, int dtype, const int* row_list, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nkv <= 0 || nh % nkv || hd <= 0 || hd > 32 * ATT_MAX_DPL) return SNK_ERR_SIZE;
  if (chunk <= 0 || chunk % ATT_TILE || num_chunks < 1 || num_chunks > 65535) return SNK_ERR_SIZE;
  if (num_chunks > 1 && scratch == nullptr) return SNK_ERR_SIZE;
  const int group = nh / nkv;
  const int warps = group < ATT_MAX_WARPS ? group : ATT_MAX_WARPS;
  const int blocks_per_kv = (group + warps - 1) / warps;
  if ((long long)nkv * blocks_per_kv > 65535) return SNK_ERR_SIZE;
  dim3 grid(M, nkv * blocks_per_kv, num_chunks);
  const size_t esz = dtype == SNK_F32 ? 4 : 2;
  if ((hd * esz) % 16 || ((uintptr_t)pool % 16)) return SNK_ERR_ALIGN;
  const size_t smem = (size_t)ATT_STAGES * 2 * ATT_TILE * (hd * esz + 16) + (size_t)warps * hd * sizeof(float);
  if (smem > 227 * 1024) return SNK_ERR_SIZE;
  float* part_o = static_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (size_t)M * nh * num_chunks * hd : nullptr;
#define ATT_LAUNCH(DPL_)                                                                             \
  do {                                                                                               \
    if (smem > 48 * 1024)                                                                            \
      cudaFuncSetAttribute(paged_attention_kernel<T, DPL_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                               \
    snk_launch(paged_attention_kernel<T, DPL_>, dim3(grid), dim3(warps * 32), smem, stream,                              \
        static_cast<const T*>(q), static_cast<const T*>(pool), block_table, max_pages, page_size,    \
        positions, row_seg, static_cast<T*>(out), part_o, part_ml, nh, nkv, hd, window, chunk,       \
        num_chunks, scale, row_list);                                                                \
  } while (0)
  SNK_DISPATCH(dtype, {
    if (hd <= 32) ATT_LAUNCH(1);
    else if (hd <= 64) ATT_LAUNCH(2);
    else if (hd <= 128) ATT_LAUNCH(4);
    else if (hd <= 256) ATT_LAUNCH(8);
    else ATT_LAUNCH(16);
  });
#undef ATT_LAUNCH
  SNK_LAUNCH_CHECK();
  if (num_chunks > 1) {
    dim3 mgrid(M, nh);
    const int threads = MERGE_ZG * (hd <= 32 ? 32 : (hd <= 64 ? 64 : 128));
    SNK_DISPATCH(dtype, snk_launch(attention_merge_kernel<T>, dim3(mgrid), dim3(threads),
                                   (size_t)MERGE_ZG * hd * sizeof(float), stream, 
                            part_o, part_ml, positions, static_cast<T*>(out), nh, hd, window,
                            chunk, num_chunks, row_list));
    SNK_LAUNCH_CHECK();
  }
  return 0;
}

// The second half of a chunked launch on its own: adds the chunks' partial results (scratch in the
// layout above) in chunk order.  For partials written by another kernel (csrc/attention_mma.cu).
SNK_API int snk_attention_merge(const void* scratch, const int* positions, void* out, int M, int nh, int hd,
                                int window, int chunk, int num_chunks, int dtype, const int* row_list,
                                cudaStream_t stream) {
  if (M <= 0 || num_chunks <= 1) return 0;
  const float* part_o = static_cast<const float*>(scratch);
  const float* part_ml = part_o + (size_t)M * nh * num_chunks * hd;
  dim3 mgrid(M, nh);
  const int threads = MERGE_ZG * (hd <= 32 ? 32 : (hd <= 64 ? 64 : 128));
  SNK_DISPATCH(dtype, snk_launch(attention_merge_kernel<T>, dim3(mgrid), dim3(threads),
                                 (size_t)MERGE_ZG * hd * sizeof(float), stream, 
                          part_o, part_ml, positions, static_cast<T*>(out), nh, hd, window, chunk, num_chunks,
                          row_list));
  SNK_LAUNCH_CHECK();
  return 0;
}

SNK_API int snk_paged_attention(const void* q, const void* pool, const int* block_table,
                                int max_pages, int page_size, const int* positions,
                                const int* row_seg, void* out, void* scratch, int M, int nh,
                                int nkv, int hd, int window, int chunk, int num_chunks,
                                float scale, int dtype, cudaStream_t stream) {
  return snk_paged_attention_rows(q, pool, block_table, max_pages, page_size, positions, row_seg, out, scratch,
                                  M, nh, nkv, hd, window, chunk, num_chunks, scale, dtype, nullptr, stream);
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (see attention_static.h for who needs it and its rules).
#include "attention_static.h"

#include <mutex>

// Scratch for the partial results of split rows.  In host code this name is only a handle for the
// symbol, not an address the GPU understands: its device address is looked up below, per device.
static __device__ __align__(256) unsigned char g_static_scratch[SNK_ATTENTION_STATIC_SCRATCH_BYTES];

#define SNK_STATIC_MAX_DEVICES 64

// Device address of g_static_scratch on the current device; looked up on the first call per device.
static int static_scratch_address(void** out) {
  static void* address[SNK_STATIC_MAX_DEVICES] = {nullptr};
  static std::mutex mu;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= SNK_STATIC_MAX_DEVICES) return SNK_ERR_STATIC_SETUP;
  std::lock_guard<std::mutex> lock(mu);
  if (address[device] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);      // resolves the symbol for the current device
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return SNK_ERR_STATIC_SETUP;
    address[device] = p;
  }
  *out = address[device];
  return 0;
}

SNK_API long long snk_paged_attention_static_need(int M, int nh, int hd, int num_chunks) {
  return snk_paged_attention_scratch_bytes(M, nh, hd, num_chunks);
}

SNK_API int snk_paged_attention_static(const void* q, const void* pool, const int* block_table, int max_pages,
                                       int page_size, const int* positions, const int* row_seg, void* out,
                                       int M, int nh, int nkv, int hd, int window, int chunk, int num_chunks,
                                       float scale, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (snk_paged_attention_scratch_bytes(M, nh, hd, num_chunks) > (long long)SNK_ATTENTION_STATIC_SCRATCH_BYTES)
    return SNK_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  // Every partial (o, max, sum) that the merge kernel reads is written by this call's first kernel, so
  // the array needs no clearing.  The regular entry point does the launches; it allocates nothing.
  return snk_paged_attention(q, pool, block_table, max_pages, page_size, positions, row_seg, out, scratch, M,
                             nh, nkv, hd, window, chunk, num_chunks, scale, dtype, stream);
}
