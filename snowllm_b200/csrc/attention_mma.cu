// Causal grouped-query attention in bfloat16 on the tensor cores (mma.sync): a kernel for prompt
// portions and, below, one for the rows of decoded tokens.
//
// Prompt portions.
// One block takes 64 consecutive rows of one request's portion and one q head and walks that
// request's cached keys in tiles of 64, from the first key any of its rows may see to the last
// row's own position (flash attention: running max and sum per row in float, the output
// accumulator rescaled as the max moves).  S = Q K^T and O += P V are mma.sync m16n8k16 with
// float accumulation; each of the 4 warps owns 16 rows.  Keys and values come straight from the
// cache pages by 16-byte cp.async into two shared-memory stages (XOR-swizzled 16-byte chunks, so
// that ldmatrix reads are free of bank conflicts); nothing outside a row's range [lo, pos] enters
// its softmax, and key rows past the tile's last position are zero-filled, never read.
//
//   s = (q . k) * scale for lo <= key position <= query position, lo = max(0, pos - window + 1)
//   with a window, else 0; softmax in float; o = softmax(s) v        (snowllm/models/lfm2/layers.py:36-70;
//   tests/test_lfm2_long_attention.py:36-47)
//
// The tile order is fixed by positions alone, so a row's result does not depend on what else the
// launch holds.  Head sizes 64 and 128; other sizes and float32 go through csrc/attention.cu.
//
// Rounding of P.  P = 2^(s log2 e - m) is rounded to bfloat16 for the P V product (the row sum is taken from
// the unrounded values).  The reference m is the running maximum rounded UP to a whole number: whatever tile
// walk, chunking or kernel a row goes through, its references differ by whole numbers, the P values by exact
// powers of two, and the rounded mantissas are the same.  So which key gets which rounding error does not
// depend on how the keys were cut, every rescaling of O and of the row sum is exact, and a plain
// implementation can round P the same way (tests/plain_lfm2.py does).  All bfloat16 attention kernels of
// this engine follow the rule.
// Pool layout: [page, 2 (k, v), kv head, page_size, head_dim].
#include "tma.cuh"

#define FA_BQ 64
#define FA_BK 64
#define FA_WARPS 4

__device__ __forceinline__ void fa_cp_async16(uint32_t dst, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void fa_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void fa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void fa_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` of row `r` in a tile whose rows hold CHUNKS chunks.
template <int CHUNKS> __device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * CHUNKS + (c ^ (r & 7))) * 16u;
}

// tiles: int32 [n_tiles][4] = {segment, first row of the tile in the batch, rows in the tile (<= 64),
// position of the first row}.
template <int HD>
__global__ void __launch_bounds__(FA_WARPS * 32)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool,
                         const int* __restrict__ block_table, int max_pages, int page_size,
                         const int* __restrict__ tiles, bf16* __restrict__ out, int nh, int nkv, int window,
                         float scale_log2) {
  pdl_begin();
  constexpr int CH = HD / 8;                       // 16-byte chunks per row
  constexpr int KT = HD / 16;                      // k-steps of the QK^T product
  constexpr int NT = HD / 8;                       // n-tiles of the output
  extern __shared__ __align__(16) unsigned char fa_smem[];
  const uint32_t sm_q = (uint32_t)__cvta_generic_to_shared(fa_smem);
  const uint32_t sm_kv = sm_q + FA_BQ * HD * 2;    // [2 stages][k | v][FA_BK rows]
  constexpr uint32_t TILE_BYTES = FA_BK * HD * 2;

  const int* tile = tiles + (size_t)blockIdx.x * 4;
  const int seg = tile[0], row0 = tile[1], rows = tile[2], pos0 = tile[3];
  const int head = blockIdx.y;
  const int kvh = head / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* bt = block_table + (size_t)seg * max_pages;
  const size_t page_stride = (size_t)2 * nkv * page_size * HD;
  const size_t v_off = (size_t)nkv * page_size * HD;

  // keys this tile needs: from the first row's lower bound to the last row's position
  const int last_pos = pos0 + rows - 1;
  const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int k_first = (key_lo / FA_BK) * FA_BK;    // key tiles are aligned to absolute positions
  const int n_kt = (last_pos - k_first) / FA_BK + 1;

  // Q tile -> shared memory (rows past the portion's end are zero)
  for (int v = threadIdx.x; v < FA_BQ * CH; v += FA_WARPS * 32) {
    const int r = v / CH, c = v % CH;
    fa_cp_async16(sm_q + swz<CH>(r, c), q + ((size_t)(row0 + min(r, rows - 1)) * nh + head) * HD + c * 8, r < rows);
  }
  auto load_kv = [&](int kt) {
    if (kt < n_kt) {
      const int k0 = k_first + kt * FA_BK;
      const uint32_t ks = sm_kv + (uint32_t)(kt & 1) * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
      for (int v = threadIdx.x; v < FA_BK * CH; v += FA_WARPS * 32) {
        const int r = v / CH, c = v % CH;
        const int kp = k0 + r;
        const bool valid = kp <= last_pos;
        const bf16* src = pool;
        if (valid) {
          const int page = bt[kp / page_size];
          src = pool + (size_t)page * page_stride + ((size_t)kvh * page_size + kp % page_size) * HD + c * 8;
        }
        fa_cp_async16(ks + swz<CH>(r, c), src, valid);
        fa_cp_async16(vs + swz<CH>(r, c), valid ? src + v_off : src, valid);
      }
    }
    fa_commit();
  };
  load_kv(0);                                      // group 0: Q and the first key tile

  float acc_o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_o[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  uint32_t qf[KT][4];
  // positions and lower bounds of this thread's two rows (g and g + 8 of the warp's 16)
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
  const int lo_lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  const int lo_hi = window > 0 ? max(0, p_hi - window + 1) : 0;

  for (int kt = 0; kt < n_kt; ++kt) {
    load_kv(kt + 1);
    fa_wait<1>();
    __syncthreads();
    if (kt == 0) {
#pragma unroll
      for (int k = 0; k < KT; ++k) {
        const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * k + (lane >> 4);
        ldmatrix_x4(sm_q + swz<CH>(r, c), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
      }
    }
    const int k0 = k_first + kt * FA_BK;
    const uint32_t ks = sm_kv + (uint32_t)(kt & 1) * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    // a warp whose rows all lie before this key tile (causal), or behind it (window), skips it
    const int warp_first_pos = pos0 + warp * 16, warp_last_pos = min(warp_first_pos + 15, last_pos);
    const int warp_lo = window > 0 ? max(0, warp_first_pos - window + 1) : 0;
    const bool active = warp * 16 < rows && k0 <= warp_last_pos && k0 + FA_BK > warp_lo;
    if (active) {
      float s[FA_BK / 8][4];
#pragma unroll
      for (int i = 0; i < FA_BK / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
#pragma unroll
        for (int n = 0; n < FA_BK / 16; ++n) {      // two 8-key tiles per ldmatrix.x4
          uint32_t b0, b1, b2, b3;
          const int r = n * 16 + (lane & 7) + 8 * (lane >> 4), c = 2 * k + ((lane >> 3) & 1);
          ldmatrix_x4(ks + swz<CH>(r, c), b0, b1, b2, b3);
          fa_mma(s[2 * n], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
          fa_mma(s[2 * n + 1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
        }
      }
      // mask and running max: s[i] = {(row g, key 8i+2t), (g, 8i+2t+1), (g+8, 8i+2t), (g+8, 8i+2t+1)}
      float mx[2] = {row_max[0], row_max[1]};
#pragma unroll
      for (int i = 0; i < FA_BK / 8; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kp = k0 + 8 * i + 2 * t + (j & 1);
          const bool hi = j >= 2;
          const bool ok = hi ? (kp <= p_hi && kp >= lo_hi) : (kp <= p_lo && kp >= lo_lo);
          s[i][j] = ok ? s[i][j] * scale_log2 : -INFINITY;
          mx[hi] = fmaxf(mx[hi], s[i][j]);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        mx[h] = ceilf(mx[h]);                              // a whole power of two as the reference (see the file's head)
      }
      float alpha[2], base[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        base[h] = mx[h] == -INFINITY ? 0.f : mx[h];        // a row with nothing to see yet: exp2(-inf) = 0
        alpha[h] = exp2f(row_max[h] - base[h]);            // row_max = -inf on the first tile: 0
        row_max[h] = mx[h];
        row_sum[h] *= alpha[h];
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc_o[i][0] *= alpha[0]; acc_o[i][1] *= alpha[0];
        acc_o[i][2] *= alpha[1]; acc_o[i][3] *= alpha[1];
      }
      uint32_t pf[FA_BK / 16][4];
#pragma unroll
      for (int i = 0; i < FA_BK / 8; ++i) {
        const float p0 = exp2f(s[i][0] - base[0]), p1 = exp2f(s[i][1] - base[0]);
        const float p2 = exp2f(s[i][2] - base[1]), p3 = exp2f(s[i][3] - base[1]);
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);       // rows g: a0 (even 8-key tile), a2 (odd)
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);   // rows g+8: a1, a3
      }
#pragma unroll
      for (int kk = 0; kk < FA_BK / 16; ++kk) {
#pragma unroll
        for (int n = 0; n < NT / 2; ++n) {
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * n + (lane >> 4);
          ldmatrix_x4_trans(vs + swz<CH>(r, c), b0, b1, b2, b3);
          fa_mma(acc_o[2 * n], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
          fa_mma(acc_o[2 * n + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
        }
      }
    }
    __syncthreads();                               // everyone is done with this stage before it is refilled
  }
  fa_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }
  const float inv_lo = 1.f / row_sum[0], inv_hi = 1.f / row_sum[1];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int d = 8 * i + 2 * t;
    if (r_lo < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_lo) * nh + head) * HD + d) =
          pack_bf16(acc_o[i][0] * inv_lo, acc_o[i][1] * inv_lo);
    if (r_hi < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_hi) * nh + head) * HD + d) =
          pack_bf16(acc_o[i][2] * inv_hi, acc_o[i][3] * inv_hi);
  }
}

SNK_API int snk_attention_prefill(const void* q, const void* pool, const int* block_table, int max_pages,
                                  int page_size, const int* tiles, int n_tiles, void* out, int nh, int nkv,
                                  int hd, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh > 65535) return SNK_ERR_SIZE;
  if (hd != 64 && hd != 128) return SNK_ERR_SIZE;
  if (((uintptr_t)q % 16) || ((uintptr_t)pool % 16) || ((uintptr_t)out % 4)) return SNK_ERR_ALIGN;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tiles, nh);
  const size_t smem = (size_t)(FA_BQ + 4 * FA_BK) * hd * 2;
  const bf16 *qp = static_cast<const bf16*>(q), *pp = static_cast<const bf16*>(pool);
  bf16* op = static_cast<bf16*>(out);
  if (hd == 64) {
    snk_launch(attention_prefill_kernel<64>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, qp, pp, block_table, max_pages, page_size,
                                                                        tiles, op, nh, nkv, window, scale_log2);
  } else {
    cudaFuncSetAttribute(attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_prefill_kernel<128>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, qp, pp, block_table, max_pages, page_size,
                                                                         tiles, op, nh, nkv, window, scale_log2);
  }
  SNK_LAUNCH_CHECK();
  return 0;
}


// ---------------------------------------------------------------------------------------------
// The prompt kernel with keys and values brought in by TMA (see the decode kernel below for the map: a
// box is one page's rows of one kv head, 64 elements wide, 128-byte swizzle).  A ring of FP_STAGES key
// tiles: lanes of warp 0 issue the loads of tile kt + FP_STAGES - 1 while the warps work on tile kt, each
// stage with an mbarrier that counts its bytes.  Pages are loaded whole, so in the first and the last
// tile rows outside [key_lo, last_pos] hold whatever was there: their scores are replaced, never used,
// and their value rows are zeroed before use.  Only tiles that cross a row's causal or window edge apply
// masks.  Blocks take the tiles from the last (most keys) to the first.  For page sizes 8, 16, 32, 64.
#ifndef FP_STAGES
#define FP_STAGES 3
#endif
#ifndef FP_MIN_BLOCKS
#define FP_MIN_BLOCKS 1
#endif
#define FP_WAIT_NS 1000000000ull

__device__ int g_fa_status;

template <int HD>
__global__ void __launch_bounds__(FA_WARPS * 32, FP_MIN_BLOCKS)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q,
                             const int* __restrict__ block_table, int max_pages, int page_size,
                             const int* __restrict__ tiles, int n_tiles, bf16* __restrict__ out, int nh, int nkv,
                             int window, float scale_log2) {
  if (threadIdx.x == 0)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
  pdl_begin();
  constexpr int CH = HD / 8, KT = HD / 16, NT = HD / 8, PANELS = HD / 64;
  constexpr uint32_t PANEL = FA_BK * 128;                 // bytes of one 64-element panel of a key tile
  constexpr uint32_t STAGE = 2 * PANELS * PANEL;          // keys, then values
  extern __shared__ unsigned char fp_raw[];
  unsigned char* fp_smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fp_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sm_kv = (uint32_t)__cvta_generic_to_shared(fp_smem);       // [FP_STAGES][k | v][PANELS][64][64]
  const uint32_t sm_q = sm_kv + FP_STAGES * STAGE;                          // [64][HD], swz<CH>
  __shared__ uint64_t full[FP_STAGES];
  __shared__ int gave_up;                                 // a wait ran out: no more loads, no more waits

  const int* tile = tiles + (size_t)(n_tiles - 1 - blockIdx.x) * 4;
  const int seg = tile[0], row0 = tile[1], rows = tile[2], pos0 = tile[3];
  const int head = blockIdx.y;
  const int kvh = head / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* bt = block_table + (size_t)seg * max_pages;

  const int last_pos = pos0 + rows - 1;
  const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int k_first = (key_lo / FA_BK) * FA_BK;
  const int n_kt = (last_pos - k_first) / FA_BK + 1;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < FP_STAGES; ++i) mbar_init(&full[i], 1);
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int v = threadIdx.x; v < FA_BQ * CH; v += FA_WARPS * 32) {
    const int r = v / CH, c = v % CH;
    fa_cp_async16(sm_q + swz<CH>(r, c), q + ((size_t)(row0 + min(r, rows - 1)) * nh + head) * HD + c * 8, r < rows);
  }
  fa_commit();
  __syncthreads();                                        // the barriers are initialised

  // warp 0 issues tile kt's pages: those that hold a key of [key_lo, last_pos]
  auto issue = [&](int kt) {
    if (warp != 0 || kt >= n_kt) return;
    if (__any_sync(0xffffffffu, *const_cast<volatile int*>(&gave_up))) return;     // the warp as one
    const int k0 = k_first + kt * FA_BK;
    const int first_page = max(k0, key_lo) / page_size;
    const int n_pages = min(k0 + FA_BK - 1, last_pos) / page_size - first_page + 1;
    unsigned char* stage = fp_smem + (size_t)(kt % FP_STAGES) * STAGE;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // rows zeroed by threads before: ordered before the loads
    if (lane == 0) mbar_expect_tx(&full[kt % FP_STAGES], (uint32_t)n_pages * page_size * 128u * 2u * PANELS);
    __syncwarp();
    for (int i = lane; i < n_pages; i += 32) {
      const int page = bt[first_page + i];
      const int row = (first_page + i) * page_size - k0;
      const int y_k = ((page * 2) * nkv + kvh) * page_size, y_v = ((page * 2 + 1) * nkv + kvh) * page_size;
#pragma unroll
      for (int p = 0; p < PANELS; ++p) {
        tma_load_2d(stage + p * PANEL + row * 128, &map_kv, &full[kt % FP_STAGES], p * 64, y_k);
        tma_load_2d(stage + (PANELS + p) * PANEL + row * 128, &map_kv, &full[kt % FP_STAGES], p * 64, y_v);
      }
    }
  };
  auto tile_off = [](int r, int cc) -> uint32_t {
    return (uint32_t)(cc >> 3) * PANEL + (uint32_t)r * 128u + (uint32_t)(((cc & 7) ^ (r & 7)) << 4);
  };
#pragma unroll
  for (int i = 0; i < FP_STAGES - 1; ++i) issue(i);

  float acc_o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_o[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  uint32_t qf[KT][4];
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
  const int lo_lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  const int lo_hi = window > 0 ? max(0, p_hi - window + 1) : 0;
  const int warp_first_pos = pos0 + warp * 16, warp_last_pos = min(warp_first_pos + 15, last_pos);
  const int warp_lo = window > 0 ? max(0, warp_first_pos - window + 1) : 0;          // lower bound of the warp's first row
  const int warp_lo_last = window > 0 ? max(0, warp_last_pos - window + 1) : 0;      // and of its last row
  fa_wait<0>();
  __syncthreads();                                        // Q is in shared memory
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * k + (lane >> 4);
    ldmatrix_x4(sm_q + swz<CH>(r, c), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
  }

  for (int kt = 0; kt < n_kt; ++kt) {
    issue(kt + FP_STAGES - 1);                            // into the stage that tile kt - 1 left
    const int st = kt % FP_STAGES;
    const uint32_t parity = (uint32_t)(kt / FP_STAGES) & 1u;
    if (!*const_cast<volatile int*>(&gave_up) && !mbar_try_wait(&full[st], parity)) {
      const uint64_t start = global_ns();
      while (!mbar_try_wait(&full[st], parity)) {
        if (*const_cast<volatile int*>(&gave_up)) break;
        if (global_ns() - start > FP_WAIT_NS) {
          gave_up = 1;                                    // the tiles that follow are not waited for (the output is void)
          atomicCAS(&g_fa_status, 0, 1);
          break;
        }
      }
    }
    const int k0 = k_first + kt * FA_BK;
    const uint32_t ks = sm_kv + (uint32_t)st * STAGE, vs = ks + PANELS * PANEL;
    if (k0 < key_lo || k0 + FA_BK - 1 > last_pos) {       // an edge tile: value rows outside the keys anyone sees
      if (threadIdx.x < FA_BK) {
        const int kp = k0 + (int)threadIdx.x;
        if (kp < key_lo || kp > last_pos) {
#pragma unroll
          for (int p = 0; p < PANELS; ++p) {
            uint4* row = reinterpret_cast<uint4*>(fp_smem + (size_t)st * STAGE + (PANELS + p) * PANEL + threadIdx.x * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) row[i] = make_uint4(0, 0, 0, 0);
          }
        }
      }
      __syncthreads();
    }
    const bool active = warp * 16 < rows && k0 <= warp_last_pos && k0 + FA_BK > warp_lo;
    if (active) {
      float s[FA_BK / 8][4];
#pragma unroll
      for (int i = 0; i < FA_BK / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
#pragma unroll
        for (int n = 0; n < FA_BK / 16; ++n) {
          uint32_t b0, b1, b2, b3;
          const int r = n * 16 + (lane & 7) + 8 * (lane >> 4), c = 2 * k + ((lane >> 3) & 1);
          ldmatrix_x4(ks + tile_off(r, c), b0, b1, b2, b3);
          fa_mma(s[2 * n], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
          fa_mma(s[2 * n + 1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
        }
      }
      float mx[2] = {row_max[0], row_max[1]};
      // every row of the warp sees every key of the tile: no masks
      const bool all_visible = k0 + FA_BK - 1 <= warp_first_pos && k0 >= warp_lo_last;
      if (all_visible) {
#pragma unroll
        for (int i = 0; i < FA_BK / 8; ++i) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s[i][j] *= scale_log2;
            mx[j >> 1] = fmaxf(mx[j >> 1], s[i][j]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < FA_BK / 8; ++i) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int kp = k0 + 8 * i + 2 * t + (j & 1);
            const bool hi = j >= 2;
            const bool ok = hi ? (kp <= p_hi && kp >= lo_hi) : (kp <= p_lo && kp >= lo_lo);
            s[i][j] = ok ? s[i][j] * scale_log2 : -INFINITY;
            mx[hi] = fmaxf(mx[hi], s[i][j]);
          }
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        mx[h] = ceilf(mx[h]);                              // a whole power of two as the reference (see the file's head)
      }
      float alpha[2], base[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        base[h] = mx[h] == -INFINITY ? 0.f : mx[h];
        alpha[h] = exp2f(row_max[h] - base[h]);
        row_max[h] = mx[h];
        row_sum[h] *= alpha[h];
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc_o[i][0] *= alpha[0]; acc_o[i][1] *= alpha[0];
        acc_o[i][2] *= alpha[1]; acc_o[i][3] *= alpha[1];
      }
      uint32_t pf[FA_BK / 16][4];
#pragma unroll
      for (int i = 0; i < FA_BK / 8; ++i) {
        const float p0 = exp2f(s[i][0] - base[0]), p1 = exp2f(s[i][1] - base[0]);
        const float p2 = exp2f(s[i][2] - base[1]), p3 = exp2f(s[i][3] - base[1]);
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int kk = 0; kk < FA_BK / 16; ++kk) {
#pragma unroll
        for (int n = 0; n < NT / 2; ++n) {
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * n + (lane >> 4);
          ldmatrix_x4_trans(vs + tile_off(r, c), b0, b1, b2, b3);
          fa_mma(acc_o[2 * n], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
          fa_mma(acc_o[2 * n + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
        }
      }
    }
    __syncthreads();                                      // the stage is free for tile kt + FP_STAGES
  }
  if (*const_cast<volatile int*>(&gave_up)) drain_after_abort();            // copies in flight land before the block returns
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }
  const float inv_lo = 1.f / row_sum[0], inv_hi = 1.f / row_sum[1];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int d = 8 * i + 2 * t;
    if (r_lo < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_lo) * nh + head) * HD + d) =
          pack_bf16(acc_o[i][0] * inv_lo, acc_o[i][1] * inv_lo);
    if (r_hi < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_hi) * nh + head) * HD + d) =
          pack_bf16(acc_o[i][2] * inv_hi, acc_o[i][3] * inv_hi);
  }
}

static bool prefill_tma_page_ok(int page_size) {
  return page_size >= 8 && page_size <= FA_BK && page_size % 8 == 0 && FA_BK % page_size == 0;
}

// num_pages: pages in the pool.  Page sizes the TMA kernel does not take give SNK_ERR_SIZE (the caller
// then uses snk_attention_prefill).
SNK_API int snk_attention_prefill_tma(const void* q, const void* pool, long long num_pages, const int* block_table,
                                      int max_pages, int page_size, const int* tiles, int n_tiles, void* out, int nh,
                                      int nkv, int hd, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh > 65535) return SNK_ERR_SIZE;
  if ((hd != 64 && hd != 128) || !prefill_tma_page_ok(page_size) || num_pages <= 0) return SNK_ERR_SIZE;
  if (num_pages * 2 * nkv * page_size >= (1ll << 31)) return SNK_ERR_SIZE;
  if (((uintptr_t)q % 16) || ((uintptr_t)pool % 16) || ((uintptr_t)out % 4)) return SNK_ERR_ALIGN;
  CUtensorMap map;
  const int rc = tensor_map(pool, num_pages * 2 * nkv * page_size, hd, page_size, 64, &map);
  if (rc) return rc;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tiles, nh);
  const size_t smem = 1024 + (size_t)FP_STAGES * 2 * (hd / 64) * FA_BK * 128 + (size_t)FA_BQ * hd * 2;
  const bf16* qp = static_cast<const bf16*>(q);
  bf16* op = static_cast<bf16*>(out);
  if (hd == 64) {
    cudaFuncSetAttribute(attention_prefill_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_prefill_tma_kernel<64>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, map, qp, block_table,
               max_pages, page_size, tiles, n_tiles, op, nh, nkv, window, scale_log2);
  } else {
    cudaFuncSetAttribute(attention_prefill_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_prefill_tma_kernel<128>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, map, qp, block_table,
               max_pages, page_size, tiles, n_tiles, op, nh, nkv, window, scale_log2);
  }
  SNK_LAUNCH_CHECK();
  return 0;
}


// ---------------------------------------------------------------------------------------------
// Rows of decoded tokens (one row per request, a long run of keys each).  One block takes one row, one
// kv head and one chunk of 256 keys.  The q heads that share the kv head are the rows of the MMA (up to
// 16), so the chunk's keys and values are read once for all of them.  Each of the 4 warps multiplies
// the heads with its own 64 keys; the 4 partial (max, sum, output) meet in shared memory in warp
// order, and the chunk's partial goes to scratch in the format of csrc/attention.cu, whose merge
// kernel adds the chunks in order (num_chunks == 1: the block writes the output itself).
#define FD_CHUNK 256

template <int HD>
__global__ void __launch_bounds__(FA_WARPS * 32)
attention_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool,
                            const int* __restrict__ block_table, int max_pages, int page_size,
                            const int* __restrict__ positions, const int* __restrict__ row_seg,
                            const int* __restrict__ row_list, bf16* __restrict__ out,
                            float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                            int window, int num_chunks, float scale_log2) {
  pdl_begin();
  constexpr int CH = HD / 8, KT = HD / 16, NT = HD / 8;
  extern __shared__ __align__(16) unsigned char fd_smem[];
  const uint32_t sm_q = (uint32_t)__cvta_generic_to_shared(fd_smem);        // [16][HD]
  const uint32_t sm_k = sm_q + 16 * HD * 2;                                 // [256][HD]
  const uint32_t sm_v = sm_k + FD_CHUNK * HD * 2;                           // [256][HD]
  float* merge = reinterpret_cast<float*>(fd_smem + 16 * HD * 2);           // reuses the key tile afterwards

  const int m = row_list ? row_list[blockIdx.x] : blockIdx.x;
  const int kvh = blockIdx.y;
  const int group = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int pos = positions[m];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int c = lo / FD_CHUNK + blockIdx.z;
  if ((long long)c * FD_CHUNK > pos) return;
  const int k0 = c * FD_CHUNK;
  const int k_begin = max(lo, k0), k_end = min(pos + 1, k0 + FD_CHUNK);
  const int* bt = block_table + (size_t)row_seg[m] * max_pages;
  const size_t page_stride = (size_t)2 * nkv * page_size * HD;
  const size_t v_off = (size_t)nkv * page_size * HD;

  for (int v = threadIdx.x; v < 16 * CH; v += FA_WARPS * 32) {
    const int r = v / CH, cc = v % CH;
    fa_cp_async16(sm_q + swz<CH>(r, cc), q + ((size_t)m * nh + kvh * group + min(r, group - 1)) * HD + cc * 8,
                  r < group);
  }
  // the chunk's pages once per block (not once per copy): first page k0 / page_size
  __shared__ int chunk_pages[FD_CHUNK + 1];
  const int first_page = k0 / page_size;
  const int n_pages = (k_end - 1) / page_size - first_page + 1;
  for (int i = threadIdx.x; i < n_pages; i += FA_WARPS * 32) chunk_pages[i] = bt[first_page + i];
  __syncthreads();
  const bool pow2 = (page_size & (page_size - 1)) == 0;
  const int shift = 31 - __clz(page_size);
  for (int v = threadIdx.x; v < FD_CHUNK * CH; v += FA_WARPS * 32) {
    const int r = v / CH, cc = v % CH;
    const int kp = k0 + r;
    const bool valid = kp >= k_begin && kp < k_end;
    const bf16* src = pool;
    if (valid) {
      const int pi = pow2 ? (kp >> shift) : kp / page_size;
      const int in_page = pow2 ? (kp & (page_size - 1)) : kp - pi * page_size;
      src = pool + (size_t)chunk_pages[pi - first_page] * page_stride + ((size_t)kvh * page_size + in_page) * HD +
            cc * 8;
    }
    fa_cp_async16(sm_k + swz<CH>(r, cc), src, valid);
    fa_cp_async16(sm_v + swz<CH>(r, cc), valid ? src + v_off : src, valid);
  }
  fa_commit();
  fa_wait<0>();
  __syncthreads();

  float acc_o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_o[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  const int w0 = k0 + warp * FA_BK;                       // first key of this warp's 64
  if (w0 < k_end && w0 + FA_BK > k_begin) {
    uint32_t qf[KT][4];
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      const int r = (lane & 7) + 8 * ((lane >> 3) & 1), cc = 2 * k + (lane >> 4);
      ldmatrix_x4(sm_q + swz<CH>(r, cc), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
    }
    float s[FA_BK / 8][4];
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int k = 0; k < KT; ++k) {
#pragma unroll
      for (int n = 0; n < FA_BK / 16; ++n) {
        uint32_t b0, b1, b2, b3;
        const int r = warp * FA_BK + n * 16 + (lane & 7) + 8 * (lane >> 4), cc = 2 * k + ((lane >> 3) & 1);
        ldmatrix_x4(sm_k + swz<CH>(r, cc), b0, b1, b2, b3);
        fa_mma(s[2 * n], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
        fa_mma(s[2 * n + 1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
      }
    }
    // s[i] = {(head g, key 8i+2t), (g, 8i+2t+1), (g+8, ...), (g+8, ...)}: every head sees the same keys
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kp = w0 + 8 * i + 2 * t + (j & 1);
        s[i][j] = (kp >= k_begin && kp < k_end) ? s[i][j] * scale_log2 : -INFINITY;
        mx[j >> 1] = fmaxf(mx[j >> 1], s[i][j]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      mx[h] = ceilf(mx[h]);                               // a whole power of two as the reference (see the file's head)
      row_max[h] = mx[h];                                 // finite: the warp has a valid key
    }
    uint32_t pf[FA_BK / 16][4];
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i) {
      const float p0 = exp2f(s[i][0] - mx[0]), p1 = exp2f(s[i][1] - mx[0]);
      const float p2 = exp2f(s[i][2] - mx[1]), p3 = exp2f(s[i][3] - mx[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int kk = 0; kk < FA_BK / 16; ++kk) {
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) {
        uint32_t b0, b1, b2, b3;
        const int r = warp * FA_BK + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = 2 * n + (lane >> 4);
        ldmatrix_x4_trans(sm_v + swz<CH>(r, cc), b0, b1, b2, b3);
        fa_mma(acc_o[2 * n], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
        fa_mma(acc_o[2 * n + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
    }
  }
  __syncthreads();                                        // all warps are done with the key tile: reuse it
  // merge area: ml [4 warps][16 heads][2], then o [4 warps][16 heads][HD]
  float* ml = merge;
  float* mo = merge + FA_WARPS * 16 * 2;
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = row_max[0];
    ml[(warp * 16 + g) * 2 + 1] = row_sum[0];
    ml[(warp * 16 + g + 8) * 2] = row_max[1];
    ml[(warp * 16 + g + 8) * 2 + 1] = row_sum[1];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int d = 8 * i + 2 * t;
    mo[(warp * 16 + g) * HD + d] = acc_o[i][0];
    mo[(warp * 16 + g) * HD + d + 1] = acc_o[i][1];
    mo[(warp * 16 + g + 8) * HD + d] = acc_o[i][2];
    mo[(warp * 16 + g + 8) * HD + d + 1] = acc_o[i][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * HD; idx += FA_WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float mxl = -INFINITY;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) mxl = fmaxf(mxl, ml[(w * 16 + r) * 2]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) {                  // warps in key order
      const float f = exp2f(ml[(w * 16 + r) * 2] - mxl);  // a warp without keys: exp2(-inf) = 0
      l += ml[(w * 16 + r) * 2 + 1] * f;
      o = fmaf(mo[(w * 16 + r) * HD + d], f, o);
    }
    const int head = kvh * group + r;
    if (num_chunks == 1) {
      out[((size_t)m * nh + head) * HD + d] = __float2bfloat16_rn(o / l);
    } else {
      const size_t slot = ((size_t)blockIdx.x * nh + head) * num_chunks + blockIdx.z;
      part_o[slot * HD + d] = o;
      if (d == 0) {
        part_ml[slot * 2] = mxl * 0.6931471805599453f;   // the merge kernel works with natural exponents
        part_ml[slot * 2 + 1] = l;
      }
    }
  }
}

// rows: M rows to serve (row_list, or rows 0..M-1); keys in chunks of 256; scratch as in
// snk_paged_attention_scratch_bytes when num_chunks > 1 (the caller then runs snk_attention_merge).
SNK_API int snk_attention_decode_mma(const void* q, const void* pool, const int* block_table, int max_pages,
                                     int page_size, const int* positions, const int* row_seg,
                                     const int* row_list, void* out, void* scratch, int M, int nh, int nkv,
                                     int hd, int window, int num_chunks, float scale, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || nkv > 65535 || num_chunks < 1 || num_chunks > 65535)
    return SNK_ERR_SIZE;
  if (hd != 64 && hd != 128) return SNK_ERR_SIZE;
  if (num_chunks > 1 && scratch == nullptr) return SNK_ERR_SIZE;
  if (((uintptr_t)q % 16) || ((uintptr_t)pool % 16)) return SNK_ERR_ALIGN;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(M, nkv, num_chunks);
  const size_t smem = (size_t)(16 + 2 * FD_CHUNK) * hd * 2;
  float* part_o = static_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (size_t)M * nh * num_chunks * hd : nullptr;
  const bf16 *qp = static_cast<const bf16*>(q), *pp = static_cast<const bf16*>(pool);
  bf16* op = static_cast<bf16*>(out);
  if (hd == 64) {
    cudaFuncSetAttribute(attention_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_decode_mma_kernel<64>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, 
        qp, pp, block_table, max_pages, page_size, positions, row_seg, row_list, op, part_o, part_ml, nh, nkv,
        window, num_chunks, scale_log2);
  } else {
    cudaFuncSetAttribute(attention_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_decode_mma_kernel<128>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, 
        qp, pp, block_table, max_pages, page_size, positions, row_seg, row_list, op, part_o, part_ml, nh, nkv,
        window, num_chunks, scale_log2);
  }
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The same kernel with the chunk's keys and values brought in by TMA: the cache pool is one 2-D tensor
// [pages * 2 * kv heads * page_size rows, head_dim] whose map has a box of page_size rows x 64 elements
// and the 128-byte swizzle, so one instruction of one lane lands a page's keys (or values) of this kv
// head in shared memory in the layout ldmatrix wants (a head of 128 elements is two such panels side by
// side).  The 128 threads no longer compute addresses and issue 16-byte copies; they wait on one
// mbarrier.  Pages are loaded whole: rows outside the chunk's valid keys hold whatever the page (or
// the shared memory before) held, so their scores are replaced, never computed with, and their value
// rows are zeroed before use.  For page sizes that divide 256 and are multiples of 8.
// The wait is bounded by wall time; when it runs out the block records it (snk_attention_decode_status)
// and goes on without the data.
#define FD_WAIT_NS 1000000000ull
__device__ int g_fd_status;

template <int HD>
__global__ void __launch_bounds__(FA_WARPS * 32)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q,
                            const int* __restrict__ block_table, int max_pages, int page_size,
                            const int* __restrict__ positions, const int* __restrict__ row_seg,
                            const int* __restrict__ row_list, bf16* __restrict__ out,
                            float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                            int window, int num_chunks, float scale_log2) {
  // the map is a kernel parameter: fetching it does not have to wait for the kernel in front
  if (threadIdx.x == 0)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
  pdl_begin();
  constexpr int CH = HD / 8, KT = HD / 16, NT = HD / 8, PANELS = HD / 64;
  constexpr uint32_t PANEL = FD_CHUNK * 128;              // bytes of one 64-element panel of the chunk's rows
  extern __shared__ unsigned char fd_raw[];
  unsigned char* fd_smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fd_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sm_k = (uint32_t)__cvta_generic_to_shared(fd_smem);        // [PANELS][256][64]
  const uint32_t sm_v = sm_k + PANELS * PANEL;
  const uint32_t sm_q = sm_v + PANELS * PANEL;                              // [16][HD], swz<CH>
  float* merge = reinterpret_cast<float*>(fd_smem);                         // reuses the key tile afterwards
  __shared__ uint64_t bar;

  const int m = row_list ? row_list[blockIdx.x] : blockIdx.x;
  const int kvh = blockIdx.y;
  const int group = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int pos = positions[m];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int c = lo / FD_CHUNK + blockIdx.z;
  if ((long long)c * FD_CHUNK > pos) return;
  const int k0 = c * FD_CHUNK;
  const int k_begin = max(lo, k0), k_end = min(pos + 1, k0 + FD_CHUNK);
  const int* bt = block_table + (size_t)row_seg[m] * max_pages;

  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int v = threadIdx.x; v < 16 * CH; v += FA_WARPS * 32) {
    const int r = v / CH, cc = v % CH;
    fa_cp_async16(sm_q + swz<CH>(r, cc), q + ((size_t)m * nh + kvh * group + min(r, group - 1)) * HD + cc * 8,
                  r < group);
  }
  fa_commit();
  __syncthreads();                                        // the barrier is initialised
  const int first_page = k_begin / page_size;
  const int n_pages = (k_end - 1) / page_size - first_page + 1;
  if (warp == 0) {
    if (lane == 0) mbar_expect_tx(&bar, (uint32_t)n_pages * page_size * 128u * 2u * PANELS);
    __syncwarp();
    for (int i = lane; i < n_pages; i += 32) {
      const int page = bt[first_page + i];
      const int row = (first_page + i) * page_size - k0;                    // the page's first row in the chunk
      const int y_k = ((page * 2) * nkv + kvh) * page_size, y_v = ((page * 2 + 1) * nkv + kvh) * page_size;
#pragma unroll
      for (int p = 0; p < PANELS; ++p) {
        tma_load_2d(fd_smem + p * PANEL + row * 128, &map_kv, &bar, p * 64, y_k);
        tma_load_2d(fd_smem + (PANELS + p) * PANEL + row * 128, &map_kv, &bar, p * 64, y_v);
      }
    }
  }
  fa_wait<0>();
  if (!mbar_try_wait(&bar, 0)) {
    const uint64_t start = global_ns();
    while (!mbar_try_wait(&bar, 0)) {
      if (global_ns() - start > FD_WAIT_NS) {
        atomicCAS(&g_fd_status, 0, 1);
        drain_after_abort();                              // the copies in flight land before the block goes on and returns
        break;
      }
    }
  }
  if (k_begin > k0 || k_end < k0 + FD_CHUNK) {            // value rows outside the valid keys: zero, whatever they held
    for (int r = threadIdx.x; r < FD_CHUNK; r += FA_WARPS * 32) {
      const int kp = k0 + r;
      if (kp < k_begin || kp >= k_end) {
#pragma unroll
        for (int p = 0; p < PANELS; ++p) {
          uint4* row = reinterpret_cast<uint4*>(fd_smem + (PANELS + p) * PANEL + r * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) row[i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }
  __syncthreads();
  // byte offset of 16-byte chunk cc of row r in a [PANELS][256][64] tile written by TMA
  auto tile_off = [](int r, int cc) -> uint32_t {
    return (uint32_t)(cc >> 3) * PANEL + (uint32_t)r * 128u + (uint32_t)(((cc & 7) ^ (r & 7)) << 4);
  };

  float acc_o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_o[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  const int w0 = k0 + warp * FA_BK;                       // first key of this warp's 64
  if (w0 < k_end && w0 + FA_BK > k_begin) {
    uint32_t qf[KT][4];
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      const int r = (lane & 7) + 8 * ((lane >> 3) & 1), cc = 2 * k + (lane >> 4);
      ldmatrix_x4(sm_q + swz<CH>(r, cc), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
    }
    float s[FA_BK / 8][4];
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int k = 0; k < KT; ++k) {
#pragma unroll
      for (int n = 0; n < FA_BK / 16; ++n) {
        uint32_t b0, b1, b2, b3;
        const int r = warp * FA_BK + n * 16 + (lane & 7) + 8 * (lane >> 4), cc = 2 * k + ((lane >> 3) & 1);
        ldmatrix_x4(sm_k + tile_off(r, cc), b0, b1, b2, b3);
        fa_mma(s[2 * n], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
        fa_mma(s[2 * n + 1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kp = w0 + 8 * i + 2 * t + (j & 1);
        s[i][j] = (kp >= k_begin && kp < k_end) ? s[i][j] * scale_log2 : -INFINITY;
        mx[j >> 1] = fmaxf(mx[j >> 1], s[i][j]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      mx[h] = ceilf(mx[h]);                               // a whole power of two as the reference (see the file's head)
      row_max[h] = mx[h];
    }
    uint32_t pf[FA_BK / 16][4];
#pragma unroll
    for (int i = 0; i < FA_BK / 8; ++i) {
      const float p0 = exp2f(s[i][0] - mx[0]), p1 = exp2f(s[i][1] - mx[0]);
      const float p2 = exp2f(s[i][2] - mx[1]), p3 = exp2f(s[i][3] - mx[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int kk = 0; kk < FA_BK / 16; ++kk) {
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) {
        uint32_t b0, b1, b2, b3;
        const int r = warp * FA_BK + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = 2 * n + (lane >> 4);
        ldmatrix_x4_trans(sm_v + tile_off(r, cc), b0, b1, b2, b3);
        fa_mma(acc_o[2 * n], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
        fa_mma(acc_o[2 * n + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
    }
  }
  __syncthreads();                                        // all warps are done with the key tile: reuse it
  float* ml = merge;
  float* mo = merge + FA_WARPS * 16 * 2;
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = row_max[0];
    ml[(warp * 16 + g) * 2 + 1] = row_sum[0];
    ml[(warp * 16 + g + 8) * 2] = row_max[1];
    ml[(warp * 16 + g + 8) * 2 + 1] = row_sum[1];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int d = 8 * i + 2 * t;
    mo[(warp * 16 + g) * HD + d] = acc_o[i][0];
    mo[(warp * 16 + g) * HD + d + 1] = acc_o[i][1];
    mo[(warp * 16 + g + 8) * HD + d] = acc_o[i][2];
    mo[(warp * 16 + g + 8) * HD + d + 1] = acc_o[i][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * HD; idx += FA_WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float mxl = -INFINITY;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) mxl = fmaxf(mxl, ml[(w * 16 + r) * 2]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) {                  // warps in key order
      const float f = exp2f(ml[(w * 16 + r) * 2] - mxl);  // a warp without keys: exp2(-inf) = 0
      l += ml[(w * 16 + r) * 2 + 1] * f;
      o = fmaf(mo[(w * 16 + r) * HD + d], f, o);
    }
    const int head = kvh * group + r;
    if (num_chunks == 1) {
      out[((size_t)m * nh + head) * HD + d] = __float2bfloat16_rn(o / l);
    } else {
      const size_t slot = ((size_t)blockIdx.x * nh + head) * num_chunks + blockIdx.z;
      part_o[slot * HD + d] = o;
      if (d == 0) {
        part_ml[slot * 2] = mxl * 0.6931471805599453f;
        part_ml[slot * 2 + 1] = l;
      }
    }
  }
}

// Whether the TMA kernel takes this page size.
static bool decode_tma_page_ok(int page_size) {
  return page_size >= 8 && page_size <= FD_CHUNK && page_size % 8 == 0 && FD_CHUNK % page_size == 0;
}

// num_pages: pages in the pool (it is [num_pages, 2, nkv, page_size, hd]).  Page sizes the TMA kernel does
// not take give SNK_ERR_SIZE (the caller then uses snk_attention_decode_mma).
SNK_API int snk_attention_decode_tma(const void* q, const void* pool, long long num_pages, const int* block_table,
                                     int max_pages, int page_size, const int* positions, const int* row_seg,
                                     const int* row_list, void* out, void* scratch, int M, int nh, int nkv,
                                     int hd, int window, int num_chunks, float scale, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || nkv > 65535 || num_chunks < 1 || num_chunks > 65535)
    return SNK_ERR_SIZE;
  if ((hd != 64 && hd != 128) || !decode_tma_page_ok(page_size) || num_pages <= 0) return SNK_ERR_SIZE;
  if (num_pages * 2 * nkv * page_size >= (1ll << 31)) return SNK_ERR_SIZE;       // row coordinates are 32-bit
  if (num_chunks > 1 && scratch == nullptr) return SNK_ERR_SIZE;
  if (((uintptr_t)q % 16) || ((uintptr_t)pool % 16)) return SNK_ERR_ALIGN;
  CUtensorMap map;
  const int rc = tensor_map(pool, num_pages * 2 * nkv * page_size, hd, page_size, 64, &map);
  if (rc) return rc;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(M, nkv, num_chunks);
  const size_t smem = 1024 + (size_t)2 * (hd / 64) * FD_CHUNK * 128 + (size_t)16 * hd * 2;
  float* part_o = static_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (size_t)M * nh * num_chunks * hd : nullptr;
  const bf16* qp = static_cast<const bf16*>(q);
  bf16* op = static_cast<bf16*>(out);
  if (hd == 64) {
    cudaFuncSetAttribute(attention_decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_decode_tma_kernel<64>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, map, qp, block_table,
               max_pages, page_size, positions, row_seg, row_list, op, part_o, part_ml, nh, nkv, window, num_chunks,
               scale_log2);
  } else {
    cudaFuncSetAttribute(attention_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(attention_decode_tma_kernel<128>, dim3(grid), dim3(FA_WARPS * 32), smem, stream, map, qp, block_table,
               max_pages, page_size, positions, row_seg, row_list, op, part_o, part_ml, nh, nkv, window, num_chunks,
               scale_log2);
  }
  SNK_LAUNCH_CHECK();
  return 0;
}

// Queue copies of the two status words (decode, prompt) into ``host`` (pinned host memory, two ints) on
// ``stream`` without waiting for them and without clearing them.  Not for use inside a stream capture.
SNK_API int snk_attention_decode_status_peek(int* host, void* stream) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(host, g_fd_status, sizeof(int), 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyFromSymbolAsync(host + 1, g_fa_status, sizeof(int), 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

// 0, or bit 0 / bit 1 when a block of an earlier decode / prompt launch gave up waiting for its keys;
// reading clears it.  Synchronises the device.
SNK_API int snk_attention_decode_status() {
  int v = 0, w = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fd_status, sizeof(int)) != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&w, g_fa_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_fd_status, &zero, sizeof(int));
  if (w) cudaMemcpyToSymbol(g_fa_status, &zero, sizeof(int));
  return v | (w << 1);
}
