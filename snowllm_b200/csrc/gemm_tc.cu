// C[M,N] = A[M,K] . W[N,K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05), for many rows
// (prefill).  Blocks are persistent: as many as the GPU holds, each walking tiles of 128 x BN of C
// (BN 256 where there are enough tiles to fill the GPU, else 128), in bands of 8 n-tiles (n-tile fastest
// inside a band, see tc_tile), so that blocks running side by side share operand tiles:
//
//   warp 0, one lane   TMA producer: 128x64 tiles of A and BNx64 tiles of W into a ring of shared-memory
//                      stages (cp.async.bulk.tensor, 128-byte swizzle, completion counted on an mbarrier)
//   warp 1, one lane   MMA issuer: per stage four tcgen05.mma (M 128, N BN, K 16) straight from shared
//                      memory into a float accumulator in tensor memory; tcgen05.commit hands the stage
//                      back to the producer and, after the last k-block, the accumulator to the epilogue
//   warps 2..5         epilogue: tcgen05.ld of the accumulator (each warp its 32 lanes = 32 rows of C),
//                      conversion, guarded stores
//
// There are two accumulators in tensor memory (2 x BN columns): the epilogue of one tile runs while
// the next tile's products are issued.
//
// Both operands are K-major, which is how activations and checkpoint weights already lie in memory,
// so nothing is re-tiled at load.  Rows past M (or past a group's end) and k past K are zero-filled
// by TMA and masked at the store.
//
// Grouped form (routed experts): rows of A are already sorted by group and contiguous; group e owns
// rows [offsets[e], offsets[e+1]) and multiplies them with W[e].  Row tiles are counted per group, so
// a tile never mixes groups in its stored rows.
//
// Every wait on an mbarrier is bounded by wall time: when it runs out the block records an error
// code (see snk_gemm_tc_status), issues no more loads and products, gives the copies in flight a moment
// to land, frees its tensor memory and returns.  snk_gemm_tc_test_lose_loads makes that happen for a test:
// the producers then issue no loads, so the waits for operands run out.
// (the role of snowllm/ops/gemm.py:33-41 and the expert products of snowllm/ops/inference.py:60-76
// at prefill shapes)
#include "tma.cuh"
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_SMEM_TILES (192 * 1024)    // bytes of shared memory given to the operand stages
#ifndef TC_BAND
#define TC_BAND 8                     // n-tiles in a band of the tile order (8, 16 and 28 measured; 8 is best or equal everywhere)
#endif
#define TC_WAIT_NS 1500000000ull      // 1.5 s per wait before giving up

enum { TC_ERR_WAIT_FULL = 1, TC_ERR_WAIT_EMPTY = 2, TC_ERR_WAIT_ACC = 3, TC_ERR_WAIT_ACC_FREE = 4 };

__device__ int g_tc_status;            // 0, or the first error code a block recorded
__device__ int g_tc_lose_loads;        // test hook: producers issue no loads (the operands then never arrive)

// Wait for a phase, for TC_WAIT_NS at most.  `aborted` (shared) short-cuts every later wait of the block.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* aborted, int code) {
  if (*aborted) return;
  if (mbar_try_wait(bar, parity)) return;
  const uint64_t start = global_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (*aborted) return;
    if (global_ns() - start > TC_WAIT_NS) {
      *aborted = 1;
      atomicCAS(&g_tc_status, 0, code);
      return;
    }
  }
}

#define TC_MAX_STAGES 6

struct __align__(16) TcShared {
  uint64_t full[TC_MAX_STAGES];
  uint64_t empty[TC_MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int aborted;
  __align__(16) float stage_out[4][TC_STAGE_FLOATS];    // one staging tile per epilogue warp (tc_store_piece)
};

// Rows of C and rows of W that tile `tile` covers.  Plain: tiles = row_tiles * n_tiles, row tile fastest.
// Grouped: row tiles are counted group by group (a tile never spans two groups).
struct TcTile {
  int row0, row_end, w_row0, n0;
  bool valid;
};

__device__ __forceinline__ TcTile tc_tile(int tile, int row_tiles, int M, int N, int BN, const int* offsets,
                                          int groups) {
  TcTile t;
  // Tiles are numbered in bands of up to TC_BAND n-tiles: inside a band the n-tile runs fastest, then the row
  // tile; then the next band.  Blocks that run side by side so share a row tile of A and read neighbouring
  // tiles of W (measured against row tiles fastest: +6 % on 2048 x 6144 x 2048, +6 to +8 % on the experts'
  // products; one band over all of a wide N lost 8 % on 2048 x 14336 x 2048).
  const int n_tiles = (N + BN - 1) / BN;
  const int bands = (n_tiles + TC_BAND - 1) / TC_BAND;
  const int band_w = (n_tiles + bands - 1) / bands;
  const int per_band = row_tiles * band_w;
  const int band = tile / per_band, in_band = tile % per_band;
  const int w_here = min(band_w, n_tiles - band * band_w);   // the last band may be narrower
  const int rt = in_band / w_here, nt = band * band_w + in_band % w_here;
  t.n0 = nt * BN;
  t.valid = t.n0 < N;
  if (!offsets) {
    t.row0 = rt * TC_BM;
    t.row_end = M;
    t.w_row0 = 0;
    return t;
  }
  int left = rt;
  t.valid = false;
  t.row0 = t.row_end = t.w_row0 = 0;
  if (nt * BN >= N) return t;
  for (int e = 0; e < groups; ++e) {
    const int begin = offsets[e], cnt = offsets[e + 1] - begin;
    const int tiles_e = (cnt + TC_BM - 1) / TC_BM;
    if (left < tiles_e) {
      t.row0 = begin + left * TC_BM;
      t.row_end = begin + cnt;
      t.w_row0 = e * N;
      t.valid = true;
      return t;
    }
    left -= tiles_e;
  }
  return t;
}

// SWIGLU: W holds gate and up rows interleaved in blocks of 8 (rows 16j..16j+7: gate of features
// 8j..8j+7, rows 16j+8..16j+15: their up rows); the store is silu(gate) * up into C[M, N/2].
template <int BN, typename OutT, bool SWIGLU>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               OutT* __restrict__ C, int M, int N, int K, const int* __restrict__ offsets, int groups,
               int row_tiles_bound, int splits) {
  constexpr int STAGE_BYTES = (TC_BM + BN) * TC_BK * 2;
  constexpr int STAGES = TC_SMEM_TILES / STAGE_BYTES < TC_MAX_STAGES ? TC_SMEM_TILES / STAGE_BYTES : TC_MAX_STAGES;
  extern __shared__ unsigned char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  TcShared* sh = reinterpret_cast<TcShared*>(tiles + (size_t)STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;

  // Barriers and tensor memory are set up before the wait for the kernel in front: none of it touches
  // global memory, and it then overlaps with that kernel's tail.
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 4);                   // one arrival per epilogue warp
    }
    sh->aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {                                       // one warp allocates both accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh->tmem_base)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = sh->tmem_base;
  volatile int* aborted = &sh->aborted;
  pdl_begin();
  // number of row tiles: known for the plain product, counted from the offsets for the grouped one
  int row_tiles = row_tiles_bound;
  if (offsets) {
    row_tiles = 0;
    for (int e = 0; e < groups; ++e) row_tiles += (offsets[e + 1] - offsets[e] + TC_BM - 1) / TC_BM;
  }
  const int n_tiles = (N + BN - 1) / BN;
  const int total = row_tiles * n_tiles;
  // splits > 1 (plain products with few tiles): work item w is tile w % total over the k-blocks of part
  // w / total, and the partial product goes to plane w / total of C, which then is float [splits, M, N]
  const int items = total * splits;
  const int k_per = (k_tiles + splits - 1) / splits;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                        // k-blocks issued so far, over all tiles
      const bool lose_loads = *const_cast<volatile int*>(&g_tc_lose_loads) != 0;
      for (int item = blockIdx.x; item < items && !*aborted; item += gridDim.x) {
        const TcTile t = tc_tile(item % total, row_tiles, M, N, BN, offsets, groups);
        if (!t.valid) continue;
        const int kt_begin = (item / total) * k_per, kt_end = min(k_tiles, kt_begin + k_per);
        for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
          const int s = it % STAGES;
          mbar_wait(&sh->empty[s], ((it / STAGES) & 1) ^ 1, aborted, TC_ERR_WAIT_EMPTY);
          if (*aborted) break;                             // a wait ran out: nothing more is issued
          if (lose_loads) continue;
          mbar_expect_tx(&sh->full[s], STAGE_BYTES);
          unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
          tma_load_2d(stage, &map_a, &sh->full[s], kt * TC_BK, t.row0);
          tma_load_2d(stage + TC_BM * TC_BK * 2, &map_w, &sh->full[s], kt * TC_BK, t.w_row0 + t.n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(TC_BM, BN);
      int it = 0, local = 0;
      for (int item = blockIdx.x; item < items && !*aborted; item += gridDim.x) {
        const TcTile t = tc_tile(item % total, row_tiles, M, N, BN, offsets, groups);
        if (!t.valid) continue;
        const int kt_begin = (item / total) * k_per, kt_end = min(k_tiles, kt_begin + k_per);
        const int buf = local & 1;
        mbar_wait(&sh->acc_empty[buf], ((local >> 1) & 1) ^ 1, aborted, TC_ERR_WAIT_ACC_FREE);
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + (uint32_t)(buf * BN);
        for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
          const int s = it % STAGES;
          mbar_wait(&sh->full[s], (it / STAGES) & 1, aborted, TC_ERR_WAIT_FULL);
          if (*aborted) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t w_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // 16 k-values = 32 bytes further along the swizzled 128-byte rows
            umma_bf16(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(w_addr + k * 32), idesc,
                      (kt > kt_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[s]);                    // the stage is free once these MMAs have read it
        }
        if (*aborted) break;
        umma_commit(&sh->acc_full[buf]);
        ++local;
      }
    }
  } else {
    const int lane_group = warp & 3;                     // a warp reads the 32 tensor-memory lanes 32*(warp%4)..
    float* stage_out = sh->stage_out[warp - 2];
    int local = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const TcTile t = tc_tile(item % total, row_tiles, M, N, BN, offsets, groups);
      if (!t.valid) continue;
      OutT* Cp = C + (size_t)(item / total) * M * N;        // the part's plane (C itself without a split)
      const int buf = local & 1;
      mbar_wait(&sh->acc_full[buf], (local >> 1) & 1, aborted, TC_ERR_WAIT_ACC);
      if (__any_sync(0xffffffffu, *aborted)) break;        // the whole warp leaves together
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        if (c0 + 32 >= BN) {                             // everything of this accumulator is in registers
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->acc_empty[buf]);
        }
        if (!*aborted)
          tc_store_piece<OutT, SWIGLU>(r, stage_out, lane, Cp, t.row0 + lane_group * 32, t.row_end, t.n0 + c0, N);
      }
      ++local;
    }
  }
  if (*aborted) drain_after_abort();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)(2 * BN))
                 : "memory");
  }
}

template <int BN, typename OutT, bool SWIGLU>
static int launch_tc(const CUtensorMap& map_a, const CUtensorMap& map_w, void* C, int M, int N, int K,
                     const int* offsets, int groups, int row_tiles, int splits, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (TC_BM + BN) * TC_BK * 2;
  constexpr int STAGES = TC_SMEM_TILES / STAGE_BYTES < TC_MAX_STAGES ? TC_SMEM_TILES / STAGE_BYTES : TC_MAX_STAGES;
  const size_t smem = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(TcShared);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_tc_kernel<BN, OutT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const long long tiles = (long long)row_tiles * ((N + BN - 1) / BN) * splits;
  const int blocks = (int)(tiles < sms ? tiles : sms);     // one block per SM (shared memory), persistent
  snk_launch(gemm_tc_kernel<BN, OutT, SWIGLU>, dim3(blocks), dim3(TC_THREADS), smem, stream, map_a, map_w, static_cast<OutT*>(C), M, N, K,
                                                                 offsets, groups, row_tiles, splits);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Products with few tiles (one row tile, a narrow N: the projections of a 64-row decode step) would leave
// most SMs idle behind a long serial walk over K.  They are split along K into parts that run side by
// side; each part leaves its float partial product in a plane of scratch, and a second kernel adds the
// planes in part order and stores C (converted, or through SwiGLU).
template <typename OutT, bool SWIGLU>
__global__ void splitk_reduce_kernel(const float* __restrict__ parts, OutT* __restrict__ C, int M, int N, int splits) {
  pdl_begin();
  const size_t plane = (size_t)M * N;
  if constexpr (SWIGLU) {
    // blocks of 16 columns: 8 gate columns, then the 8 up columns of the same features
    const size_t blocks = plane / 16;
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < splits; ++p) {
      const float4* src = reinterpret_cast<const float4*>(parts + (size_t)p * plane + b * 16);
      const float4 g0 = src[0], g1 = src[1], u0 = src[2], u1 = src[3];
      g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w; g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
      u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w; u[4] += u1.x; u[5] += u1.y; u[6] += u1.z; u[7] += u1.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(g[2 * j] / (1.f + expf(-g[2 * j])) * u[2 * j],
                                                     g[2 * j + 1] / (1.f + expf(-g[2 * j + 1])) * u[2 * j + 1]);
      o[j] = *reinterpret_cast<const uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(C + b * 8) = make_uint4(o[0], o[1], o[2], o[3]);   // row m, features 8*(b % (N/16))..
  } else {
    const size_t vecs = plane / 4;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vecs) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < splits; ++p) {
      const float4 v = reinterpret_cast<const float4*>(parts + (size_t)p * plane)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    store4<OutT>(C + 4 * i, acc.x, acc.y, acc.z, acc.w);
  }
}

// How many parts along K a plain product of these sizes is split into (1: none).
static int tc_splits(int M, int N, int K, const int* offsets) {
  static int sms = 0;
  static int off = -1;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const char* e = getenv("SNOWLLM_B200_TC_SPLIT");
    off = (e && e[0] == '0') ? 1 : 0;
  }
  if (offsets || off || N % 16) return 1;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int tiles = ((M + TC_BM - 1) / TC_BM) * ((N + 127) / 128);
  int splits = sms / tiles;                                   // parts that still find an SM each
  if (splits > 8) splits = 8;
  if (splits > k_tiles / 4) splits = k_tiles / 4;             // a part walks at least four k-blocks
  if (splits < 2) return 1;
  const int k_per = (k_tiles + splits - 1) / splits;
  return (k_tiles + k_per - 1) / k_per;                       // no part without k-blocks
}

// Bytes of scratch snk_gemm_tc wants for these sizes (0: none).
SNK_API long long snk_gemm_tc_scratch_bytes(int M, int N, int K, int grouped) {
  if (grouped) return 0;
  const int splits = tc_splits(M, N, K, nullptr);
  return splits > 1 ? (long long)splits * M * N * (long long)sizeof(float) : 0;
}

// M: rows of A (all groups together).  Grouped: offsets[groups+1] on the device, W = [groups, N, K];
// max_row_tiles bounds the number of 128-row tiles over all groups (M/128 + groups is always enough).
// scratch: snk_gemm_tc_scratch_bytes of device memory (may be null when that is 0).
SNK_API int snk_gemm_tc(const void* A, const void* W, void* C, int M, int N, int K, const int* offsets,
                        int groups, int max_row_tiles, int out_f32, int swiglu, void* scratch,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) return SNK_ERR_SIZE;                   // TMA: the row pitch is a multiple of 16 bytes
  if (swiglu && (N % 16 || out_f32)) return SNK_ERR_SIZE;
  if (((uintptr_t)A % 16) || ((uintptr_t)W % 16) || ((uintptr_t)C % 16)) return SNK_ERR_ALIGN;
  const int row_tiles = offsets ? max_row_tiles : (M + TC_BM - 1) / TC_BM;
  if (row_tiles <= 0) return SNK_ERR_SIZE;
  // wide tiles where they still give every SM work; narrow ones otherwise
  const bool wide = (long long)((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256) >= 120;
  const int splits = wide ? 1 : tc_splits(M, N, K, offsets);
  if (splits > 1 && (scratch == nullptr || ((uintptr_t)scratch % 16))) return SNK_ERR_ALIGN;
  CUtensorMap map_a, map_w;
  int rc = tensor_map(A, M, K, TC_BM, TC_BK, &map_a);
  if (rc) return rc;
  rc = tensor_map(W, (long long)(offsets ? groups : 1) * N, K, wide ? 256 : 128, TC_BK, &map_w);
  if (rc) return rc;
  if (splits > 1) {
    rc = launch_tc<128, float, false>(map_a, map_w, scratch, M, N, K, nullptr, 1, row_tiles, splits, stream);
    if (rc) return rc;
    const float* parts = static_cast<const float*>(scratch);
    const size_t work = swiglu ? (size_t)M * N / 16 : (size_t)M * N / 4;
    const dim3 grid((unsigned)((work + 255) / 256)), block(256);
    if (swiglu) snk_launch(splitk_reduce_kernel<bf16, true>, grid, block, 0, stream, parts, static_cast<bf16*>(C), M, N, splits);
    else if (out_f32) snk_launch(splitk_reduce_kernel<float, false>, grid, block, 0, stream, parts, static_cast<float*>(C), M, N, splits);
    else snk_launch(splitk_reduce_kernel<bf16, false>, grid, block, 0, stream, parts, static_cast<bf16*>(C), M, N, splits);
    SNK_LAUNCH_CHECK();
    return 0;
  }
#define TC_GO(BN_, T_, S_) launch_tc<BN_, T_, S_>(map_a, map_w, C, M, N, K, offsets, groups, row_tiles, 1, stream)
  if (swiglu) return wide ? TC_GO(256, bf16, true) : TC_GO(128, bf16, true);
  if (wide) return out_f32 ? TC_GO(256, float, false) : TC_GO(256, bf16, false);
  return out_f32 ? TC_GO(128, float, false) : TC_GO(128, bf16, false);
#undef TC_GO
}

// The product split along K with the sum left to the caller: `parts` receives the float planes
// [splits][M][N], to be added in plane order (what splitk_reduce_kernel does).  Returns the number of planes
// through *splits_out; products that are not split (see snk_gemm_tc_scratch_bytes) give SNK_ERR_SIZE.
SNK_API int snk_gemm_tc_parts(const void* A, const void* W, void* parts, int M, int N, int K, int* splits_out,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 8) return SNK_ERR_SIZE;
  if (((uintptr_t)A % 16) || ((uintptr_t)W % 16) || parts == nullptr || ((uintptr_t)parts % 16)) return SNK_ERR_ALIGN;
  const bool wide = (long long)((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256) >= 120;
  const int splits = wide ? 1 : tc_splits(M, N, K, nullptr);
  if (splits <= 1) return SNK_ERR_SIZE;
  CUtensorMap map_a, map_w;
  int rc = tensor_map(A, M, K, TC_BM, TC_BK, &map_a);
  if (rc) return rc;
  rc = tensor_map(W, N, K, 128, TC_BK, &map_w);
  if (rc) return rc;
  *splits_out = splits;
  return launch_tc<128, float, false>(map_a, map_w, parts, M, N, K, nullptr, 1, (M + TC_BM - 1) / TC_BM, splits, stream);
}

// Test hook: with on != 0 the producers of later launches issue no loads, so that the bounded waits run out
// (about 1.5 s) and the launches return with an error status instead of a product.  Synchronises.
SNK_API int snk_gemm_tc_test_lose_loads(int on) {
  return (int)cudaMemcpyToSymbol(g_tc_lose_loads, &on, sizeof(int));
}

// Queue a copy of the status word into ``host`` (pinned host memory, one int) on ``stream`` without waiting
// for it and without clearing it: a caller that synchronises with the stream anyway (an event, a read-back)
// learns of a wait that ran out at no cost.  Not for use inside a stream capture.
SNK_API int snk_gemm_tc_status_peek(int* host, void* stream) {
  return (int)cudaMemcpyFromSymbolAsync(host, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

// 0, or the first error a block of any earlier launch recorded (a wait that ran out); reading clears
// it.  Synchronises the device.
SNK_API int snk_gemm_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  return v;
}

// ---------------------------------------------------------------------------------------------
// out[r, :] = in[rows[r] / div, :]  (bfloat16 rows of K elements, K a multiple of 8)
#define GATHER_ROWS_PER_BLOCK 8
__global__ void gather_rows_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                   const int* __restrict__ rows, int div, int vecs, int R) {
  pdl_begin();
  // a block copies GATHER_ROWS_PER_BLOCK rows; every thread has one vector of each row in flight
  const int r0 = blockIdx.x * GATHER_ROWS_PER_BLOCK;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    uint4 v[GATHER_ROWS_PER_BLOCK];
#pragma unroll
    for (int j = 0; j < GATHER_ROWS_PER_BLOCK; ++j)
      if (r0 + j < R) v[j] = in[(size_t)(rows[r0 + j] / div) * vecs + i];
#pragma unroll
    for (int j = 0; j < GATHER_ROWS_PER_BLOCK; ++j)
      if (r0 + j < R) out[(size_t)(r0 + j) * vecs + i] = v[j];
  }
}

SNK_API int snk_gather_rows_bf16(const void* in, void* out, const int* rows, int div, int R, int K,
                                 cudaStream_t stream) {
  if (R <= 0) return 0;
  if (K % 8 || ((uintptr_t)in % 16) || ((uintptr_t)out % 16)) return SNK_ERR_ALIGN;
  snk_launch(gather_rows_kernel, dim3((R + GATHER_ROWS_PER_BLOCK - 1) / GATHER_ROWS_PER_BLOCK), dim3(256), 0, stream,
             static_cast<const uint4*>(in), static_cast<uint4*>(out), rows, div <= 0 ? 1 : div, K / 8, R);
  SNK_LAUNCH_CHECK();
  return 0;
}
