// C[M,N] = A[M,K] . W[N,K]^T in bfloat16 on the tcgen05 tensor cores with PAIRS of SMs (cta_group::2), for
// many rows (prefill).  The one-SM kernel of gemm_tc.cu is bound by what L2 feeds an SM: 48 KB of operands per
// k-block of a 128 x 256 tile.  Here a cluster of two blocks owns a 256 x 256 tile of C: each block loads its own
// 128 rows of A and HALF of the 256 rows of W (32 KB per k-block), the leader block issues one MMA of M 256 for
// both, and the tensor cores of the two SMs read the other block's half of W across the pair.  A third less
// operand traffic per product.
//
//   warp 0, one lane   TMA producer (both blocks): 128x64 of A and 128x64 of W into this block's stage ring; the
//                      bytes of both blocks count towards the LEADER's stage barrier (cta_group::2 loads)
//   warp 1, one lane   leader only: waits for the stage, issues four tcgen05.mma.cta_group::2; a multicast commit
//                      frees the stage in both blocks and, after the last k-block, hands the accumulator to both
//                      epilogues
//   warps 2..5         epilogue (both blocks): tcgen05.ld of this block's 128 accumulator rows, stores; then an
//                      arrival on the leader's accumulator-free barrier (remote from the peer)
//
// Row tiles are 256 rows.  Grouped products run the kernel further down, with the operands changed round.
// Every mbarrier wait is bounded by wall time (see snk_gemm_tc2_status); when one runs out both blocks of the pair
// stop issuing loads and products, give the copies in flight a moment to land, free their tensor memory and
// return.  No TMA load is multicast: each block loads what it owns.
#include "tcgen05.cuh"

#define T2_BM 128                     // rows of A per block (256 per pair)
#define T2_BN 256                     // columns of C per pair; each block loads T2_BN / 2 rows of W
#define T2_BK 64
#define T2_THREADS 192
#define T2_STAGE_BYTES ((T2_BM + T2_BN / 2) * T2_BK * 2)
#ifndef T2_STAGES
#define T2_STAGES 6
#endif
#ifndef T2_BAND
#define T2_BAND 8
#endif
#define T2_WAIT_NS 1500000000ull
#ifndef T2_ACC_BUFFERS
#define T2_ACC_BUFFERS 2              // accumulators in tensor memory: the epilogue of a tile overlaps the next tile's products
#endif

enum { T2_ERR_FULL = 1, T2_ERR_EMPTY = 2, T2_ERR_ACC = 3, T2_ERR_ACC_FREE = 4, T2_ERR_PEER = 5 };

__device__ int g_t2_status;
__device__ int g_t2_lose_loads;      // test hook: producers issue no loads (the operands then never arrive)
__device__ unsigned int g_t2_tmem[2];  // the tensor-memory base addresses the two blocks of cluster 0 were given (a probe)

__device__ __forceinline__ void t2_wait(uint64_t* bar, uint32_t parity, volatile int* aborted, int code) {
  if (*aborted) return;
  if (mbar_try_wait(bar, parity)) return;
  const uint64_t start = global_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (*aborted) return;
    if (global_ns() - start > T2_WAIT_NS) {
      *aborted = 1;
      st_cluster_u32(const_cast<int*>(aborted), cluster_ctarank() ^ 1u, 1u);   // the other block of the pair stops too
      atomicCAS(&g_t2_status, 0, code);
      return;
    }
  }
}

struct __align__(16) T2Shared {
  uint64_t full[T2_STAGES];         // (leader) both blocks' stages hold their operands
  uint64_t empty[T2_STAGES];        // the MMAs that read the stage have completed (both blocks)
  uint64_t acc_full[2];             // the tile's products have completed (both blocks)
  uint64_t acc_empty[2];            // (leader) both epilogues have read the accumulator: 8 arrivals
  uint32_t tmem_base;
  int aborted;
  __align__(16) float stage_out[4][TC_STAGE_FLOATS];    // one staging tile per epilogue warp (tc_store_piece)
};

struct T2Tile {
  int row0, row_end, w_row0, n0;
  bool valid;
};

// Pair tile `tile`: 256 rows x 256 columns.
__device__ __forceinline__ T2Tile t2_tile(int tile, int row_tiles, int M, int N) {
  T2Tile t;
  // bands of up to T2_BAND n-tiles, the n-tile fastest inside a band, then the row tile (as in gemm_tc.cu)
  const int n_tiles = (N + T2_BN - 1) / T2_BN;
  const int bands = (n_tiles + T2_BAND - 1) / T2_BAND;
  const int band_w = (n_tiles + bands - 1) / bands;
  const int per_band = row_tiles * band_w;
  const int band = tile / per_band, in_band = tile % per_band;
  const int w_here = min(band_w, n_tiles - band * band_w);
  const int rt = in_band / w_here, nt = band * band_w + in_band % w_here;
  t.n0 = nt * T2_BN;
  t.valid = t.n0 < N;
  t.row0 = rt * 2 * T2_BM;
  t.row_end = M;
  t.w_row0 = 0;
  return t;
}

template <typename OutT, bool SWIGLU>
__global__ void __launch_bounds__(T2_THREADS)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                OutT* __restrict__ C, int M, int N, int K, int row_tiles) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  T2Shared* sh = reinterpret_cast<T2Shared*>(tiles + (size_t)T2_STAGES * T2_STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();               // 0: leader, 1: peer
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;     // pairs lie along x
  const int k_tiles = (K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 8);                   // four epilogue warps of each block
    }
    sh->aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh->tmem_base)), "r"((uint32_t)(T2_ACC_BUFFERS * T2_BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync();                                        // both blocks' barriers and tensor memory are set up
  tc_fence_after();
  // the accumulator's address is the leader's: the MMA writes rows 128..255 at the same columns of the peer
  const uint32_t tmem_acc = rank == 0 ? sh->tmem_base : ld_cluster_u32(&sh->tmem_base, 0);
  if (pair == 0 && threadIdx.x == 0) g_t2_tmem[rank] = sh->tmem_base;
  volatile int* aborted = &sh->aborted;
  pdl_begin();
  const int n_tiles = (N + T2_BN - 1) / T2_BN;
  const int total = row_tiles * n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      const bool lose_loads = *const_cast<volatile int*>(&g_t2_lose_loads) != 0;
      for (int tile = pair; tile < total && !*aborted; tile += pairs) {
        const T2Tile t = t2_tile(tile, row_tiles, M, N);
        if (!t.valid) continue;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % T2_STAGES;
          t2_wait(&sh->empty[s], ((it / T2_STAGES) & 1) ^ 1, aborted, T2_ERR_EMPTY);
          if (*aborted) break;                           // a wait ran out: nothing more is issued
          if (lose_loads) continue;
          // both blocks' bytes count towards the leader's barrier: it is the leader that issues the MMAs
          if (rank == 0) mbar_expect_tx(&sh->full[s], 2 * T2_STAGE_BYTES);
          const uint32_t bar = cluster_addr(&sh->full[s], 0);
          unsigned char* stage = tiles + (size_t)s * T2_STAGE_BYTES;
          tma2_load_2d(stage, &map_a, bar, kt * T2_BK, t.row0 + (int)rank * T2_BM);
          tma2_load_2d(stage + T2_BM * T2_BK * 2, &map_w, bar, kt * T2_BK, t.w_row0 + t.n0 + (int)rank * (T2_BN / 2));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {                        // the leader issues for the pair; the peer's warp rests
      const uint32_t idesc = instr_desc_bf16(2 * T2_BM, T2_BN);
      int it = 0, local = 0;
      for (int tile = pair; tile < total && !*aborted; tile += pairs) {
        const T2Tile t = t2_tile(tile, row_tiles, M, N);
        if (!t.valid) continue;
        const int buf = local % T2_ACC_BUFFERS;
        const int use = local / T2_ACC_BUFFERS;          // how often this accumulator was used before
        t2_wait(&sh->acc_empty[buf], (use & 1) ^ 1, aborted, T2_ERR_ACC_FREE);
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + (uint32_t)(buf * T2_BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % T2_STAGES;
          t2_wait(&sh->full[s], (it / T2_STAGES) & 1, aborted, T2_ERR_FULL);   // both blocks' stage s
          if (*aborted) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * T2_STAGE_BYTES);
          const uint32_t w_addr = a_addr + T2_BM * T2_BK * 2;
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            umma2_bf16(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(w_addr + k * 32), idesc,
                       (kt > 0 || k > 0) ? 1u : 0u);
          umma2_commit(&sh->empty[s], 3);                // the stage is free in both blocks once these MMAs have read it
        }
        if (*aborted) break;
        umma2_commit(&sh->acc_full[buf], 3);
        ++local;
      }
    }
  } else {
    const int lane_group = warp & 3;
    float* stage_out = sh->stage_out[warp - 2];
    int local = 0;
    for (int tile = pair; tile < total; tile += pairs) {
      const T2Tile t = t2_tile(tile, row_tiles, M, N);
      if (!t.valid) continue;
      const int buf = local % T2_ACC_BUFFERS;
      const int use = local / T2_ACC_BUFFERS;
      t2_wait(&sh->acc_full[buf], use & 1, aborted, T2_ERR_ACC);
      if (__any_sync(0xffffffffu, *aborted)) break;      // the whole warp leaves together
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < T2_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * T2_BN + c0), r);
        if (c0 + 32 >= T2_BN) {                          // everything of this accumulator is in registers
          tc_fence_before();
          __syncwarp();
          if (lane == 0 && !*aborted) {
            if (rank == 0) mbar_arrive(&sh->acc_empty[buf]);
            else mbar_arrive_remote(&sh->acc_empty[buf], 0);
          }
        }
        if (!*aborted)
          tc_store_piece<OutT, SWIGLU>(r, stage_out, lane, C, t.row0 + (int)rank * T2_BM + lane_group * 32, t.row_end,
                                       t.n0 + c0, N);
      }
      ++local;
    }
  }
  if (*aborted) drain_after_abort();
  tc_fence_before();
  cluster_sync();                                        // nobody of the pair touches tensor memory or barriers any more
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                 ::"r"(sh->tmem_base), "r"((uint32_t)(T2_ACC_BUFFERS * T2_BN)) : "memory");
  }
}

template <typename OutT, bool SWIGLU>
static int launch_tc2(const CUtensorMap& map_a, const CUtensorMap& map_w, void* C, int M, int N, int K,
                      int row_tiles, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)T2_STAGES * T2_STAGE_BYTES + sizeof(T2Shared);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_tc2_kernel<OutT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const long long tiles = (long long)row_tiles * ((N + T2_BN - 1) / T2_BN);
  const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
  snk_launch_cluster3(gemm_tc2_kernel<OutT, SWIGLU>, dim3(2 * pairs), dim3(T2_THREADS), smem, stream, dim3(2, 1, 1),
                      map_a, map_w, static_cast<OutT*>(C), M, N, K, row_tiles);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Grouped products (experts): the operands change places.  With rows of A as the 128-row operand a group of
// 270 rows costs three one-SM tiles (two pair tiles), each as dear as a full one, and what bounds a tile is
// the operand bytes an SM takes in.  Here W is the 256-row operand of the pair (each block loads 128 rows of
// W: 16 KB per k-block) and the group's ROWS are the N side of the MMA, which may be any multiple of 16 up
// to 256: a tile is 256 columns of C by up to 256 rows, a group's last tile is as wide as it needs, and each
// block loads half of the tile's rows of A.  The accumulator holds C transposed (lanes: columns of C); the
// epilogue turns it back.
//
// Items in order: group, then 256-column tile of C, then the group's row tiles, so that the pairs that
// read the same rows of W run side by side; item i goes to pair i % pairs.  (Measured and dropped: runs of
// neighbouring items of equal modelled cost per pair, 157 -> 180 us on the experts' gate|up product of 2,048
// tokens, as pairs side by side then read far-apart memory; items drawn from a counter as pairs get free,
// 159 us; L2 prefetch of an item's rows of W in one piece, 184 to 198 us.)
#define T2G_MAX_GROUPS 256
#define T2G_STAGE_BYTES ((T2_BM + T2_BM) * T2_BK * 2)  // 128 rows of W and up to 128 of the tile's rows of A
#define T2G_BOXES 5                  // tensor maps of A with boxes of 128, 64, 32, 16 and 8 rows

struct T2GMaps {
  CUtensorMap a[T2G_BOXES];
};

struct T2GItem {
  int row0, row_end, nt, w_row0, f0;  // rows row0 .. of A (nt of them in the MMA, a multiple of 16), W rows w_row0 + f0 ..
  bool valid;
};

// first[e]: the number of items before group e (shared memory, groups + 1 entries)
__device__ __forceinline__ T2GItem t2g_item(int item, const int* first, const int* __restrict__ offsets, int groups,
                                            int N) {
  T2GItem t;
  t.valid = false;
  int lo = 0, hi = groups;                               // the group e with first[e] <= item < first[e + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (first[mid] <= item) lo = mid; else hi = mid;
  }
  if (item >= first[groups]) return t;
  const int begin = offsets[lo], cnt = offsets[lo + 1] - begin;
  const int row_tiles = (cnt + 2 * T2_BM - 1) / (2 * T2_BM);
  const int in_group = item - first[lo];
  const int ft = in_group / row_tiles, tt = in_group % row_tiles;
  // A group's rows are dealt evenly to its row tiles (in steps of 16): every tile streams the same rows of W,
  // so a group of 270 rows as 144 + 128 costs two half-length products, where 256 + 16 costs a full one and
  // a second pass over W for 16 rows (with 2,048 tokens, top 4 of 32 experts, half the groups are just
  // above 256 rows).
  const int per = ((cnt + row_tiles - 1) / row_tiles + 15) & ~15;
  t.row0 = begin + tt * per;
  t.row_end = min(begin + cnt, t.row0 + per);
  const int left = t.row_end - t.row0;
  t.nt = left <= 0 ? 16 : (left + 15) & ~15;
  t.w_row0 = lo * N;
  t.f0 = ft * T2_BN;
  t.valid = true;
  return t;
}

// The box of A for nt / 2 rows per block: the smallest of 128, 64, 32, 16, 8 that holds them.
__device__ __forceinline__ int t2g_box(int half_rows) {
  int b = 0, rows = 128;
  while (b + 1 < T2G_BOXES && (rows >> 1) >= half_rows) { rows >>= 1; ++b; }
  return b;
}

template <typename OutT, bool SWIGLU>
__global__ void __launch_bounds__(T2_THREADS)
gemm_tc2_grouped_kernel(const __grid_constant__ T2GMaps maps, const __grid_constant__ CUtensorMap map_w,
                        OutT* __restrict__ C, int N, int K, const int* __restrict__ offsets, int groups) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  T2Shared* sh = reinterpret_cast<T2Shared*>(tiles + (size_t)T2_STAGES * T2G_STAGE_BYTES);
  int* first = reinterpret_cast<int*>(sh + 1);           // groups + 1 entries

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int k_tiles = (K + T2_BK - 1) / T2_BK;
  const int n_tiles = (N + T2_BN - 1) / T2_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 8);
    }
    sh->aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh->tmem_base)), "r"((uint32_t)(T2_ACC_BUFFERS * T2_BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_acc = rank == 0 ? sh->tmem_base : ld_cluster_u32(&sh->tmem_base, 0);
  volatile int* aborted = &sh->aborted;
  pdl_begin();                                           // offsets are written by the kernel before this one
  for (int e = threadIdx.x; e < groups; e += blockDim.x)  // the groups' item counts side by side, then their running sum
    first[e + 1] = ((offsets[e + 1] - offsets[e] + 2 * T2_BM - 1) / (2 * T2_BM)) * n_tiles;
  __syncthreads();
  if (threadIdx.x == 0) {
    first[0] = 0;
    for (int e = 0; e < groups; ++e) first[e + 1] += first[e];
  }
  __syncthreads();
  const int total = first[groups];

  int it = 0;                                            // k-blocks so far (producer and MMA thread)
  const bool lose_loads = *const_cast<volatile int*>(&g_t2_lose_loads) != 0;
  auto issue_loads = [&](int item) {
    const T2GItem t = t2g_item(item, first, offsets, groups, N);
    const int half = t.nt >> 1, box = t2g_box(half);
    const uint32_t bytes = (uint32_t)(T2_BM * T2_BK * 2 + (128 >> box) * T2_BK * 2);
    for (int kt = 0; kt < k_tiles; ++kt, ++it) {
      const int s = it % T2_STAGES;
      t2_wait(&sh->empty[s], ((it / T2_STAGES) & 1) ^ 1, aborted, T2_ERR_EMPTY);
      if (*aborted) return;                              // a wait ran out: nothing more is issued
      if (lose_loads) continue;
      if (rank == 0) mbar_expect_tx(&sh->full[s], 2 * bytes);
      const uint32_t bar = cluster_addr(&sh->full[s], 0);
      unsigned char* stage = tiles + (size_t)s * T2G_STAGE_BYTES;
      tma2_load_2d(stage, &map_w, bar, kt * T2_BK, t.w_row0 + t.f0 + (int)rank * T2_BM);
      tma2_load_2d(stage + T2_BM * T2_BK * 2, &maps.a[box], bar, kt * T2_BK, t.row0 + (int)rank * half);
    }
  };

  if (warp == 0) {
    if (lane == 0)
      for (int item = pair; item < total && !*aborted; item += pairs) issue_loads(item);
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      int local = 0;
      for (int item = pair; item < total && !*aborted; item += pairs, ++local) {
        const T2GItem t = t2g_item(item, first, offsets, groups, N);
        const uint32_t idesc = instr_desc_bf16(2 * T2_BM, t.nt);
        const int buf = local % T2_ACC_BUFFERS;
        const int use = local / T2_ACC_BUFFERS;
        t2_wait(&sh->acc_empty[buf], (use & 1) ^ 1, aborted, T2_ERR_ACC_FREE);
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + (uint32_t)(buf * T2_BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % T2_STAGES;
          t2_wait(&sh->full[s], (it / T2_STAGES) & 1, aborted, T2_ERR_FULL);
          if (*aborted) break;
          tc_fence_after();
          const uint32_t w_addr = smem_u32(tiles + (size_t)s * T2G_STAGE_BYTES);
          const uint32_t a_addr = w_addr + T2_BM * T2_BK * 2;
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            umma2_bf16(d_tmem, smem_desc_sw128(w_addr + k * 32), smem_desc_sw128(a_addr + k * 32), idesc,
                       (kt > 0 || k > 0) ? 1u : 0u);
          umma2_commit(&sh->empty[s], 3);
        }
        if (*aborted) break;
        umma2_commit(&sh->acc_full[buf], 3);
      }
    }
  } else {
    const int lane_group = warp & 3;
    float* stage_out = sh->stage_out[warp - 2];
    int local = 0;
    for (int item = pair; item < total; item += pairs, ++local) {
      const T2GItem t = t2g_item(item, first, offsets, groups, N);
      const int buf = local % T2_ACC_BUFFERS;
      const int use = local / T2_ACC_BUFFERS;
      t2_wait(&sh->acc_full[buf], use & 1, aborted, T2_ERR_ACC);
      if (__any_sync(0xffffffffu, *aborted)) break;      // the whole warp leaves together
      tc_fence_after();
      const int col0 = t.f0 + (int)rank * T2_BM + lane_group * 32;     // this warp's 32 columns of C: one per lane
#pragma unroll 1
      for (int c0 = 0; c0 < t.nt; c0 += 32) {
        uint32_t r[32];                                  // this lane's column of C at rows row0 + c0 ..
        tmem_ld32(tmem_acc + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * T2_BN + c0), r);
        if (c0 + 32 >= t.nt) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0 && !*aborted) {
            if (rank == 0) mbar_arrive(&sh->acc_empty[buf]);
            else mbar_arrive_remote(&sh->acc_empty[buf], 0);
          }
        }
        if (*aborted) continue;
        if constexpr (SWIGLU) {
          // turned in shared memory: lane = row, 32 columns (8 gates, their 8 ups, twice), as tc_store_piece wants
#pragma unroll
          for (int j = 0; j < 32; ++j) stage_out[j * TC_STAGE_PITCH + lane] = __uint_as_float(r[j]);
          __syncwarp();
          uint32_t q[32];
          const uint4* mine = reinterpret_cast<const uint4*>(stage_out + lane * TC_STAGE_PITCH);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = mine[c];
            q[4 * c] = v.x; q[4 * c + 1] = v.y; q[4 * c + 2] = v.z; q[4 * c + 3] = v.w;
          }
          __syncwarp();
          tc_store_piece<OutT, true>(q, stage_out, lane, C, t.row0 + c0, t.row_end, col0, N);
        } else {
          // a warp's store writes 32 neighbouring columns of one row
          if (col0 + lane < N) {
            OutT* dst = C + (size_t)(t.row0 + c0) * N + col0 + lane;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (t.row0 + c0 + j < t.row_end) dst[(size_t)j * N] = from_f<OutT>(__uint_as_float(r[j]));
          }
        }
      }
    }
  }
  if (*aborted) drain_after_abort();
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                 ::"r"(sh->tmem_base), "r"((uint32_t)(T2_ACC_BUFFERS * T2_BN)) : "memory");
  }
}

template <typename OutT, bool SWIGLU>
static int launch_tc2_grouped(const T2GMaps& maps, const CUtensorMap& map_w, void* C, int M, int N, int K,
                              const int* offsets, int groups, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)T2_STAGES * T2G_STAGE_BYTES + sizeof(T2Shared) + (T2G_MAX_GROUPS + 1) * sizeof(int);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_tc2_grouped_kernel<OutT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  // at most M / 256 full row tiles and one partial tile per group
  const long long items = ((long long)M / (2 * T2_BM) + groups) * ((N + T2_BN - 1) / T2_BN);
  const int pairs = (int)(items < sms / 2 ? items : sms / 2);
  snk_launch_cluster3(gemm_tc2_grouped_kernel<OutT, SWIGLU>, dim3(2 * pairs), dim3(T2_THREADS), smem, stream,
                      dim3(2, 1, 1), maps, map_w, static_cast<OutT*>(C), N, K, offsets, groups);
  SNK_LAUNCH_CHECK();
  return 0;
}

// M: rows of A (all groups together).  Grouped: offsets[groups+1] on the device, W = [groups, N, K].
SNK_API int snk_gemm_tc2(const void* A, const void* W, void* C, int M, int N, int K, const int* offsets,
                         int groups, int out_f32, int swiglu, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) return SNK_ERR_SIZE;
  if (swiglu && (N % 16 || out_f32)) return SNK_ERR_SIZE;
  if (((uintptr_t)A % 16) || ((uintptr_t)W % 16) || ((uintptr_t)C % 16)) return SNK_ERR_ALIGN;
  if (offsets) {
    if (groups <= 0 || groups > T2G_MAX_GROUPS) return SNK_ERR_SIZE;
    T2GMaps maps;
    for (int b = 0; b < T2G_BOXES; ++b) {
      const int rc = tensor_map(A, M, K, 128 >> b, T2_BK, &maps.a[b]);
      if (rc) return rc;
    }
    CUtensorMap gw;
    const int rc = tensor_map(W, (long long)groups * N, K, T2_BM, T2_BK, &gw);
    if (rc) return rc;
    if (swiglu) return launch_tc2_grouped<bf16, true>(maps, gw, C, M, N, K, offsets, groups, stream);
    if (out_f32) return launch_tc2_grouped<float, false>(maps, gw, C, M, N, K, offsets, groups, stream);
    return launch_tc2_grouped<bf16, false>(maps, gw, C, M, N, K, offsets, groups, stream);
  }
  const int row_tiles = (M + 2 * T2_BM - 1) / (2 * T2_BM);
  if (row_tiles <= 0) return SNK_ERR_SIZE;
  CUtensorMap map_a, map_w;
  int rc = tensor_map(A, M, K, T2_BM, T2_BK, &map_a);
  if (rc) return rc;
  rc = tensor_map(W, N, K, T2_BN / 2, T2_BK, &map_w);
  if (rc) return rc;
  if (swiglu) return launch_tc2<bf16, true>(map_a, map_w, C, M, N, K, row_tiles, stream);
  if (out_f32) return launch_tc2<float, false>(map_a, map_w, C, M, N, K, row_tiles, stream);
  return launch_tc2<bf16, false>(map_a, map_w, C, M, N, K, row_tiles, stream);
}

// Test hook: with on != 0 the producers of later launches issue no loads, so that the bounded waits run out
// (about 1.5 s) and the launches return with an error status instead of a product.  Synchronises.
SNK_API int snk_gemm_tc2_test_lose_loads(int on) {
  return (int)cudaMemcpyToSymbol(g_t2_lose_loads, &on, sizeof(int));
}

// Queue a copy of the status word into ``host`` (pinned host memory, one int) on ``stream`` without waiting
// for it and without clearing it: a caller that synchronises with the stream anyway (an event, a read-back)
// learns of a wait that ran out at no cost.  Not for use inside a stream capture.
SNK_API int snk_gemm_tc2_status_peek(int* host, void* stream) {
  return (int)cudaMemcpyFromSymbolAsync(host, g_t2_status, sizeof(int), 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

// 0, or the first error a block of any earlier launch recorded (a wait that ran out); reading clears it.
// tmem (may be null): the tensor-memory addresses the two blocks of the first pair were given.  Synchronises.
SNK_API int snk_gemm_tc2_status(unsigned int* tmem) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_t2_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_t2_status, &zero, sizeof(int));
  if (tmem && cudaMemcpyFromSymbol(tmem, g_t2_tmem, 2 * sizeof(unsigned int)) != cudaSuccess) return -1;
  return v;
}
