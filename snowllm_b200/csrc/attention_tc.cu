// Causal attention for prompt portions on the tcgen05 tensor cores, head size 64, bfloat16.
//
//   S = Q K^T * scale; key kp is seen by the row at position p when lo(p) <= kp <= p, lo(p) = 0 or
//   p - window + 1; P = softmax(S) in float (base-2 exponentials of scores scaled by log2 e), rounded to
//   bfloat16 for P V; O = P V / sum(P) accumulated in float
//   (snowllm/ops/attention_full.py:14-38; snowllm/models/lfm2/layers.py:60-71)
//
// One block takes 128 rows of one request and one q head and walks the keys in tiles of 128:
//   warp 0        TMA: the block's rows of q once, then per key tile the pages that hold its keys and
//                 values (a box is one page's rows of one kv head, 64 elements wide, 128-byte swizzle)
//                 into two rings, AT_KSTAGES slots of keys and AT_VSTAGES slots of values
//   warp 1        one lane issues the MMAs: S[j] = Q K[j]^T (M 128, N 128, four k-steps) into tensor
//                 memory, then, once the softmax warps have written P[j] to shared memory,
//                 O += P[j] V[j] (M 128, N 64, eight k-steps; V is the MN-major operand: its rows are keys
//                 as they lie in the cache).  S[j+1] is issued as soon as the softmax warps hold S[j] in
//                 registers, before P[j] V[j]: the tensor cores work on the next scores meanwhile.
//   warps 2..5    softmax: a thread owns a row.  It reads its 128 scores from tensor memory, masks them
//                 in tiles that cross a causal or window edge, keeps the running maximum and sum,
//                 writes its row of P in the swizzled layout the MMA reads, and rescales its row of O
//                 in tensor memory when the reference maximum moved (it moves only when the row's maximum
//                 has grown by more than 8 in the exponent: until then the exponentials are taken against
//                 the old one, which float holds easily, and O needs no pass).  At the end it divides O
//                 by the sum and stores its row.  (Two threads per row, half the keys each, were slower:
//                 981 against 654 us on 8,192 tokens.)
// Two blocks share an SM (112 KB of shared memory and 256 columns of tensor memory each): while one
// block's softmax warps compute, the other's are there to issue, and so are its MMAs.
// Pages are loaded whole; pages without a key of [lowest key any row sees, last row's position] are not
// loaded, so value rows outside that range are zeroed in shared memory before the MMA reads them (their
// P is zero, but zero times stale bits is not), and scores there are masked.
// A row's sums do not depend on the block it is in: key tiles start at multiples of 128 counted from
// the window's first tile, and a tile in which the row sees no key leaves its state as it is.
// q is the A operand from tensor memory (the softmax warps move each row there once, two bfloat16 to a
// column): the 16 KB it held in shared memory are a third slot of keys.
// Measured on 8,192 tokens of 32 heads (470 us, 585 TFLOP/s; the mma.sync kernel 1,122 us): without the MMAs
// and without the softmax arithmetic the launch still took 450 of 501 us, so what bounds a block is the
// chain of hand-overs per tile (loads, Q K^T, softmax, P V, each waiting for the one before), not a pipe;
// two blocks per SM give two such chains.  Keys and values in one ring cost 654 us, one block per SM with
// two score buffers 1,635 us; the third slot of keys brought 499 -> 467 us, keys issued a tile ahead of the
// values nothing more.  P in tensor memory as well, in the scores' place (256 columns hold no second place),
// gave 600 us: the next tile's Q K^T must then wait for P V.
// Every wait is bounded by wall time; a block that gives up sets a status word (snk_attention_tc_status).
#include "tcgen05.cuh"

#define AT_BQ 128
#define AT_BK 128
#define AT_HD 64
#ifndef AT_KSTAGES
#define AT_KSTAGES 3                                    // slots of keys
#endif
#ifndef AT_VSTAGES
#define AT_VSTAGES 2                                    // slots of values
#endif
#define AT_THREADS 192
#define AT_WAIT_NS 1000000000ull
#define AT_Q_BYTES (AT_BQ * AT_HD * 2)
#define AT_KV_BYTES (AT_BK * AT_HD * 2)                 // keys of a tile; values the same
#define AT_P_BYTES (AT_BQ * AT_BK * 2)                  // two panels of 64 keys
#define AT_TMEM_COLS 256
#define AT_TMEM_O 128                                   // S at column 0, O at 128
#define AT_TMEM_Q 192                                   // the rows of q, two bfloat16 to a column: 32 columns
#define AT_RESCALE_STEP 8.f                             // the reference maximum follows the row's maximum in steps of more than this

enum { AT_ERR_Q = 1, AT_ERR_KV = 2, AT_ERR_KV_FREE = 3, AT_ERR_S = 4, AT_ERR_S_FREE = 5, AT_ERR_P = 6, AT_ERR_PV = 7 };

__device__ int g_at_status;

struct __align__(16) AtShared {
  uint64_t q_full;
  uint64_t q_ready;                 // the softmax warps have moved q into tensor memory
  uint64_t k_full[AT_KSTAGES];      // the slot's pages of keys have landed
  uint64_t k_empty[AT_KSTAGES];     // Q K^T of the tile that used the slot has completed
  uint64_t v_full[AT_VSTAGES];      // the same for the values
  uint64_t v_empty[AT_VSTAGES];     // P V of the tile that used the slot has completed
  uint64_t s_full;                  // Q K^T of a tile has completed
  uint64_t s_empty;                 // the four softmax warps hold the scores in registers
  uint64_t p_full;                  // P is in shared memory, O is rescaled, stale value rows are zeroed
  uint64_t pv_done;                 // P V of a tile has completed
  uint32_t tmem_base;
  int aborted;
};

__device__ __forceinline__ void at_wait(uint64_t* bar, uint32_t parity, volatile int* aborted, int code) {
  // the clock is read once in 64 polls: reading it costs more than a poll, and a waiter that is busy
  // reading it sees the barrier late
  uint64_t start = 0;
  for (uint32_t polls = 1; !mbar_try_wait(bar, parity); ++polls) {
    if ((polls & 63) != 0) continue;
    if (*aborted) return;
    const uint64_t now = global_ns();
    if (start == 0) start = now;
    if (now - start > AT_WAIT_NS) {
      *aborted = 1;
      atomicCAS(&g_at_status, 0, code);
      return;
    }
  }
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 columns of this warp's 32 lanes; the caller waits (tcgen05.wait::ld) after the last of several
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// D += A B with A in tensor memory (lane = row, a column = two consecutive bfloat16 of the row) and B by descriptor.
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ uint32_t at_pack(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const int* __restrict__ block_table, int max_pages, int page_size,
                            const int* __restrict__ tiles, int n_tiles, bf16* __restrict__ out, int nh, int nkv,
                            int window, float scale_log2) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sm_k = smem;                                             // [AT_KSTAGES][128 keys][64], swizzled by TMA
  unsigned char* sm_v = sm_k + (size_t)AT_KSTAGES * AT_KV_BYTES;          // [AT_VSTAGES][128 keys][64]
  unsigned char* sm_p = sm_v + (size_t)AT_VSTAGES * AT_KV_BYTES;          // [2 panels][128 rows][64 keys]
  unsigned char* sm_q = sm_p;                                             // q lands in P's place and moves on to tensor memory
  AtShared* sh = reinterpret_cast<AtShared*>(sm_p + AT_P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_ready, 4);
    for (int i = 0; i < AT_KSTAGES; ++i) {
      mbar_init(&sh->k_full[i], 1);
      mbar_init(&sh->k_empty[i], 1);
    }
    for (int i = 0; i < AT_VSTAGES; ++i) {
      mbar_init(&sh->v_full[i], 1);
      mbar_init(&sh->v_empty[i], 1);
    }
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->s_empty, 4);
    mbar_init(&sh->p_full, 4);
    mbar_init(&sh->pv_done, 1);
    sh->aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh->tmem_base)), "r"((uint32_t)AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  volatile int* aborted = &sh->aborted;
  pdl_begin();                                           // q, the pages and the tiles are written by kernels before this one

  const int* tile = tiles + (size_t)(n_tiles - 1 - blockIdx.x) * 4;       // tiles with the most keys first
  const int seg = tile[0], row0 = tile[1], rows = tile[2], pos0 = tile[3];
  const int head = blockIdx.y;
  const int kvh = head / (nh / nkv);
  const int last_pos = pos0 + rows - 1;
  const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;          // the lowest key any row sees
  const int k_first = (key_lo / AT_BK) * AT_BK;
  const int n_kt = (last_pos - k_first) / AT_BK + 1;

  if (warp == 0) {
    const int* bt = block_table + (size_t)seg * max_pages;
    if (lane == 0) {
      mbar_expect_tx(&sh->q_full, AT_Q_BYTES);
      tma_load_2d(sm_q, &map_q, &sh->q_full, head * AT_HD, row0);
    }
    // keys and values have rings of their own: a slot of keys is free again when Q K^T of its tile has
    // completed, long before the tile's values are.  A tile has at most 16 pages: lane i looks up page i,
    // one tile ahead, so that the look-up (a trip to L2) is not part of the wait for a free slot.
    auto tile_pages = [&](int j, int& first_page, int& n_pages) {
      const int k0 = k_first + j * AT_BK;
      first_page = max(k0, key_lo) / page_size;
      n_pages = min(k0 + AT_BK - 1, last_pos) / page_size - first_page + 1;
    };
    // The keys run one tile ahead of the values (K[0], K[1], V[0], K[2], V[1], ...): a slot of values is
    // free late, and keys asked for behind that wait would be late too.
    int fp_k, np_k, fp_v = 0, np_v = 0;
    tile_pages(0, fp_k, np_k);
    int page_k = lane < np_k ? bt[fp_k + lane] : 0, page_v = 0, page_next = 0;
    for (int t = 0; t <= n_kt; ++t) {
      if (t + 1 < n_kt) {                                                 // the look-up for the keys of the next round
        int fp, np;
        tile_pages(t + 1, fp, np);
        page_next = lane < np ? bt[fp + lane] : 0;
      }
      if (t < n_kt) {
        const int ks = t % AT_KSTAGES;
        const int k0 = k_first + t * AT_BK;
        tile_pages(t, fp_k, np_k);
        at_wait(&sh->k_empty[ks], ((t / AT_KSTAGES) & 1) ^ 1, aborted, AT_ERR_KV_FREE);
        if (__any_sync(0xffffffffu, *aborted)) break;      // a wait ran out: nothing more is issued
        if (lane == 0) mbar_expect_tx(&sh->k_full[ks], (uint32_t)np_k * page_size * 128u);
        __syncwarp();
        if (lane < np_k)
          tma_load_2d(sm_k + (size_t)ks * AT_KV_BYTES + ((fp_k + lane) * page_size - k0) * 128, &map_kv,
                      &sh->k_full[ks], 0, ((page_k * 2) * nkv + kvh) * page_size);
      }
      if (t >= 1) {
        const int j = t - 1, vs = j % AT_VSTAGES;
        const int k0 = k_first + j * AT_BK;
        at_wait(&sh->v_empty[vs], ((j / AT_VSTAGES) & 1) ^ 1, aborted, AT_ERR_KV_FREE);
        if (__any_sync(0xffffffffu, *aborted)) break;
        if (lane == 0) mbar_expect_tx(&sh->v_full[vs], (uint32_t)np_v * page_size * 128u);
        __syncwarp();
        if (lane < np_v)
          tma_load_2d(sm_v + (size_t)vs * AT_KV_BYTES + ((fp_v + lane) * page_size - k0) * 128, &map_kv,
                      &sh->v_full[vs], 0, ((page_v * 2 + 1) * nkv + kvh) * page_size);
      }
      fp_v = fp_k; np_v = np_k; page_v = page_k;                          // this round's keys are the next round's values
      page_k = page_next;
      __syncwarp();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc_bf16(AT_BQ, AT_BK);
      const uint32_t idesc_o = instr_desc_bf16(AT_BQ, AT_HD) | (1u << 16);     // B (values) is MN-major
      at_wait(&sh->q_ready, 0, aborted, AT_ERR_Q);
      auto scores = [&](int j) {
        const int st = j % AT_KSTAGES;
        at_wait(&sh->k_full[st], (j / AT_KSTAGES) & 1, aborted, AT_ERR_KV);
        at_wait(&sh->s_empty, (j & 1) ^ 1, aborted, AT_ERR_S_FREE);
        if (*aborted) return;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sm_k + (size_t)st * AT_KV_BYTES);
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k)                 // 16 elements of q = 8 columns of tensor memory
          umma_bf16_ta(tmem, tmem + AT_TMEM_Q + k * 8, smem_desc_sw128(k_addr + k * 32), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(&sh->k_empty[st]);
        umma_commit(&sh->s_full);
      };
      scores(0);
      for (int j = 0; j < n_kt; ++j) {
        if (j + 1 < n_kt) scores(j + 1);
        const int st = j % AT_VSTAGES;
        at_wait(&sh->p_full, j & 1, aborted, AT_ERR_P);
        at_wait(&sh->v_full[st], (j / AT_VSTAGES) & 1, aborted, AT_ERR_KV);
        if (*aborted) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sm_p);
        const uint32_t v_addr = smem_u32(sm_v + (size_t)st * AT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < AT_BK / 16; ++kk)
          // P: panel kk / 4 (64 keys), 32 bytes per k-step inside it; V: 16 keys = 16 rows of 128 bytes further
          umma_bf16(tmem + AT_TMEM_O, smem_desc_sw128(p_addr + (kk >> 2) * (AT_BQ * 128) + (kk & 3) * 32),
                    smem_desc_sw128(v_addr + kk * 16 * 128), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh->v_empty[st]);
        umma_commit(&sh->pv_done);
      }
    }
  } else {
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;              // the tensor-memory lane = the row of the tile
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    const int pos = pos0 + row;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int lo_last = window > 0 ? max(0, last_pos - window + 1) : 0;   // the last row's lowest key
    {                                                    // this row of q: shared memory -> tensor memory
      at_wait(&sh->q_full, 0, aborted, AT_ERR_Q);
      uint32_t qr[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(sm_q + row * 128 + ((c ^ (row & 7)) << 4));
        qr[4 * c] = v.x; qr[4 * c + 1] = v.y; qr[4 * c + 2] = v.z; qr[4 * c + 3] = v.w;
      }
      tmem_st32(tmem + t_lane + AT_TMEM_Q, qr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_ready);
    }
    float m_ref = -INFINITY, l = 0.f;                    // the maximum the exponentials are taken against (scaled), the sum
    for (int j = 0; j < n_kt; ++j) {
      const int st = j % AT_VSTAGES;
      const int k0 = k_first + j * AT_BK;
      at_wait(&sh->s_full, j & 1, aborted, AT_ERR_S);
      if (__any_sync(0xffffffffu, *aborted)) break;        // the whole warp leaves together
      tc_fence_after();
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32_nowait(tmem + t_lane + (uint32_t)(c * 32), r[c]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->s_empty);
      // tiles that cross an edge: a key above the first row's position, or below the last row's window
      if (k0 + AT_BK - 1 > pos0 || k0 < lo_last) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kp = k0 + c * 32 + i;
            if (kp > pos || kp < lo) r[c][i] = 0xff800000u;      // -inf
          }
      }
      float mc[4];                                       // chains side by side (a maximum does not depend on the order)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float a0 = __uint_as_float(r[c][0]), a1 = __uint_as_float(r[c][1]);
        float a2 = __uint_as_float(r[c][2]), a3 = __uint_as_float(r[c][3]);
#pragma unroll
        for (int i = 4; i < 32; i += 4) {
          a0 = fmaxf(a0, __uint_as_float(r[c][i]));
          a1 = fmaxf(a1, __uint_as_float(r[c][i + 1]));
          a2 = fmaxf(a2, __uint_as_float(r[c][i + 2]));
          a3 = fmaxf(a3, __uint_as_float(r[c][i + 3]));
        }
        mc[c] = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
      }
      float mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
      mx *= scale_log2;                                  // the scale is positive
      float alpha = 1.f;
      if (mx > m_ref + AT_RESCALE_STEP || m_ref == -INFINITY) {
        const float m_new = mx == -INFINITY ? -INFINITY : ceilf(mx);       // a whole number: P's rounding does not
                                                                           // depend on the tile walk (csrc/attention_mma.cu)
        alpha = m_new == -INFINITY ? 1.f : at_exp2(m_ref - m_new);       // m_ref = -inf: nothing summed yet, 0
        m_ref = m_new;
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;              // a row that has seen no key yet
      float sc[4];                                       // per chunk two chains (even and odd pairs), then chunk sums 0+1, 2+3, both
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float e0 = 0.f, e1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          const float p0 = at_exp2(fmaf(__uint_as_float(r[c][2 * i]), scale_log2, neg_m));
          const float p1 = at_exp2(fmaf(__uint_as_float(r[c][2 * i + 1]), scale_log2, neg_m));
          const float p2 = at_exp2(fmaf(__uint_as_float(r[c][2 * i + 2]), scale_log2, neg_m));
          const float p3 = at_exp2(fmaf(__uint_as_float(r[c][2 * i + 3]), scale_log2, neg_m));
          e0 += p0 + p1;
          e1 += p2 + p3;
          r[c][i] = at_pack(p0, p1);                     // in place: entry i now holds keys 2i, 2i + 1 of the chunk
          r[c][i + 1] = at_pack(p2, p3);
        }
        sc[c] = e0 + e1;
      }
      l = l * alpha + ((sc[0] + sc[1]) + (sc[2] + sc[3]));
      if (j > 0) {                                       // P of the tile before has been read, O holds the tiles before this one
        at_wait(&sh->pv_done, (j - 1) & 1, aborted, AT_ERR_PV);
        tc_fence_after();
      }
      unsigned char* p_row = sm_p + row * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {                 // 8 keys = one 16-byte piece of the row
          const int piece = (c & 1) * 4 + q8;            // 16-byte piece of the 128-byte row of panel c / 2
          *reinterpret_cast<uint4*>(p_row + (c >> 1) * (AT_BQ * 128) + ((piece ^ (row & 7)) << 4)) =
              make_uint4(r[c][4 * q8], r[c][4 * q8 + 1], r[c][4 * q8 + 2], r[c][4 * q8 + 3]);
        }
      if (k0 < key_lo || k0 + AT_BK - 1 > last_pos) {    // value rows no row sees: zero, whatever they held
        at_wait(&sh->v_full[st], (j / AT_VSTAGES) & 1, aborted, AT_ERR_KV);
        const int kp = k0 + row;
        if (kp < key_lo || kp > last_pos) {
          uint4* v_row = reinterpret_cast<uint4*>(sm_v + (size_t)st * AT_KV_BYTES + row * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) v_row[i] = make_uint4(0, 0, 0, 0);
        }
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < AT_HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem + t_lane + (uint32_t)(AT_TMEM_O + c * 32), o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem + t_lane + (uint32_t)(AT_TMEM_O + c * 32), o);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // P and the zeroed rows, for the MMA's reads
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_full);
    }
    at_wait(&sh->pv_done, (n_kt - 1) & 1, aborted, AT_ERR_PV);
    tc_fence_after();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    bf16* dst = out + ((size_t)(row0 + row) * nh + head) * AT_HD;
#pragma unroll
    for (int c = 0; c < AT_HD / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tmem + t_lane + (uint32_t)(AT_TMEM_O + c * 32), o);
      if (row < rows && !*aborted) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(
              at_pack(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
              at_pack(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
              at_pack(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
              at_pack(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
      }
    }
  }
  if (*aborted) drain_after_abort();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)AT_TMEM_COLS)
                 : "memory");
  }
}

static bool at_page_ok(int page_size) {
  return page_size >= 8 && page_size <= AT_BK && page_size % 8 == 0 && AT_BK % page_size == 0;
}

// q [M, nh, 64], out [M, nh * 64] bfloat16; tiles int32 [n, 4] = (segment, first row, rows <= 128, position of
// the first row); num_pages: pages in the pool [pages, 2, nkv, page_size, 64].  Sizes it does not take give
// SNK_ERR_SIZE (the caller then uses the mma.sync kernels).
SNK_API int snk_attention_prefill_tc(const void* q, long long M, const void* pool, long long num_pages,
                                     const int* block_table, int max_pages, int page_size, const int* tiles,
                                     int n_tiles, void* out, int nh, int nkv, int hd, int window, float scale,
                                     cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh > 65535 || M <= 0) return SNK_ERR_SIZE;
  if (hd != AT_HD || !at_page_ok(page_size) || num_pages <= 0) return SNK_ERR_SIZE;
  if (num_pages * 2 * nkv * page_size >= (1ll << 31)) return SNK_ERR_SIZE;
  if (((uintptr_t)q % 16) || ((uintptr_t)pool % 16) || ((uintptr_t)out % 16)) return SNK_ERR_ALIGN;
  CUtensorMap map_q, map_kv;
  int rc = tensor_map(q, M, (long long)nh * hd, AT_BQ, 64, &map_q);
  if (rc) return rc;
  rc = tensor_map(pool, num_pages * 2 * nkv * page_size, hd, page_size, 64, &map_kv);
  if (rc) return rc;
  const size_t smem = (size_t)(AT_KSTAGES + AT_VSTAGES) * AT_KV_BYTES + AT_P_BYTES + sizeof(AtShared);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  snk_launch(attention_prefill_tc_kernel, dim3(n_tiles, nh), dim3(AT_THREADS), smem, stream, map_q, map_kv,
             block_table, max_pages, page_size, tiles, n_tiles, static_cast<bf16*>(out), nh, nkv, window,
             scale * 1.4426950408889634f);
  SNK_LAUNCH_CHECK();
  return 0;
}

// Queue a copy of the status word into ``host`` (pinned host memory, one int) on ``stream`` without waiting
// for it and without clearing it: a caller that synchronises with the stream anyway (an event, a read-back)
// learns of a wait that ran out at no cost.  Not for use inside a stream capture.
SNK_API int snk_attention_tc_status_peek(int* host, void* stream) {
  return (int)cudaMemcpyFromSymbolAsync(host, g_at_status, sizeof(int), 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

// 0, or the code of the first wait that ran out in a block of an earlier launch; reading clears it.  Synchronises.
SNK_API int snk_attention_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_at_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_at_status, &zero, sizeof(int));
  return v;
}
