// tcgen05 (5th-generation tensor cores): operand descriptors, MMA issue, commit, tensor-memory loads and
// fences, for one SM (cta_group::1) and for a pair of SMs (cta_group::2).
#pragma once
#include "tma.cuh"

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, written by TMA with the
// 128-byte swizzle: 8-row groups lie 1024 bytes apart (stride byte offset); the leading byte offset is
// not used by swizzled K-major layouts; descriptor version 1; layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);          // start address, bits [0, 14)
  d |= (uint64_t)1 << 16;                               // leading byte offset (unused), bits [16, 30)
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset, bits [32, 46)
  d |= (uint64_t)1 << 46;                               // version, bits [46, 48)
  d |= (uint64_t)2 << 61;                               // layout type, bits [61, 64)
  return d;
}

// Instruction descriptor of kind::f16: D float, A and B bfloat16, both K-major, M m (128; 256 for a pair of
// SMs), N n.
__device__ __forceinline__ uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


// ---------------------------------------------------------------------------------------------
// The store of a 32 x 32 piece of an accumulator that tcgen05.ld left with one ROW per lane (r[0..31]: the
// row's 32 columns).  Stored straight from there, a warp's instruction would touch 32 rows, 16 bytes each.
// So the piece goes through shared memory (rows 144 bytes apart: 16-byte stores and loads without bank
// conflicts) and comes back with 8 lanes side by side along a row: every store instruction then writes whole
// 128-byte (float) or 64-byte (bfloat16) runs of 4 rows.  (With SwiGLU a lane's row shrinks to 32 bytes, which two
// 16-byte stores from the registers write faster.)
//   first_row: row of C of lane 0; rows >= row_end are not stored; col0: first column of the piece (a multiple
//   of 32); N: columns of the product (SwiGLU: C has N / 2).  Pieces that reach past N take the slow path.
#define TC_STAGE_PITCH 36                 // floats between rows of the staging tile
#define TC_STAGE_FLOATS (32 * TC_STAGE_PITCH)

template <typename OutT, bool SWIGLU>
__device__ __forceinline__ void tc_store_piece(const uint32_t (&r)[32], float* stage, int lane, OutT* __restrict__ C,
                                               int first_row, int row_end, int col0, int N) {
  if constexpr (SWIGLU) {
    // columns: 8 gates, their 8 ups, 8 gates, their 8 ups -> 16 outputs of this lane's row, two 16-byte stores
    // (measured: faster from the registers than through the staging tile, 106 against 123 us on 2048 x 14336 x 2048)
    const int row = first_row + lane;
    if (row >= row_end) return;
    OutT* dst = C + (size_t)row * (N / 2) + col0 / 2;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      if (col0 + blk * 16 + 16 <= N) {
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float g0 = __uint_as_float(r[blk * 16 + 2 * j]), g1 = __uint_as_float(r[blk * 16 + 2 * j + 1]);
          const float u0 = __uint_as_float(r[blk * 16 + 8 + 2 * j]), u1 = __uint_as_float(r[blk * 16 + 9 + 2 * j]);
          const __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * u0, g1 / (1.f + expf(-g1)) * u1);
          p[j] = *reinterpret_cast<const uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(dst + blk * 8) = make_uint4(p[0], p[1], p[2], p[3]);
      }
    }
    return;
  } else {
    if (col0 + 32 <= N && (N % 8) == 0) {
      uint4* mine = reinterpret_cast<uint4*>(stage + lane * TC_STAGE_PITCH);
#pragma unroll
      for (int c = 0; c < 8; ++c) mine[c] = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), row = first_row + rr;
        const float4 v = *reinterpret_cast<const float4*>(stage + rr * TC_STAGE_PITCH + (lane & 7) * 4);
        if (row < row_end) store4<OutT>(C + (size_t)row * N + col0 + (lane & 7) * 4, v.x, v.y, v.z, v.w);
      }
      __syncwarp();
      return;
    }
    // a piece at the right edge, or a width the vector stores do not take: this lane's row, element by element
    const int row = first_row + lane;
    if (row >= row_end) return;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < N) C[(size_t)row * N + col0 + i] = from_f<OutT>(__uint_as_float(r[i]));
  }
}

// ---- a pair of SMs (cta_group::2): the leader block issues; operands lie at the same shared-memory
// offsets in both blocks (each block its 128 rows of A and its half of B's rows), the accumulator rows
// 0..127 in the leader's tensor memory and 128..255 in the peer's, at the same columns.
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives once on the barrier at this shared-memory offset in every block of `cta_mask` when the MMAs issued so
// far have completed.
__device__ __forceinline__ void umma2_commit(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}
// A tile load whose bytes count towards a barrier that may lie in the peer block of the pair (`cluster_bar`: the
// barrier's shared::cluster address, from cluster_addr); not a multicast: the data goes to this block only.
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
// The shared::cluster address of the variable at this shared-memory offset in block `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}
// One arrival on the barrier at the same offset in block `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(const uint32_t* local, uint32_t rank) {
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ void st_cluster_u32(const void* local, uint32_t rank, uint32_t v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
