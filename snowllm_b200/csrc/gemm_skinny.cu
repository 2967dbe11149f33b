// C[M,N] = A[M,K] . W[N,K]^T in bfloat16 for few rows (decode: M up to 64), bound by the read of W.
//
// Weights stream from HBM exactly once, straight into tensor-core fragments; nothing of W passes
// through shared memory.  A block owns 16 rows of W (16 output features).  Its 8 warps split K in
// interleaved 32-element blocks; a warp multiplies its 16x32 piece of W with up to 64 tokens by
// mma.sync m16n8k16 (W as the 16-row operand, 8 tokens as the 8-column operand) and the 8 partial
// sums meet in shared memory, added in warp order: no atomics, the same bits every run, and a
// token's result does not depend on which other tokens the launch holds.
//
// Fragment trick: lane (g, t) loads 16 contiguous bytes (8 k-values at k0 + 8t) of W rows g and
// g + 8 and of token row g.  The first four values feed one MMA, the last four a second one; the
// two MMAs see a permutation of the 32 k-values, the same one for both operands, which a dot
// product does not mind.  So every global load is a full 16-byte vector and no shuffle is needed.
//
// Few output features (N/16 blocks would leave SMs idle): a thread-block cluster of S blocks along z
// shares one 16-row strip of W and splits K S ways more; the S partial sums meet in the first block
// through distributed shared memory, added in rank order.  S depends on N and K alone.
//
// Grouped form (routed experts): rows are sorted by group; group e owns rows
// [offsets[e], offsets[e+1]) and uses W + e*N*K; a_rows gathers A (row r reads A[a_rows[r] / a_div]).
// A group with more than 64 rows is walked in passes of 64 (W is then re-read from L2).
// (the role of snowllm/ops/gemm.py:33-41 and the expert products of snowllm/ops/inference.py:60-76
// at decode shapes)
#include "common.cuh"

#ifndef SK_WARPS
#define SK_WARPS 8
#endif
#define SK_ROWS 16
#define SK_KBLOCK 32
#ifndef SK_UNROLL
#define SK_UNROLL 4
#endif
#ifndef SK_PREFETCH_LINES
#define SK_PREFETCH_LINES 4    // rounds of 16 lines of 128 bytes per row that a block asks L2 for ahead of its wait
                               // (measured in the decode step, 0 / 2 / 4 rounds: 1.497 / 1.482 / 1.476 ms at batch 1)
#endif

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// SWIGLU: W holds gate and up rows interleaved in blocks of 8 (rows 16j..16j+7: gate of features
// 8j..8j+7, rows 16j+8..16j+15: their up rows), so a block's 16 rows are 8 features' gate and up; the
// store is then silu(gate) * up into C[M, N/2].
template <int MT, typename OutT, bool SWIGLU>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, OutT* __restrict__ C, int M,
                   int N, int K, const int* __restrict__ a_rows, int a_div,
                   const int* __restrict__ offsets) {
#if SK_PREFETCH_LINES > 0
  if (offsets == nullptr) {
    // A plain product's W is a constant and this block's 16 rows of it are known from the block's number
    // alone: while the kernel before this one ends, ask L2 for the first lines of each row (128 bytes a
    // thread and round; no register is held, nothing is read into the SM).  A grouped product does not
    // know before the wait which groups own rows.
    const int row = min((int)(blockIdx.x * SK_ROWS + (threadIdx.x >> 4)), N - 1);
    const char* base = reinterpret_cast<const char*>(W + (size_t)row * K);
    const int row_bytes = K * 2;
    const int first = blockIdx.z * (row_bytes / (int)gridDim.z) & ~127;      // a cluster's blocks split K
#pragma unroll
    for (int i = 0; i < SK_PREFETCH_LINES; ++i) {
      const int off = first + ((threadIdx.x & 15) + 16 * i) * 128;
      if (off < row_bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
    }
  }
#endif
  pdl_begin();
  __shared__ float red[SK_WARPS][MT * 8][SK_ROWS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * SK_ROWS;
  int row_begin = 0, row_end = M;
  const bf16* Wg = W;
  if (offsets) {
    row_begin = offsets[blockIdx.y];
    row_end = offsets[blockIdx.y + 1];
    Wg = W + (size_t)blockIdx.y * N * K;
  }
  if (row_begin >= row_end) return;
  // the two W rows of this lane (rows past N read row N-1 and are dropped at the store)
  const bf16* w_lo = Wg + (size_t)min(n0 + g, N - 1) * K + 8 * t;
  const bf16* w_hi = Wg + (size_t)min(n0 + g + 8, N - 1) * K + 8 * t;
  const int kblocks = (K + SK_KBLOCK - 1) / SK_KBLOCK;
  const int split = gridDim.z, rank = blockIdx.z;         // the cluster spans z: S blocks split K further
  const int vwarp = rank * SK_WARPS + warp, vwarps = split * SK_WARPS;

  for (int m0 = row_begin; m0 < row_end; m0 += MT * 8) {
    const bf16* a_ptr[MT];
    bool a_ok[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int r = m0 + i * 8 + g;
      a_ok[i] = r < row_end;
      const int src = a_ok[i] ? (a_rows ? a_rows[r] / a_div : r) : 0;
      a_ptr[i] = A + (size_t)src * K + 8 * t;
    }
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int kb0 = vwarp; kb0 < kblocks; kb0 += vwarps * SK_UNROLL) {
      uint4 wl[SK_UNROLL], wh[SK_UNROLL];
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        const int kb = kb0 + u * vwarps;
        const int k = kb * SK_KBLOCK + 8 * t;
        if (kb < kblocks && k < K) {              // K is a multiple of 8: a lane's 8 values are all in or all out
          wl[u] = ldg_stream(w_lo + (size_t)kb * SK_KBLOCK);
          wh[u] = ldg_stream(w_hi + (size_t)kb * SK_KBLOCK);
        } else {
          wl[u] = make_uint4(0, 0, 0, 0);
          wh[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        const int kb = kb0 + u * vwarps;
        const int k = kb * SK_KBLOCK + 8 * t;
        const bool k_ok = kb < kblocks && k < K;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          uint4 x = make_uint4(0, 0, 0, 0);
          if (k_ok && a_ok[i]) x = *reinterpret_cast<const uint4*>(a_ptr[i] + (size_t)kb * SK_KBLOCK);
          mma_bf16(acc[i], wl[u].x, wh[u].x, wl[u].y, wh[u].y, x.x, x.y);
          mma_bf16(acc[i], wl[u].z, wh[u].z, wl[u].w, wh[u].w, x.z, x.w);
        }
      }
    }
    // acc[i] = {(row g, token 2t), (row g, token 2t+1), (row g+8, token 2t), (row g+8, token 2t+1)}
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      red[warp][i * 8 + 2 * t][g] = acc[i][0];
      red[warp][i * 8 + 2 * t + 1][g] = acc[i][1];
      red[warp][i * 8 + 2 * t][g + 8] = acc[i][2];
      red[warp][i * 8 + 2 * t + 1][g + 8] = acc[i][3];
    }
    __syncthreads();
    if (split > 1) {
      // this block's sum over its warps goes to red[0]; the first block then adds the blocks' sums in rank order
      for (int idx = threadIdx.x; idx < MT * 8 * SK_ROWS; idx += SK_WARPS * 32) {
        const int tok = idx / SK_ROWS, r = idx % SK_ROWS;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += red[w][tok][r];
        red[0][tok][r] = sum;                               // read and written by this thread alone
      }
      cluster_sync();
      if (rank == 0) {
        for (int idx = threadIdx.x; idx < MT * 8 * SK_ROWS; idx += SK_WARPS * 32) {
          const int tok = idx / SK_ROWS, r = idx % SK_ROWS;
          float sum = red[0][tok][r];
          for (int q = 1; q < split; ++q) sum += ld_cluster_f32(&red[0][tok][r], q);
          red[1][tok][r] = sum;
        }
        __syncthreads();
        if constexpr (SWIGLU) {
          for (int idx = threadIdx.x; idx < MT * 8 * (SK_ROWS / 2); idx += SK_WARPS * 32) {
            const int tok = idx / (SK_ROWS / 2), r = idx % (SK_ROWS / 2);
            const int m = m0 + tok, n = n0 + r;
            if (m < row_end && n + 8 < N) {
              const float gate = red[1][tok][r], up = red[1][tok][r + 8];
              C[(size_t)m * (N / 2) + n0 / 2 + r] = from_f<OutT>(gate / (1.f + expf(-gate)) * up);
            }
          }
        } else {
          for (int idx = threadIdx.x; idx < MT * 8 * SK_ROWS; idx += SK_WARPS * 32) {
            const int tok = idx / SK_ROWS, r = idx % SK_ROWS;
            const int m = m0 + tok, n = n0 + r;
            if (m < row_end && n < N) C[(size_t)m * N + n] = from_f<OutT>(red[1][tok][r]);
          }
        }
      }
      cluster_sync();                                       // the others' shared memory lives until it has been read
      continue;
    }
    if constexpr (SWIGLU) {
      for (int idx = threadIdx.x; idx < MT * 8 * (SK_ROWS / 2); idx += SK_WARPS * 32) {
        const int tok = idx / (SK_ROWS / 2), r = idx % (SK_ROWS / 2);
        const int m = m0 + tok, n = n0 + r;
        if (m < row_end && n + 8 < N) {
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < SK_WARPS; ++w) {
            gate += red[w][tok][r];
            up += red[w][tok][r + 8];
          }
          C[(size_t)m * (N / 2) + n0 / 2 + r] = from_f<OutT>(gate / (1.f + expf(-gate)) * up);
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < MT * 8 * SK_ROWS; idx += SK_WARPS * 32) {
        const int tok = idx / SK_ROWS, r = idx % SK_ROWS;
        const int m = m0 + tok, n = n0 + r;
        if (m < row_end && n < N) {
          float s = 0.f;
#pragma unroll
          for (int w = 0; w < SK_WARPS; ++w) s += red[w][tok][r];
          C[(size_t)m * N + n] = from_f<OutT>(s);
        }
      }
    }
  }
}

template <int MT>
static int launch_skinny(const void* A, const void* W, void* C, int M, int N, int K, const int* a_rows,
                         int a_div, const int* offsets, int groups, int out_f32, int swiglu, int split,
                         cudaStream_t stream) {
  dim3 grid((N + SK_ROWS - 1) / SK_ROWS, offsets ? groups : 1, split);
  const dim3 block(SK_WARPS * 32);
  const bf16 *a = static_cast<const bf16*>(A), *w = static_cast<const bf16*>(W);
  if (swiglu)
    snk_launch_cluster(gemm_skinny_kernel<MT, bf16, true>, grid, block, 0, stream, split, a, w,
                       static_cast<bf16*>(C), M, N, K, a_rows, a_div, offsets);
  else if (out_f32)
    snk_launch_cluster(gemm_skinny_kernel<MT, float, false>, grid, block, 0, stream, split, a, w,
                       static_cast<float*>(C), M, N, K, a_rows, a_div, offsets);
  else
    snk_launch_cluster(gemm_skinny_kernel<MT, bf16, false>, grid, block, 0, stream, split, a, w,
                       static_cast<bf16*>(C), M, N, K, a_rows, a_div, offsets);
  SNK_LAUNCH_CHECK();
  return 0;
}

// How many blocks share one strip of W (a cluster along z).  A plain product with fewer strips than
// the GPU has SMs is split 4 ways, as long as every warp of the cluster keeps two k-blocks of its own.
// Measured in a replayed chain of launches at 8 rows: 2048 x 2048 6.8 -> 5.1 us, 2048 x 7168 20.6 -> 9.2 us;
// with 384 strips (6144 x 2048) any split lost (8.1 -> 11.0 us), and so did 8 ways everywhere.
// Depends on N and K alone, so a row's sum has the same order whatever else the launch holds.
#define SK_SPLIT 4
#define SK_SPLIT_MAX_STRIPS 148
static int skinny_split(int N, int K, const int* offsets) {
  static int off = -1;                                     // SNOWLLM_B200_SKINNY_SPLIT=0 in the environment: never split
  if (off < 0) {
    const char* e = getenv("SNOWLLM_B200_SKINNY_SPLIT");
    off = (e && e[0] == '0') ? 1 : 0;
  }
  if (offsets || off) return 1;                            // grouped: the groups already multiply the blocks
  const int strips = (N + SK_ROWS - 1) / SK_ROWS, kblocks = (K + SK_KBLOCK - 1) / SK_KBLOCK;
  return (strips <= SK_SPLIT_MAX_STRIPS && kblocks >= 2 * SK_SPLIT * SK_WARPS) ? SK_SPLIT : 1;
}

// rows_hint: the most rows one group (or the whole product) is expected to hold; picks how many
// 8-token tiles a pass covers.  More rows than that still give the right result, in more passes.
// swiglu: W is gate/up interleaved in blocks of 8 rows and C is [M, N/2] bfloat16 = silu(gate) * up.
SNK_API int snk_gemm_skinny(const void* A, const void* W, void* C, int M, int N, int K, const int* a_rows,
                            int a_div, const int* offsets, int groups, int rows_hint, int out_f32, int swiglu,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) return SNK_ERR_SIZE;
  if (swiglu && (N % 16 || out_f32)) return SNK_ERR_SIZE;
  if (((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return SNK_ERR_ALIGN;
  if (groups > 65535) return SNK_ERR_SIZE;
  if (a_div <= 0) a_div = 1;
  const int split = skinny_split(N, K, offsets);
  if (rows_hint <= 8) return launch_skinny<1>(A, W, C, M, N, K, a_rows, a_div, offsets, groups, out_f32, swiglu, split, stream);
  if (rows_hint <= 16) return launch_skinny<2>(A, W, C, M, N, K, a_rows, a_div, offsets, groups, out_f32, swiglu, split, stream);
  if (rows_hint <= 32) return launch_skinny<4>(A, W, C, M, N, K, a_rows, a_div, offsets, groups, out_f32, swiglu, split, stream);
  return launch_skinny<8>(A, W, C, M, N, K, a_rows, a_div, offsets, groups, out_f32, swiglu, split, stream);
}
