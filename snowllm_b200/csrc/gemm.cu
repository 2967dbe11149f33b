// C[M,N] = A[M,K] . W[N,K]^T on the CUDA cores, with float accumulation in k order.
//
// This is the matrix product of the true 32-bit path (plain FFMA: no TF32, no split
// tricks), and the reference kernel that the tensor-core products are checked against.
// Each output element is one thread's sum over k = 0..K-1 in ascending order, so a row's
// result does not depend on how many other rows the launch holds.
//
// Grouped form (routed experts): rows are sorted by group; group e owns rows
// [offsets[e], offsets[e+1]) and multiplies them with W + e*N*K.  `a_rows` gathers A: the
// A row of output row r is a_rows[r] / a_div (a_rows == nullptr: row r itself).
// (the role of snowllm/ops/gemm.py:33-41 and of the expert products in
// snowllm/ops/inference.py:60-76)
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
};

template <typename T>
__device__ __forceinline__ void load4(const T* row, int k, int K, bool row_ok, bool vec, float (&v)[4]) {
  if (!row_ok) { v[0] = v[1] = v[2] = v[3] = 0.f; return; }
  if (vec && k + 3 < K) { Vec4<T>::load(row + k, v); return; }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (k + i < K) ? to_f<T>(row[k + i]) : 0.f;
}

template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, OutT* __restrict__ C, int M,
                 int N, int K, const int* __restrict__ a_rows, int a_div,
                 const int* __restrict__ offsets, int vec) {
  pdl_begin();
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Ws[BK][BN + 4];
  int row_begin = 0, row_end = M;
  const T* Wg = W;
  if (offsets) {
    row_begin = offsets[blockIdx.z];
    row_end = offsets[blockIdx.z + 1];
    Wg = W + (size_t)blockIdx.z * N * K;
  }
  const int m0 = row_begin + blockIdx.y * BM;
  if (m0 >= row_end) return;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int lr = tid >> 2, lk = (tid & 3) * 4;       // tile-load coordinates
  const int ty = tid >> 4, tx = tid & 15;            // 4x4 outputs at (ty*4, tx*4)

  const int arow = m0 + lr;
  const bool a_ok = arow < row_end;
  const T* a_ptr = nullptr;
  if (a_ok) a_ptr = A + (size_t)(a_rows ? a_rows[arow] / a_div : arow) * K;
  const int wrow = n0 + lr;
  const bool w_ok = wrow < N;
  const T* w_ptr = w_ok ? Wg + (size_t)wrow * K : nullptr;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float av[4], wv[4];
    load4<T>(a_ptr, k0 + lk, K, a_ok, vec, av);
    load4<T>(w_ptr, k0 + lk, K, w_ok, vec, wv);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lr] = av[i];
      Ws[lk + i][lr] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cidx = n0 + tx * 4 + j;
      if (cidx < N) C[(size_t)r * N + cidx] = from_f<OutT>(acc[i][j]);
    }
  }
}

// out_f32: C is float whatever the compute dtype.  groups <= 1 and offsets == nullptr: plain
// product.  max_rows_per_group bounds the rows any one group can own (for the grid).
SNK_API int snk_gemm_simt(const void* A, const void* W, void* C, int M, int N, int K,
                          const int* a_rows, int a_div, const int* offsets, int groups,
                          int max_rows_per_group, int out_f32, int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return SNK_ERR_SIZE;
  const int rows = offsets ? max_rows_per_group : M;
  if (rows <= 0) return 0;
  dim3 grid((N + BN - 1) / BN, (rows + BM - 1) / BM, offsets ? groups : 1);
  if (grid.y > 65535u || grid.z > 65535u) return SNK_ERR_SIZE;
  const size_t esz = dtype == SNK_F32 ? 4 : 2;
  const int vec = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0) &&
                  (((size_t)K * esz) % 8 == 0);
  if (a_div <= 0) a_div = 1;
  SNK_DISPATCH(dtype, {
    if (out_f32 || dtype == SNK_F32)
      snk_launch(gemm_simt_kernel<T, float>, dim3(grid), dim3(256), 0, stream, 
          static_cast<const T*>(A), static_cast<const T*>(W), static_cast<float*>(C), M, N, K,
          a_rows, a_div, offsets, vec);
    else
      snk_launch(gemm_simt_kernel<T, T>, dim3(grid), dim3(256), 0, stream, 
          static_cast<const T*>(A), static_cast<const T*>(W), static_cast<T*>(C), M, N, K, a_rows,
          a_div, offsets, vec);
  });
  SNK_LAUNCH_CHECK();
  return 0;
}
