// Shared helpers of the sm_100a kernels: dtype traits, reductions, launch checks.
//
// Every entry point is a plain C function (`snk_*`) that takes device pointers, sizes
// and a stream, launches on that stream and returns 0 or an error code; it never
// allocates and never synchronises.  Activations come in the engine's compute dtype
// (float or bfloat16, `dtype` argument); statistics, accumulators and the residual
// stream are always float.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define SNK_API extern "C" __attribute__((visibility("default")))

enum { SNK_F32 = 0, SNK_BF16 = 1 };

// Error codes above any cudaError_t value.
enum {
  SNK_ERR_DTYPE = 20001,      // dtype code not known
  SNK_ERR_SIZE = 20002,       // a size this kernel refuses
  SNK_ERR_ALIGN = 20003,      // a pointer or a row pitch that is not aligned as required
};

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// The value after a round trip through T: the identity for float, round-to-nearest-even
// for bfloat16.  Marks the places where the 16-bit path rounds an intermediate.
template <typename T> __device__ __forceinline__ float round_f(float v) { return to_f<T>(from_f<T>(v)); }

// A small vector (norm weight, conv taps, router matrix) that stays float when the file
// stores it so, whatever the compute dtype.
struct SmallVec {
  const void* p;
  int is_f32;
  __device__ __forceinline__ float operator[](size_t i) const {
    return is_f32 ? static_cast<const float*>(p)[i]
                  : __bfloat162float(static_cast<const bf16*>(p)[i]);
  }
};

// Four consecutive outputs in the compute dtype, by one store (16-byte aligned for float, 8 for bfloat16).
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo),
                                            *reinterpret_cast<const uint32_t*>(&hi));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` is 33 floats
// of shared memory.  The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Thread-block clusters: a barrier over all threads of the cluster's blocks, and the shared memory of
// another block of the cluster (distributed shared memory) by the address the same variable has here.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The float at the same shared-memory address in block `rank` of this cluster.
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Programmatic dependent launch.  pdl_wait() holds a kernel until the kernels before it have completed
// and their writes are visible; before it a kernel touches no memory.  pdl_trigger() lets the next
// kernel of the stream be scheduled while this one still runs, so that its launch latency hides behind
// this kernel's tail.  The trigger always comes after the wait: a kernel that triggered first would let
// the one after it trigger too, and a whole chain of waiting kernels would take the SMs from the one
// that runs (measured on the decode step: 4.6 ms against 3.1 ms without any of this).  Small kernels
// trigger right after their wait (pdl_begin); kernels of several waves trigger when a block's loads
// are done, or not at all (the next kernel then starts when the last block ends).  A kernel launched
// without the attribute passes both instructions without effect.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_begin() {
  pdl_wait();
  pdl_trigger();
}

// Launch with the programmatic-serialization attribute (off with SNOWLLM_B200_PDL=0 in the environment, or
// at run time through snk_pdl_set, which every library exports: a measurement that wants each kernel's own
// duration switches it off, since a kernel launched early spends the wait inside its measured time).
inline int& snk_pdl_flag() {
  static int on = -1;
  return on;
}
inline int snk_pdl_enabled() {
  int& on = snk_pdl_flag();
  if (on < 0) {
    const char* e = getenv("SNOWLLM_B200_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}
SNK_API void snk_pdl_set(int on) { snk_pdl_flag() = on ? 1 : 0; }

// Thread-block clusters of cluster.x x cluster.y x cluster.z blocks (each grid dimension a multiple of the
// cluster's); all ones: no clusters.
template <typename... KArgs, typename... Args>
inline cudaError_t snk_launch_cluster3(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = snk_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster.x;
    attr[1].val.clusterDim.y = cluster.y;
    attr[1].val.clusterDim.z = cluster.z;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// cluster_z > 1: clusters of that many blocks along z.
template <typename... KArgs, typename... Args>
inline cudaError_t snk_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, int cluster_z, Args&&... args) {
  return snk_launch_cluster3(kernel, grid, block, smem, stream, dim3(1, 1, (unsigned)(cluster_z > 1 ? cluster_z : 1)),
                             static_cast<Args&&>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t snk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  return snk_launch_cluster(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

#define SNK_LAUNCH_CHECK()                       \
  do {                                           \
    cudaError_t e_ = cudaGetLastError();         \
    if (e_ != cudaSuccess) return (int)e_;       \
  } while (0)

#define SNK_DISPATCH(dtype, ...)                                  \
  do {                                                            \
    if ((dtype) == SNK_F32) { typedef float T; __VA_ARGS__; }     \
    else if ((dtype) == SNK_BF16) { typedef bf16 T; __VA_ARGS__; }\
    else return SNK_ERR_DTYPE;                                    \
  } while (0)
