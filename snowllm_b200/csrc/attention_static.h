// Paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in SnowLLM/SnowLLM: it is an addition of this engine.
//
// Who needs it: code that runs where a call to cudaMalloc (or to any allocator that may fall through
// to it, torch's caching allocator included) is not allowed or not wanted: a plugin inside a host
// application that owns all device memory, a real-time loop that must not hit an allocation stall, a
// process that is already at its memory limit, or a C program that links this library without a
// tensor framework at all.  The regular entry point, snk_paged_attention, needs scratch memory from
// its caller whenever a row's keys are split into more than one chunk; this one brings its own.
//
// How: the scratch is a fixed array in the library's device image, SNK_ATTENTION_STATIC_SCRATCH_BYTES
// long.  Every GPU that loads the library holds those bytes until the process exits, so the limit is
// kept modest.  A call whose partial results would not fit is refused with
// SNK_ERR_STATIC_SCRATCH before anything is launched; nothing is ever allocated or freed.
//
// What to know before calling:
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and keeps it.  Make that first call outside of any stream capture.
//   * All calls share the one array and it keeps whatever the last call left in it.  The kernels
//     write every partial result they later read, so nothing has to be cleared between calls; but two
//     calls that overlap on the GPU (different streams, no ordering between them) race on it.  Order
//     them on one stream, or with events.
//   * Inputs, outputs and their meaning are those of snk_paged_attention; only `scratch` is gone.
#pragma once
#include <cuda_runtime.h>

#define SNK_ATTENTION_STATIC_SCRATCH_BYTES (8u << 20)   /* 8 MiB */
#define SNK_ERR_STATIC_SCRATCH 20010                    /* the call needs more scratch than the array holds */
#define SNK_ERR_STATIC_SETUP 20011                      /* the array's device address could not be found */

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of the static array that a call with these sizes would use (0 when num_chunks <= 1). */
long long snk_paged_attention_static_need(int M, int nh, int hd, int num_chunks);

/* Same computation and same result as snk_paged_attention, with the library's own scratch.
   Returns 0, a cudaError_t value, or one of the SNK_ERR_* codes. */
int snk_paged_attention_static(const void* q, const void* pool, const int* block_table, int max_pages,
                               int page_size, const int* positions, const int* row_seg, void* out, int M,
                               int nh, int nkv, int hd, int window, int chunk, int num_chunks, float scale,
                               int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
