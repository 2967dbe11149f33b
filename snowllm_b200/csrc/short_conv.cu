// Gated short convolution over a flat batch of segments, and its per-request history.
//
//   bcx row = [B | C | x] (thirds);  g = round(B * x)
//   conv[t,c] = sum_{j<L} w[c,j] * g~[t-(L-1)+j, c], float accumulation in tap order, where g~
//   is the request's history (the last L-1 rows of g of earlier steps; zeros for a request
//   that starts at position 0, whatever its slot holds) followed by this step's g
//   y = round(C * conv);   state <- the last L-1 rows of g~ (oldest first)
//   (snowllm/models/lfm2/layers.py:26-33; snowllm/ops/lfm2.py:8-26; tests/test_lfm2.py:41-49)
//
// Two launches: the first only reads the state, the second rewrites it, so that tokens of
// one segment may be spread over many blocks.  Each value depends on its own segment only,
// and the taps are summed in one fixed order, so a sequence gives the same bits however it
// is cut into steps.
#include "common.cuh"

#define CONV_MAX_L 16
#define CONV_ROWS_PER_BLOCK 1

template <typename T>
__device__ __forceinline__ float gated(const T* __restrict__ bcx, size_t row, int H, int c) {
  const T* r = bcx + row * 3 * (size_t)H;
  return round_f<T>(to_f<T>(r[c]) * to_f<T>(r[2 * H + c]));
}

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ bcx, SmallVec w, const T* __restrict__ state,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ seg_start,
                                  const int* __restrict__ seg_slot, const int* __restrict__ row_seg,
                                  T* __restrict__ out, int M, int H, int L) {
  pdl_begin();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float taps[CONV_MAX_L];
#pragma unroll
  for (int j = 0; j < CONV_MAX_L; ++j) taps[j] = j < L ? w[(size_t)c * L + j] : 0.f;
  const int row0 = blockIdx.y * CONV_ROWS_PER_BLOCK;
  for (int m = row0; m < min(M, row0 + CONV_ROWS_PER_BLOCK); ++m) {
    const int seg = row_seg[m];
    const int first = cu_seqlens[seg];
    const int t = m - first;                         // index within this step's segment
    const bool has_state = seg_start[seg] > 0;
    const T* st = state + (size_t)seg_slot[seg] * (L - 1) * H;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_L; ++j) {
      if (j < L) {
        const int s = t - (L - 1) + j;               // index into this step's g; < 0: history
        float g;
        if (s >= 0) g = gated<T>(bcx, (size_t)(first + s), H, c);
        else g = has_state ? to_f<T>(st[(size_t)(s + L - 1) * H + c]) : 0.f;
        acc = fmaf(taps[j], g, acc);
      }
    }
    const float cgate = to_f<T>(bcx[(size_t)m * 3 * H + H + c]);
    out[(size_t)m * H + c] = from_f<T>(cgate * acc);
  }
}

template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, T* __restrict__ state,
                                        const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seg_start,
                                        const int* __restrict__ seg_slot, int H, int L) {
  pdl_begin();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  const int seg = blockIdx.y;
  const int first = cu_seqlens[seg], n = cu_seqlens[seg + 1] - first;
  if (n <= 0) return;
  const bool has_state = seg_start[seg] > 0;
  T* st = state + (size_t)seg_slot[seg] * (L - 1) * H;
  float next[CONV_MAX_L];
  // history ++ g has L-1+n rows; the new state is rows n .. n+L-2 of it.
#pragma unroll
  for (int i = 0; i < CONV_MAX_L; ++i) {
    if (i < L - 1) {
      const int idx = n + i;
      if (idx < L - 1) next[i] = has_state ? to_f<T>(st[(size_t)idx * H + c]) : 0.f;
      else next[i] = gated<T>(bcx, (size_t)(first + idx - (L - 1)), H, c);
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_L; ++i)
    if (i < L - 1) st[(size_t)i * H + c] = from_f<T>(next[i]);
}

// Many rows (prompt portions): a thread owns VEC consecutive channels (one vector) and walks CONV_STRIP
// consecutive rows, keeping the last L-1 values of g in registers, so B, C and x of a row are read
// once.  Every load of the strip, and of the L-1 rows before it, is issued before the first value is
// used: the loads do not wait for the segment look-ups, and a thread has the whole strip in flight.
// Up to 4 taps (L is a template parameter); the state is brought up to date by the second kernel.
#ifndef CONV_STRIP
#define CONV_STRIP 8
#endif
#define CONV_FAST_L 4

template <typename T> struct ConvVec;
template <> struct ConvVec<float> {
  static constexpr int N = 4;
  using Raw = float4;
  static __device__ __forceinline__ void unpack(const Raw& t, float (&v)[4]) {
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ Raw pack(const float (&v)[4]) { return make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct ConvVec<bf16> {
  static constexpr int N = 4;
  using Raw = uint2;
  static __device__ __forceinline__ void unpack(const Raw& t, float (&v)[4]) {
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
  static __device__ __forceinline__ Raw pack(const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  }
};

template <typename T, int L>
__global__ void __launch_bounds__(128)
short_conv_strip_kernel(const T* __restrict__ bcx, SmallVec w, const T* __restrict__ state,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ seg_start,
                        const int* __restrict__ seg_slot, const int* __restrict__ row_seg,
                        T* __restrict__ out, int M, int H) {
  pdl_begin();
  constexpr int VEC = ConvVec<T>::N;
  using Raw = typename ConvVec<T>::Raw;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= H) return;
  const int m_begin = blockIdx.y * CONV_STRIP;
  const size_t pitch = 3 * (size_t)H;
  Raw rb[CONV_STRIP], rc[CONV_STRIP], rx[CONV_STRIP], pb[L - 1], px[L - 1];
  int sgs[CONV_STRIP];
#pragma unroll
  for (int r = 0; r < CONV_STRIP; ++r) {
    if (m_begin + r < M) {
      const T* row = bcx + (size_t)(m_begin + r) * pitch + c0;
      rb[r] = *reinterpret_cast<const Raw*>(row);
      rc[r] = *reinterpret_cast<const Raw*>(row + H);
      rx[r] = *reinterpret_cast<const Raw*>(row + 2 * H);
      sgs[r] = row_seg[m_begin + r];
    }
  }
#pragma unroll
  for (int i = 0; i < L - 1; ++i) {                  // the rows before the strip: used if they are of its segment
    const int mm = m_begin - (L - 1) + i;
    if (mm >= 0) {
      const T* row = bcx + (size_t)mm * pitch + c0;
      pb[i] = *reinterpret_cast<const Raw*>(row);
      px[i] = *reinterpret_cast<const Raw*>(row + 2 * H);
    }
  }
  float taps[L][VEC];
#pragma unroll
  for (int j = 0; j < L; ++j)
#pragma unroll
    for (int e = 0; e < VEC; ++e) taps[j][e] = w[(size_t)(c0 + e) * L + j];
  float hist[L - 1][VEC];                            // hist[0] is the oldest of the L-1 values before the row
  int seg = -1;
#pragma unroll
  for (int r = 0; r < CONV_STRIP; ++r) {
    const int m = m_begin + r;
    if (m < M) {
      const int sg = sgs[r];
      if (r == 0 || sg != seg) {                     // (re)build the window: rows of this step, else the state
        seg = sg;
        const int t = m - cu_seqlens[sg];            // > 0 only at r == 0: a new segment starts at t == 0
        const bool has_state = seg_start[sg] > 0;
        const T* st = state + (size_t)seg_slot[sg] * (L - 1) * H;
#pragma unroll
        for (int i = 0; i < L - 1; ++i) {
          const int s = t - (L - 1) + i;             // index into this step's rows; < 0: history
          if (s >= 0) {                              // then r == 0 and the row is m_begin - (L-1) + i
            float b[VEC], x[VEC];
            ConvVec<T>::unpack(pb[i], b);
            ConvVec<T>::unpack(px[i], x);
#pragma unroll
            for (int e = 0; e < VEC; ++e) hist[i][e] = round_f<T>(b[e] * x[e]);
          } else if (has_state) {
            ConvVec<T>::unpack(*reinterpret_cast<const Raw*>(st + (size_t)(s + L - 1) * H + c0), hist[i]);
          } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) hist[i][e] = 0.f;
          }
        }
      }
      float b[VEC], cg[VEC], x[VEC], y[VEC];
      ConvVec<T>::unpack(rb[r], b);
      ConvVec<T>::unpack(rc[r], cg);
      ConvVec<T>::unpack(rx[r], x);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float g = round_f<T>(b[e] * x[e]);
        float acc = 0.f;                             // taps in order: oldest first, the current token last
#pragma unroll
        for (int i = 0; i < L - 1; ++i) acc = fmaf(taps[i][e], hist[i][e], acc);
        acc = fmaf(taps[L - 1][e], g, acc);
        y[e] = cg[e] * acc;
#pragma unroll
        for (int i = 0; i < L - 2; ++i) hist[i][e] = hist[i + 1][e];
        hist[L - 2][e] = g;
      }
      *reinterpret_cast<Raw*>(out + (size_t)m * H + c0) = ConvVec<T>::pack(y);
    }
  }
}

// Every segment holds one token (a decode step): one thread per (segment, channel) reads the
// history, computes the output and writes the new history; no second launch.
template <typename T>
__global__ void short_conv_decode_kernel(const T* __restrict__ bcx, SmallVec w, T* __restrict__ state,
                                         const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                                         T* __restrict__ out, int H, int L) {
  pdl_begin();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  const int seg = blockIdx.y;                        // = the row: one token per segment
  const bool has_state = seg_start[seg] > 0;
  T* st = state + (size_t)seg_slot[seg] * (L - 1) * H;
  float hist[CONV_MAX_L];
#pragma unroll
  for (int j = 0; j < CONV_MAX_L; ++j)
    if (j < L - 1) hist[j] = has_state ? to_f<T>(st[(size_t)j * H + c]) : 0.f;
  const float g = gated<T>(bcx, (size_t)seg, H, c);
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_L; ++j)
    if (j < L - 1) acc = fmaf(w[(size_t)c * L + j], hist[j], acc);
  acc = fmaf(w[(size_t)c * L + L - 1], g, acc);
  const float cgate = to_f<T>(bcx[(size_t)seg * 3 * H + H + c]);
  out[(size_t)seg * H + c] = from_f<T>(cgate * acc);
#pragma unroll
  for (int j = 0; j < CONV_MAX_L; ++j)
    if (j < L - 1) st[(size_t)j * H + c] = from_f<T>(j + 1 < L - 1 ? hist[j + 1] : g);
}

SNK_API int snk_short_conv(const void* bcx, const void* w, int w_is_f32, void* state,
                           const int* cu_seqlens, const int* seg_start, const int* seg_slot,
                           const int* row_seg, void* out, int M, int B, int H, int L, int dtype,
                           cudaStream_t stream) {
  if (M <= 0 || B <= 0) return 0;
  if (L < 1 || L > CONV_MAX_L) return SNK_ERR_SIZE;
  const int threads = 128;
  if (M == B && L > 1 && B <= 65535) {               // one token per segment
    dim3 dgrid((H + threads - 1) / threads, B);
    SmallVec dw{w, w_is_f32};
    SNK_DISPATCH(dtype, snk_launch(short_conv_decode_kernel<T>, dim3(dgrid), dim3(threads), 0, stream, 
                            static_cast<const T*>(bcx), dw, static_cast<T*>(state), seg_start, seg_slot,
                            static_cast<T*>(out), H, L));
    SNK_LAUNCH_CHECK();
    return 0;
  }
  SmallVec wv{w, w_is_f32};
  const int vec = 4;                                 // channels per thread: 16 bytes of float, 8 of bfloat16
  const size_t vbytes = dtype == SNK_F32 ? 16 : 8;
  const bool aligned = H % vec == 0 && (uintptr_t)bcx % vbytes == 0 && (uintptr_t)state % vbytes == 0 &&
                       (uintptr_t)out % vbytes == 0;
  if (L >= 2 && L <= CONV_FAST_L && aligned && M >= 4 * CONV_STRIP) {
    dim3 sgrid((H / vec + threads - 1) / threads, (M + CONV_STRIP - 1) / CONV_STRIP);
    if (sgrid.y > 65535u) return SNK_ERR_SIZE;
#define CONV_STRIP_LAUNCH(L_)                                                                          \
    snk_launch(short_conv_strip_kernel<T, L_>, dim3(sgrid), dim3(threads), 0, stream,                  \
               static_cast<const T*>(bcx), wv, static_cast<const T*>(state), cu_seqlens, seg_start,    \
               seg_slot, row_seg, static_cast<T*>(out), M, H)
    SNK_DISPATCH(dtype, {
      if (L == 2) CONV_STRIP_LAUNCH(2);
      else if (L == 3) CONV_STRIP_LAUNCH(3);
      else CONV_STRIP_LAUNCH(4);
    });
#undef CONV_STRIP_LAUNCH
  } else {
    dim3 grid((H + threads - 1) / threads, (M + CONV_ROWS_PER_BLOCK - 1) / CONV_ROWS_PER_BLOCK);
    if (grid.y > 65535u) return SNK_ERR_SIZE;
    SNK_DISPATCH(dtype, snk_launch(short_conv_kernel<T>, dim3(grid), dim3(threads), 0, stream, 
                            static_cast<const T*>(bcx), wv, static_cast<const T*>(state), cu_seqlens,
                            seg_start, seg_slot, row_seg, static_cast<T*>(out), M, H, L));
  }
  SNK_LAUNCH_CHECK();
  if (L > 1) {
    dim3 sgrid((H + threads - 1) / threads, B);
    SNK_DISPATCH(dtype, snk_launch(short_conv_state_kernel<T>, dim3(sgrid), dim3(threads), 0, stream, 
                            static_cast<const T*>(bcx), static_cast<T*>(state), cu_seqlens,
                            seg_start, seg_slot, H, L));
    SNK_LAUNCH_CHECK();
  }
  return 0;
}
