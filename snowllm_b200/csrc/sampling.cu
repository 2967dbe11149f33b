// Sampling over float logits [B, V]: argmax, penalties / bans, temperature + top-k + top-p draw.
//
//   argmax: NaN counts as -inf; equal values give the lowest index
//           (snowllm/ops/sampling.py:65-72; tests/test_sampling_argmax.py:29-31)
//   draw:   softmax(logits / temperature); keep the top_k most probable (0: all); of those the
//           smallest set of the most probable whose mass reaches top_p (ties at either cut are
//           kept); renormalise; walk the CDF in index order to u * mass for the supplied uniform
//           u (snowllm/engine/sampler.py:86-104; snowllm/ops/sampling.py:39-62).  A row with
//           temperature <= 0 is an argmax row (snowllm/engine/request.py:27-35).
//   penalties over the tokens a request has seen (snowllm/engine/request.py:19-21,
//           snowllm/engine/sampler.py:187-219): repetition r divides a positive logit and
//           multiplies a negative one, for prompt and output tokens; frequency f and presence p
//           subtract f*count + p*(count > 0) with the count of the token in the output.
//           A count of -1 marks a banned token (no_repeat_ngram_size): its logit becomes -inf.
// All sums are block reductions in a fixed order: same inputs, same token.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float clean(float v) { return v != v ? -INFINITY : v; }

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgPair { float v; int i; };

__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ ArgPair block_argmax(const float* __restrict__ row, int V, ArgPair* red) {
  ArgPair best{-INFINITY, 0x7fffffff};
  int done = 0;
  if ((uintptr_t)row % 16 == 0) {          // four values a load; a thread still meets its indices in ascending order
    done = V & ~3;
#pragma unroll 4
    for (int i = threadIdx.x * 4; i < done; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      best = better(best, ArgPair{clean(v.x), i});
      best = better(best, ArgPair{clean(v.y), i + 1});
      best = better(best, ArgPair{clean(v.z), i + 2});
      best = better(best, ArgPair{clean(v.w), i + 3});
    }
  }
  for (int i = done + threadIdx.x; i < V; i += blockDim.x) best = better(best, ArgPair{clean(row[i]), i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (warp == 0) {
    ArgPair t = lane < nwarp ? red[lane] : ArgPair{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgPair other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = better(t, other);
    }
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  ArgPair r = red[32];
  if (r.i == 0x7fffffff) r.i = 0;      // every value -inf or NaN
  return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  pdl_begin();
  __shared__ ArgPair red[33];
  const ArgPair r = block_argmax(logits + (size_t)blockIdx.x * V, V, red);
  if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

SNK_API int snk_argmax(const float* logits, int* out, int B, int V, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0) return SNK_ERR_SIZE;
  snk_launch(argmax_kernel, dim3(B), dim3(V >= 4096 ? 1024 : 256), 0, stream, logits, out, V);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
__global__ void penalties_kernel(float* __restrict__ logits, const int* __restrict__ row_offsets,
                                 const int* __restrict__ ids, const int* __restrict__ counts,
                                 const float* __restrict__ presence, const float* __restrict__ frequency,
                                 const float* __restrict__ repetition, int V) {
  pdl_begin();
  const int b = blockIdx.x;
  float* row = logits + (size_t)b * V;
  const float pp = presence[b], fp = frequency[b], rp = repetition[b];
  for (int i = row_offsets[b] + threadIdx.x; i < row_offsets[b + 1]; i += blockDim.x) {
    const int t = ids[i];
    if (t < 0 || t >= V) continue;
    const int c = counts[i];
    if (c < 0) { row[t] = -INFINITY; continue; }
    float v = row[t];
    if (rp != 1.f) v = v > 0.f ? v / rp : v * rp;
    v -= fp * (float)c + (c > 0 ? pp : 0.f);
    row[t] = v;
  }
}

// ids of one row must be distinct.
SNK_API int snk_apply_penalties(float* logits, const int* row_offsets, const int* ids,
                                const int* counts, const float* presence, const float* frequency,
                                const float* repetition, int B, int V, cudaStream_t stream) {
  if (B <= 0) return 0;
  snk_launch(penalties_kernel, dim3(B), dim3(256), 0, stream, logits, row_offsets, ids, counts, presence, frequency,
                                          repetition, V);
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_f(float v, float* red) { return block_sum(v, red); }

__device__ int block_sum_i(int v, int* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int t = lane < nwarp ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out, int V) {
  pdl_begin();
  __shared__ ArgPair ared[33];
  __shared__ float fred[33];
  __shared__ int ired[33];
  __shared__ float scan[SAMPLE_THREADS];
  __shared__ int chosen;
  const int b = blockIdx.x;
  const float* row = logits + (size_t)b * V;
  const ArgPair top = block_argmax(row, V, ared);
  const float temp = temperature[b];
  if (!(temp > 0.f) || top.v == -INFINITY) {
    if (threadIdx.x == 0) out[b] = top.i;
    return;
  }
  const float inv_t = 1.f / temp;
  const float mx = top.v;
  // unnormalised weight of a token
  auto weight = [&](float l) { return expf((l - mx) * inv_t); };

  unsigned cut = 0u;                                   // keep tokens whose key >= cut
  const int k = top_k[b];
  if (k > 0 && k < V) {
    unsigned u = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = u | (1u << bit);
      int c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += ordered_key(clean(row[i])) >= cand;
      if (block_sum_i(c, ired) >= k) u = cand;
    }
    cut = u;
  }
  const float p = top_p[b];
  if (p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = clean(row[i]);
      if (ordered_key(l) >= cut) z += weight(l);
    }
    z = block_sum_f(z, fred);
    const float need = p * z;
    unsigned u = 0u;                                   // largest key whose upper set reaches `need`
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = u | (1u << bit);
      const unsigned both = cand > cut ? cand : cut;
      float s = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = clean(row[i]);
        if (ordered_key(l) >= both) s += weight(l);
      }
      if (block_sum_f(s, fred) >= need) u = cand;
    }
    cut = u > cut ? u : cut;
  }
  // inverse CDF in index order over the kept tokens; thread t owns a contiguous run
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * per), end = min(V, begin + per);
  float local = 0.f;
  for (int i = begin; i < end; ++i) {
    const float l = clean(row[i]);
    if (ordered_key(l) >= cut) local += weight(l);
  }
  scan[threadIdx.x] = local;
  if (threadIdx.x == 0) chosen = top.i;                // fallback: the most probable token
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int t = 0; t < (int)blockDim.x; ++t) { const float v = scan[t]; scan[t] = run; run += v; }
    fred[0] = run;
  }
  __syncthreads();
  const float total = fred[0];
  float u01 = uniform[b];
  u01 = u01 < 0.f ? 0.f : (u01 >= 1.f ? 0.99999994f : u01);
  const float target = u01 * total;
  const float before = scan[threadIdx.x];
  if (local > 0.f && before <= target && target < before + local) {
    float run = before;
    int pick = -1, last = -1;
    for (int i = begin; i < end; ++i) {
      const float l = clean(row[i]);
      if (ordered_key(l) >= cut) {
        run += weight(l);
        last = i;
        if (run > target) { pick = i; break; }
      }
    }
    chosen = pick >= 0 ? pick : last;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[b] = chosen;
}

SNK_API int snk_sample(const float* logits, const float* temperature, const int* top_k,
                       const float* top_p, const float* uniform, int* out, int B, int V,
                       cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0) return SNK_ERR_SIZE;
  snk_launch(sample_kernel, dim3(B), dim3(SAMPLE_THREADS), 0, stream, logits, temperature, top_k, top_p, uniform, out, V);
  SNK_LAUNCH_CHECK();
  return 0;
}
