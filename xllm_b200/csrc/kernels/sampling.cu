// Device sampler: penalties, temperature, top-k, top-p, greedy / random choice, log-probability.
//
// Behavioural parity with Sampler::forward of the reference
// (xllm/core/framework/sampling/sampler.cpp:29-180: penalties -> temperature/top-k/top-p ->
// softmax -> greedy | multinomial -> log_softmax of the *filtered* logits gathered at the sample)
// and with its FlashInfer-backed `random_sample` (xllm/core/kernels/cuda/random_sample.cpp:60-93).
// The reference runs this as ~10 torch ops plus a library kernel; here one CTA per row does the
// whole chain without materialising probabilities or sorting the vocabulary:
//   * e_i = exp((x_i - max) / T) is recomputed from the logits on every pass (row lives in L2);
//   * the kept set of top-k ∩ top-p is {e_i >= t*}; keep(v) = (#{e > v} < k) && (sum{e > v} < p*Z)
//     is monotone in v, so t* is found by bisection on the fp32 bit pattern (exact, 31 passes);
//   * the sample is drawn by an ordered block scan over the kept mass.
#include "common.cuh"
#include <curand_kernel.h>

namespace xllm {

constexpr int kSampleThreads = 1024;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p, int64_t i) { return __bfloat162float(p[i]); }

struct SampleParams {
  const void* logits;   // [B, V]
  int64_t row_stride;
  const float* temperature;  // [B] (<= 0 or null => greedy)
  const int32_t* top_k;      // [B] (<= 0 or null => no limit)
  const float* top_p;        // [B] (>= 1 or null => no limit)
  int64_t* out_ids;          // [B]
  float* out_logprob;        // [B] or null
  int V;
  unsigned long long seed, offset;
  // per-row random streams: seed of the row's sequence and how many draws it has made (tokens
  // generated so far).  Null: the batch-level (seed, offset) with the row as the subsequence.
  const unsigned long long* seeds;
  const int32_t* offsets;
};

__device__ __forceinline__ void block_argmax(float& v, int& idx, float* redv, int* redi) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  if (lane == 0) { redv[wid] = v; redi[wid] = idx; }
  __syncthreads();
  const int nw = blockDim.x >> 5;
  v = lane < nw ? redv[lane] : -INFINITY;
  idx = lane < nw ? redi[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleParams p) {
  __shared__ float red[32];
  __shared__ float redv[32];
  __shared__ int redi[32];
  __shared__ float scan[kSampleThreads / 32];
  __shared__ int s_choice;
  const int row = blockIdx.x;
  const T* x = reinterpret_cast<const T*>(p.logits) + (int64_t)row * p.row_stride;
  const int V = p.V;
  pdl_wait();

  float mx = -INFINITY;
  int arg = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kSampleThreads) {
    const float v = ldf<T>(x, i);
    if (v > mx) { mx = v; arg = i; }
  }
  block_argmax(mx, arg, redv, redi);

  const float temp = p.temperature ? p.temperature[row] : 0.f;
  const bool greedy = !(temp > 0.f);
  if (greedy && p.out_logprob == nullptr) {
    if (threadIdx.x == 0) p.out_ids[row] = arg;
    return;
  }
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const float sc = inv_t * 1.4426950408889634f;
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += kSampleThreads) z += exp2f((ldf<T>(x, i) - mx) * sc);
  const float Z = block_sum(z, red);
  if (greedy) {
    if (threadIdx.x == 0) {
      p.out_ids[row] = arg;
      p.out_logprob[row] = -logf(Z);  // e_arg == 1
    }
    return;
  }

  int k = p.top_k ? p.top_k[row] : 0;
  if (k <= 0 || k > V) k = V;
  float tp = p.top_p ? p.top_p[row] : 1.f;
  const bool filter = (k < V) || (tp < 1.f);
  float thr = 0.f;  // kept set = {e >= thr}
  if (filter) {
    const float mass_limit = tp * Z;
    uint32_t lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      const float v = __uint_as_float(mid);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        const float e = exp2f((ldf<T>(x, i) - mx) * sc);
        if (e > v) { cnt += 1.f; mass += e; }
      }
      cnt = block_sum(cnt, red);
      mass = block_sum(mass, red);
      const bool ok = (cnt < (float)k) && (tp >= 1.f || mass < mass_limit);
      if (ok) hi = mid; else lo = mid + 1;
    }
    thr = __uint_as_float(hi);
  }

  // ordered scan over contiguous per-thread chunks
  const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
  const int beg = min(threadIdx.x * chunk, V), end = min(beg + chunk, V);
  float local = 0.f;
  for (int i = beg; i < end; ++i) {
    const float e = exp2f((ldf<T>(x, i) - mx) * sc);
    if (e >= thr) local += e;
  }
  // inclusive scan of `local` across the block
  float incl = local;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) scan[wid] = incl;
  if (threadIdx.x == 0) s_choice = -1;
  __syncthreads();
  float wprefix = 0.f, total = 0.f;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    const float s = scan[w];
    if (w < wid) wprefix += s;
    total += s;
  }
  const float excl = wprefix + incl - local;
  curandStatePhilox4_32_10_t st;
  if (p.seeds != nullptr)
    curand_init(p.seeds[row], 0ull, p.offsets ? (unsigned long long)p.offsets[row] : 0ull, &st);
  else
    curand_init(p.seed, (unsigned long long)row, p.offset, &st);
  const float u = curand_uniform(&st);  // (0, 1]
  const float target = u * total;
  // the owner is the first thread whose inclusive prefix reaches the target
  if (local > 0.f && excl < target && target <= excl + local) {
    float run = excl;
    int pick = -1;
    for (int i = beg; i < end; ++i) {
      const float e = exp2f((ldf<T>(x, i) - mx) * sc);
      if (e >= thr) {
        run += e;
        pick = i;
        if (run >= target) break;
      }
    }
    atomicMax(&s_choice, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = s_choice;
    if (c < 0) c = arg;  // rounding left no owner: fall back to the mode (always in the kept set)
    p.out_ids[row] = c;
    if (p.out_logprob) {
      const float e = exp2f((ldf<T>(x, c) - mx) * sc);
      p.out_logprob[row] = logf(e / total);
    }
  }
}

// The n most likely tokens of every row with their log-probabilities under softmax(logits)
// (Sampler::forward's top_logprobs, xllm/core/framework/sampling/sampler.cpp:166-169; the reference
// sorts with torch.topk).  One CTA per row: max and normaliser in two passes, then n arg-max
// passes, each restricted to the elements that come after the previous pick in the order
// (value descending, index ascending).  n is small (<= 20 in the OpenAI API) and the row is in L2.
template <typename T>
__global__ void __launch_bounds__(kSampleThreads) top_logprobs_kernel(const T* logits, int64_t row_stride, int V, int n,
                                                                      int32_t* out_ids, float* out_lp) {
  __shared__ float red[32];
  __shared__ float redv[32];
  __shared__ int redi[32];
  const int row = blockIdx.x;
  const T* x = logits + (int64_t)row * row_stride;
  pdl_wait();
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kSampleThreads) mx = fmaxf(mx, ldf<T>(x, i));
  mx = block_max(mx, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += kSampleThreads) z += __expf(ldf<T>(x, i) - mx);
  const float logz = logf(block_sum(z, red));
  float pv = INFINITY;
  int pi = -1;
  for (int k = 0; k < n; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
      const float v = ldf<T>(x, i);
      const bool after = (v < pv) || (v == pv && i > pi);
      if (after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
    }
    block_argmax(bv, bi, redv, redi);
    if (threadIdx.x == 0) {
      out_ids[(int64_t)row * n + k] = bi == 0x7fffffff ? -1 : bi;
      out_lp[(int64_t)row * n + k] = bi == 0x7fffffff ? -INFINITY : bv - mx - logz;
    }
    pv = bv;
    pi = bi;
  }
}

// logits[row, id] adjusted for every (row, j) with id = ids[row, j] >= 0:
//   repetition: x = x > 0 ? x / r : x * r ;  then  x -= freq * count + presence * (count > 0)
template <typename T>
__global__ void penalties_kernel(T* logits, int64_t row_stride, const int32_t* ids,
                                 const int32_t* counts, int max_unique, const float* freq,
                                 const float* presence, const float* repetition, int V) {
  const int row = blockIdx.x;
  const float f = freq ? freq[row] : 0.f, pr = presence ? presence[row] : 0.f;
  const float rp = repetition ? repetition[row] : 1.f;
  for (int j = threadIdx.x; j < max_unique; j += blockDim.x) {
    const int id = ids[(int64_t)row * max_unique + j];
    if (id < 0 || id >= V) continue;
    const int c = counts ? counts[(int64_t)row * max_unique + j] : 1;
    if (c <= 0) continue;
    T* px = logits + (int64_t)row * row_stride + id;
    float v = (float)*px;
    if (rp != 1.f) v = v > 0.f ? v / rp : v * rp;
    v -= f * (float)c + pr;
    *px = (T)v;
  }
}

}  // namespace xllm

// dtype: 0 = bf16 logits, 1 = fp32 logits.
XLLM_API int xllm_sample(const void* logits, int64_t row_stride, int dtype, int batch, int vocab,
                         const void* temperature, const void* top_k, const void* top_p,
                         void* out_ids, void* out_logprob, unsigned long long seed,
                         unsigned long long offset, void* stream) {
  using namespace xllm;
  if (batch == 0) return 0;
  SampleParams p;
  p.logits = logits; p.row_stride = row_stride; p.temperature = (const float*)temperature;
  p.top_k = (const int32_t*)top_k; p.top_p = (const float*)top_p; p.out_ids = (int64_t*)out_ids;
  p.out_logprob = (float*)out_logprob; p.V = vocab; p.seed = seed; p.offset = offset;
  p.seeds = nullptr; p.offsets = nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) launch_pdl(sample_kernel<bf16>, dim3(batch), dim3(kSampleThreads), 0, s, p);
  else launch_pdl(sample_kernel<float>, dim3(batch), dim3(kSampleThreads), 0, s, p);
  return XLLM_LAUNCH_CHECK();
}

// Same sampler with one random stream per row: seeds [batch] u64 (the row's sequence seed) and
// offsets [batch] i32 (draws that sequence has made so far), both device arrays, so the launch does
// not depend on host values and can be replayed from a CUDA graph.
XLLM_API int xllm_sample_rows(const void* logits, int64_t row_stride, int dtype, int batch, int vocab,
                              const void* temperature, const void* top_k, const void* top_p, void* out_ids,
                              void* out_logprob, const void* seeds, const void* offsets, void* stream) {
  using namespace xllm;
  if (batch == 0) return 0;
  if (seeds == nullptr) return (int)cudaErrorInvalidValue;
  SampleParams p;
  p.logits = logits; p.row_stride = row_stride; p.temperature = (const float*)temperature;
  p.top_k = (const int32_t*)top_k; p.top_p = (const float*)top_p; p.out_ids = (int64_t*)out_ids;
  p.out_logprob = (float*)out_logprob; p.V = vocab; p.seed = 0; p.offset = 0;
  p.seeds = (const unsigned long long*)seeds; p.offsets = (const int32_t*)offsets;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) launch_pdl(sample_kernel<bf16>, dim3(batch), dim3(kSampleThreads), 0, s, p);
  else launch_pdl(sample_kernel<float>, dim3(batch), dim3(kSampleThreads), 0, s, p);
  return XLLM_LAUNCH_CHECK();
}

// out_ids [batch, n] int32 and out_lp [batch, n] fp32: the n most likely tokens of every row and
// their log-probabilities under softmax(logits), most likely first (ties: lowest index).
XLLM_API int xllm_top_logprobs(const void* logits, int64_t row_stride, int dtype, int batch, int vocab, int n,
                               void* out_ids, void* out_lp, void* stream) {
  using namespace xllm;
  if (batch == 0 || n == 0) return 0;
  if (n < 0 || n > vocab) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0)
    launch_pdl(top_logprobs_kernel<bf16>, dim3(batch), dim3(kSampleThreads), 0, s, (const bf16*)logits, row_stride,
               vocab, n, (int32_t*)out_ids, (float*)out_lp);
  else
    launch_pdl(top_logprobs_kernel<float>, dim3(batch), dim3(kSampleThreads), 0, s, (const float*)logits, row_stride,
               vocab, n, (int32_t*)out_ids, (float*)out_lp);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_apply_penalties(void* logits, int64_t row_stride, int dtype, int batch, int vocab,
                                  const void* ids, const void* counts, int max_unique,
                                  const void* freq, const void* presence, const void* repetition,
                                  void* stream) {
  using namespace xllm;
  if (batch == 0 || max_unique == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0)
    penalties_kernel<bf16><<<batch, 256, 0, s>>>((bf16*)logits, row_stride, (const int32_t*)ids,
                                                 (const int32_t*)counts, max_unique, (const float*)freq,
                                                 (const float*)presence, (const float*)repetition, vocab);
  else
    penalties_kernel<float><<<batch, 256, 0, s>>>((float*)logits, row_stride, (const int32_t*)ids,
                                                  (const int32_t*)counts, max_unique, (const float*)freq,
                                                  (const float*)presence, (const float*)repetition, vocab);
  return XLLM_LAUNCH_CHECK();
}
