// Selection kernels of beam search and generative recommendation.
//
//   log_softmax      : row-wise log-softmax of logits (bf16 / fp32 in, fp32 out)
//   radix_topk       : the k largest entries of every row by radix selection, sorted, optionally as
//                      log-probabilities (the row's log-normaliser is subtracted)
//   beam_step        : one beam-search step for B requests x W beams: the W best of the W x k
//                      candidates (cumulative score of the parent + candidate log-probability),
//                      with their parents and tokens
//
// Parity: xllm/core/kernels/cuda/air_log_softmax_last_dim.cu:35-250 (log-softmax),
// topk_last_dim.cuh:1556-1986 (radix top-k over the last dimension), rec_beam_search.cu:503-1063
// (beam step of the recommendation models) and beam_search.cu.
//
// Radix selection works on a 56-bit composite key: [order-preserving image of the fp32 value : 32]
// [0xFFFFFF - index : 24].  Keys are unique, so "the k largest" is a well-defined set and ties in
// the value go to the lowest index, like a stable sort; seven 8-bit passes find the k-th key, one
// more pass gathers the k winners, a bitonic network in shared memory orders them.  Rows are
// re-read from L2 (a 152k-entry bf16 row is 300 KB).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"

namespace xllm {

constexpr int kTopkThreads = 1024;
constexpr int kTopkMax = 2048;   // the DSA indexer keeps 2048 context tokens per query

template <typename T> __device__ __forceinline__ float beam_ld(const T* x, int64_t i);
template <> __device__ __forceinline__ float beam_ld<float>(const float* x, int64_t i) { return x[i]; }
template <> __device__ __forceinline__ float beam_ld<bf16>(const bf16* x, int64_t i) { return __bfloat162float(x[i]); }

__device__ __forceinline__ uint32_t float_key(float f) {
  if (f != f) f = -INFINITY;                       // NaN sorts last
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint64_t make_key(float v, int i) {
  return ((uint64_t)float_key(v) << 24) | (uint64_t)(0xFFFFFFu - (uint32_t)i);
}

__device__ __forceinline__ float topk_block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  return v;
}
__device__ __forceinline__ float topk_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  return v;
}

// ------------------------------------------------------------------------------------------ log-softmax
// f(value, index) for every element of the row, this thread's share: 16-byte loads over the aligned body
// (each thread takes whole vectors, so a warp reads 512 contiguous bytes per step), scalar head and tail.
template <typename T, typename F>
__device__ __forceinline__ void row_for_each(const T* __restrict__ r, int V, F f) {
  constexpr int PER = 16 / (int)sizeof(T);
  const int mis = (int)(((uintptr_t)r & 15) / sizeof(T));
  const int head = mis == 0 ? 0 : min(V, PER - mis);
  const int nvec = (V - head) / PER;
  for (int i = threadIdx.x; i < head; i += blockDim.x) f(beam_ld<T>(r, i), i);
  const uint4* rv = reinterpret_cast<const uint4*>(r + head);
  for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
    const uint4 raw = rv[j];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int t = 0; t < PER; ++t) f(beam_ld<T>(e, t), head + j * PER + t);
  }
  for (int i = head + nvec * PER + threadIdx.x; i < V; i += blockDim.x) f(beam_ld<T>(r, i), i);
}

// log-sum-exp of the row in ONE pass: every thread keeps a running maximum and the sum of exponentials
// relative to it, the block combines them.
template <typename T>
__device__ __forceinline__ float row_lse(const T* __restrict__ r, int V, float* red) {
  float m = -INFINITY, z = 0.f;
  row_for_each<T>(r, V, [&](float v, int) {
    if (v > m) {
      z = z * __expf(m - v) + 1.f;                // m = -inf: z is 0 and so is the factor
      m = v;
    } else if (v > -INFINITY) {
      z += __expf(v - m);
    }
  });
  const float mx = topk_block_max(m, red);
  z = (m > -INFINITY) ? z * __expf(m - mx) : 0.f;
  return mx + logf(topk_block_sum(z, red));
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads) log_softmax_kernel(const T* __restrict__ x, int64_t row_stride, int V,
                                                                   float* __restrict__ out) {
  __shared__ float red[32];
  const T* r = x + (int64_t)blockIdx.x * row_stride;
  const float lse = row_lse<T>(r, V, red);
  float* o = out + (int64_t)blockIdx.x * V;
  // the second read of the row hits L2; 16-byte loads and, where the output lines up, 16-byte stores
  constexpr int PER = 16 / (int)sizeof(T);
  const int mis = (int)(((uintptr_t)r & 15) / sizeof(T));
  const int head = mis == 0 ? 0 : min(V, PER - mis);
  const int nvec = (V - head) / PER;
  for (int i = threadIdx.x; i < head; i += blockDim.x) o[i] = beam_ld<T>(r, i) - lse;
  const uint4* rv = reinterpret_cast<const uint4*>(r + head);
  const bool o_aligned = (((uintptr_t)(o + head)) & 15) == 0;
  for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
    const uint4 raw = rv[j];
    const T* e = reinterpret_cast<const T*>(&raw);
    float f[PER];
#pragma unroll
    for (int t = 0; t < PER; ++t) f[t] = beam_ld<T>(e, t) - lse;
    float* dst = o + head + (int64_t)j * PER;
    if (o_aligned) {
#pragma unroll
      for (int t = 0; t < PER; t += 4) *reinterpret_cast<float4*>(dst + t) = make_float4(f[t], f[t + 1], f[t + 2], f[t + 3]);
    } else {
#pragma unroll
      for (int t = 0; t < PER; ++t) dst[t] = f[t];
    }
  }
  for (int i = head + nvec * PER + threadIdx.x; i < V; i += blockDim.x) o[i] = beam_ld<T>(r, i) - lse;
}

// ------------------------------------------------------------------------------------------ selection core
// Value of candidate i of this row; Loader::n() entries.
template <typename T>
struct RowLoader {
  const T* x;
  int V;
  __device__ __forceinline__ int n() const { return V; }
  __device__ __forceinline__ float operator()(int i) const { return beam_ld<T>(x, i); }
};
// W beams x k candidates: score = cum[w] + lp[w][j]; finished parents (cum = -inf) drop out by themselves
struct BeamLoader {
  const float* lp;    // [W * k]
  const float* cum;   // [W]
  int W, k;
  __device__ __forceinline__ int n() const { return W * k; }
  __device__ __forceinline__ float operator()(int i) const { return lp[i] + cum[i / k]; }
};

constexpr int kCandMax = 3072;   // candidates kept in shared memory once the selection has narrowed to that few

// Adds one key's digit to the histogram: one shared atomic per distinct digit of the warp.
__device__ __forceinline__ void hist_add(uint32_t* s_hist, int digit) {
  const unsigned peers = __match_any_sync(0xffffffffu, digit);
  if (digit >= 0 && (int)(__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&s_hist[digit], (uint32_t)__popc(peers));
}

// Leaves the k largest keys of the row, sorted descending, in s_keys[0..k).  k <= kTopkMax, k <= n.
//
// Radix selection from the most significant byte of the 56-bit key down.  The passes read the row from
// global memory only until the keys that still tie with the prefix number at most kCandMax; one more pass
// then moves those candidates into shared memory (and the keys already known to be among the k largest
// straight into s_keys), and the remaining bytes are resolved there.  For bf16 rows that is after two
// passes (the 16 value bits), so a row is read three times instead of eight.
// s_int: [0] remaining, [1] winners written, [2] ties with the new prefix, [3] candidates written.
template <typename Loader>
__device__ void radix_select_sorted(const Loader& ld, int k, uint64_t* s_keys, uint32_t* s_hist, uint64_t* s_prefix,
                                    int* s_int, uint64_t* s_cand) {
  const int n = ld.n();
  uint64_t prefix = 0;
  int remaining = k;
  int n_cand = -1;                                  // < 0: the row is still read from global memory
  int p2 = 1;
  while (p2 < k) p2 <<= 1;
  for (int i = threadIdx.x; i < p2; i += blockDim.x) s_keys[i] = 0ull;
  if (threadIdx.x == 0) s_int[1] = 0;
  for (int pass = 6; pass >= 0; --pass) {
    const int shift = pass * 8;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    const uint64_t hi_mask = pass == 6 ? 0ull : (~0ull << (shift + 8));
    const int count = n_cand < 0 ? n : n_cand;
    for (int base = 0; base < count; base += blockDim.x) {
      const int i = base + threadIdx.x;
      int digit = -1;
      if (i < count) {
        const uint64_t key = n_cand < 0 ? make_key(ld(i), i) : s_cand[i];
        if ((key & hi_mask) == prefix) digit = (int)((key >> shift) & 255u);
      }
      hist_add(s_hist, digit);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, d = 255;
      for (; d > 0; --d) {
        if (acc + (int)s_hist[d] >= remaining) break;
        acc += (int)s_hist[d];
      }
      s_int[0] = remaining - acc;
      s_int[2] = (int)s_hist[d];
      s_int[3] = 0;
      *s_prefix = prefix | ((uint64_t)d << shift);
    }
    __syncthreads();
    prefix = *s_prefix;
    remaining = s_int[0];
    const int ties = s_int[2];
    __syncthreads();
    if (n_cand < 0 && pass > 0 && ties <= kCandMax) {
      const uint64_t mask = ~0ull << shift;         // the bytes decided so far
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const uint64_t key = make_key(ld(i), i);
        const uint64_t top = key & mask;
        if (top == prefix) {
          const int slot = atomicAdd(&s_int[3], 1);
          if (slot < kCandMax) s_cand[slot] = key;
        } else if (top > prefix) {                  // larger in a decided byte: one of the k largest for certain
          const int slot = atomicAdd(&s_int[1], 1);
          if (slot < p2) s_keys[slot] = key;
        }
      }
      __syncthreads();
      n_cand = min(s_int[3], kCandMax);
    }
  }
  // prefix is now the k-th largest key: everything >= it that is not in s_keys yet joins (k keys in all)
  if (n_cand < 0) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint64_t key = make_key(ld(i), i);
      if (key >= prefix) {
        const int slot = atomicAdd(&s_int[1], 1);
        if (slot < p2) s_keys[slot] = key;
      }
    }
  } else {
    for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
      const uint64_t key = s_cand[i];
      if (key >= prefix) {
        const int slot = atomicAdd(&s_int[1], 1);
        if (slot < p2) s_keys[slot] = key;
      }
    }
  }
  __syncthreads();
  // bitonic sort, descending
  for (int size = 2; size <= p2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (p2 >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const uint64_t a = s_keys[lo], b = s_keys[hi];
        if ((a < b) == desc) { s_keys[lo] = b; s_keys[hi] = a; }
      }
      __syncthreads();
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads) radix_topk_kernel(const T* __restrict__ x, int64_t row_stride, int V, int k,
                                                                  int normalize, float* __restrict__ out_vals,
                                                                  int32_t* __restrict__ out_ids) {
  __shared__ uint64_t s_keys[kTopkMax];
  __shared__ uint32_t s_hist[256];
  __shared__ uint64_t s_prefix;
  __shared__ int s_int[4];
  __shared__ uint64_t s_cand[kCandMax];
  __shared__ float red[32];
  const T* r = x + (int64_t)blockIdx.x * row_stride;
  float lse = 0.f;
  if (normalize) {
    lse = row_lse<T>(r, V, red);
  }
  RowLoader<T> ld{r, V};
  radix_select_sorted(ld, k, s_keys, s_hist, &s_prefix, s_int, s_cand);
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const uint64_t key = s_keys[i];
    out_ids[(int64_t)blockIdx.x * k + i] = (int32_t)(0xFFFFFFu - (uint32_t)(key & 0xFFFFFFu));
    out_vals[(int64_t)blockIdx.x * k + i] = key_float((uint32_t)(key >> 24)) - lse;
  }
}

// One CTA per request.  cand_lp / cand_ids: [B, W, k]; cum: [B, W]; outputs [B, W].
__global__ void __launch_bounds__(kTopkThreads) beam_step_kernel(const float* __restrict__ cand_lp,
                                                                 const int32_t* __restrict__ cand_ids,
                                                                 const float* __restrict__ cum, int W, int k, int n_out,
                                                                 int32_t* __restrict__ out_token,
                                                                 int32_t* __restrict__ out_parent,
                                                                 float* __restrict__ out_score) {
  __shared__ uint64_t s_keys[kTopkMax];
  __shared__ uint32_t s_hist[256];
  __shared__ uint64_t s_prefix;
  __shared__ int s_int[4];
  __shared__ uint64_t s_cand[kCandMax];
  const int b = blockIdx.x;
  BeamLoader ld{cand_lp + (int64_t)b * W * k, cum + (int64_t)b * W, W, k};
  radix_select_sorted(ld, n_out, s_keys, s_hist, &s_prefix, s_int, s_cand);
  for (int i = threadIdx.x; i < n_out; i += blockDim.x) {
    const uint64_t key = s_keys[i];
    const int idx = (int)(0xFFFFFFu - (uint32_t)(key & 0xFFFFFFu));
    out_parent[(int64_t)b * n_out + i] = idx / k;
    out_token[(int64_t)b * n_out + i] = cand_ids[(int64_t)b * W * k + idx];
    out_score[(int64_t)b * n_out + i] = key_float((uint32_t)(key >> 24));
  }
}

}  // namespace xllm

// dtype: 0 bf16, 1 fp32.  out: fp32 [rows, V] dense.
XLLM_API int xllm_log_softmax(const void* x, int64_t row_stride, int dtype, int rows, int V, void* out, void* stream) {
  using namespace xllm;
  if (rows == 0) return 0;
  if (V <= 0) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) log_softmax_kernel<bf16><<<rows, kTopkThreads, 0, s>>>((const bf16*)x, row_stride, V, (float*)out);
  else log_softmax_kernel<float><<<rows, kTopkThreads, 0, s>>>((const float*)x, row_stride, V, (float*)out);
  return XLLM_LAUNCH_CHECK();
}

// The k largest entries of every row, sorted descending (ties: lowest index first).  normalize != 0:
// values are log-probabilities of the row.  1 <= k <= min(V, 2048), V < 2^24.
XLLM_API int xllm_radix_topk(const void* x, int64_t row_stride, int dtype, int rows, int V, int k, int normalize,
                             void* out_vals, void* out_ids, void* stream) {
  using namespace xllm;
  if (rows == 0) return 0;
  if (k < 1 || k > kTopkMax || k > V || V >= (1 << 24)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0)
    radix_topk_kernel<bf16><<<rows, kTopkThreads, 0, s>>>((const bf16*)x, row_stride, V, k, normalize, (float*)out_vals,
                                                           (int32_t*)out_ids);
  else
    radix_topk_kernel<float><<<rows, kTopkThreads, 0, s>>>((const float*)x, row_stride, V, k, normalize, (float*)out_vals,
                                                            (int32_t*)out_ids);
  return XLLM_LAUNCH_CHECK();
}

// The n_out best of W x k candidates per request.  n_out <= min(W * k, 2048).
XLLM_API int xllm_beam_step(const void* cand_lp, const void* cand_ids, const void* cum, int B, int W, int k, int n_out,
                            void* out_token, void* out_parent, void* out_score, void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  if (W < 1 || k < 1 || n_out < 1 || n_out > kTopkMax || n_out > W * k || (int64_t)W * k >= (1 << 24))
    return (int)cudaErrorInvalidValue;
  beam_step_kernel<<<B, kTopkThreads, 0, (cudaStream_t)stream>>>((const float*)cand_lp, (const int32_t*)cand_ids,
                                                                 (const float*)cum, W, k, n_out, (int32_t*)out_token,
                                                                 (int32_t*)out_parent, (float*)out_score);
  return XLLM_LAUNCH_CHECK();
}
