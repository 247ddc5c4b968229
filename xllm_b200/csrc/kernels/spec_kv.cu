// Speculative-decoding verification and PD (prefill/decode disaggregation) KV-block push.
//
//   spec_verify : rejection sampling over K draft tokens per sequence — greedy (ids must match the
//                 target arg-max) or stochastic (accept with min(1, p/q), resample the first rejected
//                 position from norm(max(p - q, 0)), bonus token from the last target distribution)
//   kv_push     : copy a list of KV blocks of one layer into a peer GPU's cache over NVLink with
//                 plain 16-byte stores (optionally re-slicing KV heads when the two sides use a
//                 different TP degree), then publish a per-layer flag; kv_wait is the bounded wait
//                 on the receiving side
//
// Parity: RejectionSampler (xllm/core/framework/sampling/rejection_sampler.cpp:65-360, a chain of
// torch ops) and KVCacheTransfer::push_kv_blocks_async with per-layer synchronisation
// (xllm/core/framework/kv_cache_transfer/kv_cache_transfer.h:63-165), which the reference only has
// through Mooncake on non-CUDA back ends (kv_cache_transfer.cpp:368-402).
#include "common.cuh"
#include <curand_kernel.h>

namespace xllm {

struct VerifyParams {
  const int64_t* draft_ids;   // [B, K]
  const float* target_probs;  // [B, K + 1, V]
  const float* draft_probs;   // [B, K, V] or null (deterministic drafts: q = one-hot)
  const uint8_t* greedy;      // [B] 1 = greedy row, or null (all stochastic)
  int64_t* out_tokens;        // [B, K + 1], -1 padded
  int32_t* out_len;           // [B] tokens emitted (accepted drafts + 1)
  int K, V;
  unsigned long long seed, offset;
  // per-row random streams (null: batch-level seed with the row as sub-stream): the seed of the
  // row's sequence and the number of tokens it has generated; a step draws at most 2 (K + 1) numbers
  const unsigned long long* seeds;
  const int32_t* offsets;
};

__global__ void __launch_bounds__(256) spec_verify_kernel(VerifyParams p) {
  __shared__ float red[32];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ int s_decision;   // -1 continue, else token chosen at the stopping position
  __shared__ float s_u;
  const int b = blockIdx.x;
  const int K = p.K, V = p.V;
  const float* P = p.target_probs + (int64_t)b * (K + 1) * V;
  const float* Q = p.draft_probs ? p.draft_probs + (int64_t)b * K * V : nullptr;
  const bool greedy = p.greedy ? p.greedy[b] != 0 : false;
  curandStatePhilox4_32_10_t st;
  if (threadIdx.x == 0) {
    if (p.seeds != nullptr)
      curand_init(p.seeds[b], 1ull, (unsigned long long)(p.offsets ? p.offsets[b] : 0) * (2ull * (p.K + 1)), &st);
    else
      curand_init(p.seed, (unsigned long long)b, p.offset, &st);
  }
  int n_out = 0;
  for (int i = 0; i <= K; ++i) {
    const float* pi = P + (int64_t)i * V;
    const float* qi = (Q && i < K) ? Q + (int64_t)i * V : nullptr;
    const int x = i < K ? (int)p.draft_ids[(int64_t)b * K + i] : -1;
    // ---- decide whether draft token x is accepted at position i
    bool accept = false;
    if (i < K) {
      if (greedy) {
        // arg-max of the target row
        float bv = -1.f; int bi = 0x7fffffff;
        for (int v = threadIdx.x; v < V; v += blockDim.x) { const float t = pi[v]; if (t > bv) { bv = t; bi = v; } }
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = bv; s_idx[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
          for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
          s_decision = (bi == x) ? -1 : bi;  // mismatch: the target's own token replaces the draft
        }
        __syncthreads();
        accept = s_decision == -1;
        if (!accept) {
          if (threadIdx.x == 0) p.out_tokens[(int64_t)b * (K + 1) + n_out] = s_decision;
          ++n_out;
          break;
        }
      } else {
        if (threadIdx.x == 0) {
          const float px = pi[x], qx = qi ? qi[x] : 1.f;
          const float u = curand_uniform(&st);
          s_decision = (qx > 0.f && u * qx <= px) ? -1 : -2;
          s_u = curand_uniform(&st);
        }
        __syncthreads();
        accept = s_decision == -1;
      }
      if (accept) {
        if (threadIdx.x == 0) p.out_tokens[(int64_t)b * (K + 1) + n_out] = x;
        ++n_out;
        __syncthreads();
        continue;
      }
    } else if (threadIdx.x == 0) {
      s_u = curand_uniform(&st);
    }
    __syncthreads();
    // ---- sample at the stopping position: recovered distribution max(p - q, 0) after a
    //      rejection, the plain target distribution for the bonus token (arg-max when greedy)
    if (greedy) {  // only reached for i == K
      float bv = -1.f; int bi = 0x7fffffff;
      for (int v = threadIdx.x; v < V; v += blockDim.x) { const float t = pi[v]; if (t > bv) { bv = t; bi = v; } }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = bv; s_idx[threadIdx.x >> 5] = bi; }
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
          if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        p.out_tokens[(int64_t)b * (K + 1) + n_out] = bi;
      }
      ++n_out;
      break;
    }
    auto weight = [&](int v) -> float {
      const float pv = pi[v];
      if (i == K) return pv;
      const float qv = qi ? qi[v] : (v == x ? 1.f : 0.f);
      return fmaxf(pv - qv, 0.f);
    };
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int beg = min((int)threadIdx.x * chunk, V), end = min(beg + chunk, V);
    float local = 0.f;
    for (int v = beg; v < end; ++v) local += weight(v);
    // block inclusive scan
    float incl = local;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
    if (lane == 31) red[wid] = incl;
    if (threadIdx.x == 0) s_decision = -1;
    __syncthreads();
    float wprefix = 0.f, total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { const float s = red[w]; if (w < wid) wprefix += s; total += s; }
    const float excl = wprefix + incl - local;
    const float target = s_u * total;
    if (local > 0.f && excl < target && target <= excl + local) {
      float run = excl; int pick = -1;
      for (int v = beg; v < end; ++v) { const float w = weight(v); if (w > 0.f) { run += w; pick = v; if (run >= target) break; } }
      atomicMax(&s_decision, pick);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = s_decision;
      if (c < 0) {  // degenerate (p == q everywhere): fall back to the target's mode
        float bv = -1.f; c = 0;
        for (int v = 0; v < V; ++v) if (pi[v] > bv) { bv = pi[v]; c = v; }
      }
      p.out_tokens[(int64_t)b * (K + 1) + n_out] = c;
    }
    ++n_out;
    break;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.out_len[b] = n_out;
    for (int i = n_out; i <= K; ++i) p.out_tokens[(int64_t)b * (K + 1) + i] = -1;
  }
}

// ------------------------------------------------------------------------------------------ KV push
struct PushParams {
  const uint8_t* src;       // this layer's cache (K or V) on the sending GPU
  uint8_t* dst;             // the same layer's cache on the receiving GPU (peer mapping)
  const int32_t* pairs;     // [n, 2] (source block, destination block)
  int64_t src_block_bytes, dst_block_bytes, head_bytes;
  int src_head0, dst_head0, n_heads;
  uint32_t* flag;           // on the receiver: set to `value` when every block has landed
  uint32_t value;
  uint32_t* arrive;         // local arrival counter (zero before and after the launch)
};

__global__ void __launch_bounds__(256) kv_push_kernel(PushParams p) {
  const int pair = blockIdx.y;
  const int64_t sb = p.pairs[2 * pair], db = p.pairs[2 * pair + 1];
  const int64_t vec_per_head = p.head_bytes >> 4;
  const int64_t total = vec_per_head * p.n_heads;
  const uint4* s = reinterpret_cast<const uint4*>(p.src + sb * p.src_block_bytes + (int64_t)p.src_head0 * p.head_bytes);
  uint4* d = reinterpret_cast<uint4*>(p.dst + db * p.dst_block_bytes + (int64_t)p.dst_head0 * p.head_bytes);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) d[i] = s[i];
  // last CTA to finish publishes the flag to the receiver
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned n_ctas = gridDim.x * gridDim.y;
    if (atomicAdd(p.arrive, 1u) == n_ctas - 1) {
      *p.arrive = 0;
      __threadfence_system();
      if (p.flag) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag), "r"(p.value) : "memory");
    }
  }
}

// status[0] = 0 when flag >= value was observed within the budget, else 1
__global__ void kv_wait_kernel(const uint32_t* flag, uint32_t value, int* status, long long budget_cycles) {
  const long long t0 = clock64();
  uint32_t v;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - value) >= 0) { *status = 0; return; }
    if (clock64() - t0 > budget_cycles) { *status = 1; return; }
  }
}

// The same for n flags at once (one per layer): thread i waits for flags[i]; status[0] = 0 when all
// arrived, else 1 + the index of a flag that did not arrive within the budget.
__global__ void kv_wait_many_kernel(const uint32_t* flags, int n, uint32_t value, int* status, long long budget_cycles) {
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long long t0 = clock64();
    uint32_t v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
      if ((int32_t)(v - value) >= 0) break;
      if (clock64() - t0 > budget_cycles) { atomicMax(&s_bad, i + 1); break; }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *status = s_bad;
}

}  // namespace xllm

XLLM_API int xllm_spec_verify(const void* draft_ids, const void* target_probs, const void* draft_probs,
                              const void* greedy, void* out_tokens, void* out_len, int B, int K, int V,
                              unsigned long long seed, unsigned long long offset, void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  VerifyParams p;
  p.draft_ids = (const int64_t*)draft_ids; p.target_probs = (const float*)target_probs;
  p.draft_probs = (const float*)draft_probs; p.greedy = (const uint8_t*)greedy; p.out_tokens = (int64_t*)out_tokens;
  p.out_len = (int32_t*)out_len; p.K = K; p.V = V; p.seed = seed; p.offset = offset;
  p.seeds = nullptr; p.offsets = nullptr;
  spec_verify_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(p);
  return XLLM_LAUNCH_CHECK();
}

// Same with one random stream per row: seeds [B] u64, offsets [B] i32 (tokens generated so far).
XLLM_API int xllm_spec_verify_rows(const void* draft_ids, const void* target_probs, const void* draft_probs,
                                   const void* greedy, void* out_tokens, void* out_len, int B, int K, int V,
                                   const void* seeds, const void* offsets, void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  if (seeds == nullptr) return (int)cudaErrorInvalidValue;
  VerifyParams p;
  p.draft_ids = (const int64_t*)draft_ids; p.target_probs = (const float*)target_probs;
  p.draft_probs = (const float*)draft_probs; p.greedy = (const uint8_t*)greedy; p.out_tokens = (int64_t*)out_tokens;
  p.out_len = (int32_t*)out_len; p.K = K; p.V = V; p.seed = 0; p.offset = 0;
  p.seeds = (const unsigned long long*)seeds; p.offsets = (const int32_t*)offsets;
  spec_verify_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(p);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_kv_push(const void* src, void* dst, const void* pairs, int n_pairs, int64_t src_block_bytes,
                          int64_t dst_block_bytes, int64_t head_bytes, int src_head0, int dst_head0, int n_heads,
                          void* flag, uint32_t value, void* arrive, void* stream) {
  using namespace xllm;
  if (head_bytes % 16) return (int)cudaErrorInvalidValue;
  PushParams p;
  p.src = (const uint8_t*)src; p.dst = (uint8_t*)dst; p.pairs = (const int32_t*)pairs;
  p.src_block_bytes = src_block_bytes; p.dst_block_bytes = dst_block_bytes; p.head_bytes = head_bytes;
  p.src_head0 = src_head0; p.dst_head0 = dst_head0; p.n_heads = n_heads; p.flag = (uint32_t*)flag; p.value = value;
  p.arrive = (uint32_t*)arrive;
  if (n_pairs == 0) return 0;  // nothing to copy; the caller publishes the flag itself
  const int64_t vec = (head_bytes >> 4) * n_heads;
  int gx = (int)((vec + 255) / 256);
  if (gx > 8) gx = 8;
  dim3 grid(gx, n_pairs);
  kv_push_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_kv_wait(const void* flag, uint32_t value, void* status, long long budget_cycles, void* stream) {
  using namespace xllm;
  kv_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const uint32_t*)flag, value, (int*)status, budget_cycles);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_kv_wait_many(const void* flags, int n, uint32_t value, void* status, long long budget_cycles,
                               void* stream) {
  using namespace xllm;
  if (n <= 0) return (int)cudaErrorInvalidValue;
  kv_wait_many_kernel<<<1, 128, 0, (cudaStream_t)stream>>>((const uint32_t*)flags, n, value, (int*)status, budget_cycles);
  return XLLM_LAUNCH_CHECK();
}
