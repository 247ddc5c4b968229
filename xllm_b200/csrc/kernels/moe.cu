// Mixture-of-experts routing, token permutation and finalisation.
//
//   moe_route    : softmax / sigmoid scoring (+ selection bias), group-limited top-k
//                  (n_group / topk_group), renormalisation, routed scaling; emits expert ids,
//                  weights, per-expert counts and each token's slot inside its expert
//   moe_offsets  : padded exclusive scan of the counts (segments start on 128-row tiles, so a
//                  GEMM tile never straddles two experts) + the tile -> expert table the grouped
//                  GEMM walks
//   moe_permute  : gather token rows into expert-major order
//   moe_finalize : out[t] = sum_k w[t,k] * y[row(t,k)]  (+ optional shared-expert output)
//
// Parity: moe_topk_softmax / moe_topk_sigmoid (xllm/core/kernels/cuda/moe/moe_topk_softmax_kernels.cuh,
// moe_topk_sigmoid_kernels.cuh), moe_compute_index (moe_compute_index.cu:37-153) and moe_combine
// (moe_combine.cu:37-102).  The reference's CUDA path drops n_group / topk_group
// (ops_api.cpp:666-671); here group-limited routing (DeepSeek-V3) is implemented.
// Experts outside [expert_begin, expert_end) are not local to this rank (expert parallelism): their
// (token, k) pairs get row -1 and contribute nothing.
#include "common.cuh"

namespace xllm {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;
constexpr int kMoeTile = 128;

struct RouteParams {
  const void* logits;   // [T, E] bf16 or fp32
  const float* bias;    // [E] selection bias (e_score_correction_bias) or null
  int32_t* topk_ids;    // [T, K]
  float* topk_w;        // [T, K]
  int32_t* counts;      // [E] zeroed by the caller (or by moe_offsets of the previous call)
  int32_t* slot;        // [T, K] position of the pair inside its expert's segment
  int T, E, K, n_group, topk_group, scoring, renorm, logits_fp32, expert_begin, expert_end;
  float scale;
};

// one warp per token; lane l owns experts l, l+32, ...
__global__ void __launch_bounds__(128) moe_route_kernel(RouteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  pdl_wait();
  if (t >= p.T) return;
  constexpr int PER = kMaxExperts / 32;
  float score[PER], sel[PER];
  const int per = (p.E + 31) / 32;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    float v = -INFINITY;
    if (i < per && e < p.E)
      v = p.logits_fp32 ? reinterpret_cast<const float*>(p.logits)[(int64_t)t * p.E + e]
                        : __bfloat162float(reinterpret_cast<const bf16*>(p.logits)[(int64_t)t * p.E + e]);
    score[i] = v;
    mx = fmaxf(mx, v);
  }
  if (p.scoring == 0) {  // softmax
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      score[i] = (i < per && lane + i * 32 < p.E) ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) score[i] *= inv;
  } else {  // sigmoid
#pragma unroll
    for (int i = 0; i < PER; ++i) score[i] = (i < per && lane + i * 32 < p.E) ? 1.f / (1.f + __expf(-score[i])) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    sel[i] = (i < per && e < p.E) ? score[i] + (p.bias ? p.bias[e] : 0.f) : -INFINITY;
  }
  // group-limited routing: keep the topk_group groups with the largest (sum of top-2 | max) score
  if (p.n_group > 1 && p.topk_group < p.n_group) {
    const int gsz = p.E / p.n_group;
    float keep_thr_group[1];
    (void)keep_thr_group;
    // group score for every group, computed redundantly by all lanes through shuffles
    float gscore = -INFINITY;  // lane g (< n_group) holds group g's score
    for (int g = 0; g < p.n_group; ++g) {
      float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = lane + i * 32;
        if (i < per && e < p.E && e / gsz == g) {
          const float v = sel[i];
          if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v;
        }
      }
      // merge top-2 across lanes
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
        const float a = fmaxf(m1, o1);
        const float b = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
        m1 = a; m2 = b;
      }
      const float gs = p.bias ? m1 + (m2 > -INFINITY ? m2 : 0.f) : m1;
      if (lane == g) gscore = gs;
    }
    // rank of each group = number of groups with a strictly better score (ties: lower index wins)
    bool keep_group = false;
    {
      int better = 0;
      for (int g = 0; g < p.n_group; ++g) {
        const float og = __shfl_sync(0xffffffffu, gscore, g);
        if (lane < p.n_group && (og > gscore || (og == gscore && g < lane))) ++better;
      }
      keep_group = lane < p.n_group && better < p.topk_group;
    }
    const unsigned keep_mask = __ballot_sync(0xffffffffu, keep_group);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      if (i < per && e < p.E && !((keep_mask >> (e / gsz)) & 1u)) sel[i] = -INFINITY;
    }
  }
  // iterative top-k by warp arg-max over the selection scores
  float wsum = 0.f;
  float my_w[kMaxTopK];
  int my_id[kMaxTopK];
  for (int k = 0; k < p.K; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      if (i < per && e < p.E && (sel[i] > bv || (sel[i] == bv && e < be))) { bv = sel[i]; be = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // the owner lane supplies the un-biased score as the weight and retires the expert
    float w = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (lane + i * 32 == be) { w = score[i]; sel[i] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, be & 31);
    my_w[k] = w;
    my_id[k] = be;
    wsum += w;
  }
  const float norm = (p.renorm && wsum > 0.f) ? 1.f / wsum : 1.f;
  if (lane < p.K) {
    // lane k writes pair k
    float w = 0.f;
    int e = 0;
#pragma unroll
    for (int k = 0; k < kMaxTopK; ++k)
      if (k == lane && k < p.K) { w = my_w[k]; e = my_id[k]; }
    p.topk_ids[(int64_t)t * p.K + lane] = e;
    p.topk_w[(int64_t)t * p.K + lane] = w * norm * p.scale;
    int s = -1;
    if (e >= p.expert_begin && e < p.expert_end) s = atomicAdd(&p.counts[e], 1);
    p.slot[(int64_t)t * p.K + lane] = s;
  }
}

// offsets[e] = first row of expert e in the permuted buffer (multiple of 128); tile_expert[i] =
// expert of row tile i (or -1); counts are cleared for the next call; meta[0] = rows used.
__global__ void moe_offsets_kernel(int32_t* counts, int32_t* offsets, int32_t* tile_expert, int32_t* meta, int E,
                                   int max_tiles, int expert_begin) {
  __shared__ int s_off[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + kMoeTile - 1) / kMoeTile * kMoeTile;
    }
    s_off[E] = acc;
    meta[0] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    offsets[e] = s_off[e];
    const int t0 = s_off[e] / kMoeTile, t1 = s_off[e + 1] / kMoeTile;
    for (int i = t0; i < t1 && i < max_tiles; ++i) tile_expert[i] = e - expert_begin;  // index into the local weights
  }
  for (int i = s_off[E] / kMoeTile + threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
}

// xp[row(t,k), :] = x[t, :]; rows[t,k] = offsets[e] + slot (or -1 for non-local experts)
__global__ void __launch_bounds__(256)
moe_permute_kernel(bf16* __restrict__ xp, int32_t* __restrict__ rows, const bf16* __restrict__ x,
                   const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ slot,
                   const int32_t* __restrict__ offsets, int T, int K, int H) {
  const int pair = blockIdx.x;
  const int t = pair / K;
  const int s = slot[pair];
  int row = -1;
  if (s >= 0) row = offsets[topk_ids[pair]] + s;
  if (threadIdx.x == 0) rows[pair] = row;
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * H);
  uint4* dst = reinterpret_cast<uint4*>(xp + (int64_t)row * H);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = src[v];
}

__global__ void __launch_bounds__(256)
moe_finalize_kernel(bf16* __restrict__ out, const bf16* __restrict__ y, const int32_t* __restrict__ rows,
                    const float* __restrict__ w, const bf16* __restrict__ shared_out, int T, int K, int H) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float acc[8];
    if (shared_out) unpack8(reinterpret_cast<const bf16x8*>(shared_out + (int64_t)t * H)[v], acc);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const int row = rows[t * K + k];
      if (row < 0) continue;
      const float wk = w[t * K + k];
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(y + (int64_t)row * H)[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * f[j];
    }
    reinterpret_cast<bf16x8*>(out + (int64_t)t * H)[v] = pack8(acc);
  }
}

}  // namespace xllm

// scoring: 0 softmax, 1 sigmoid.  counts must be zero on entry (moe_offsets re-zeroes it).
XLLM_API int xllm_moe_route(const void* logits, int logits_fp32, const void* bias, void* topk_ids, void* topk_w,
                            void* counts, void* slot, int T, int E, int K, int n_group, int topk_group, int scoring,
                            int renorm, float scale, int expert_begin, int expert_end, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (E > kMaxExperts || K > kMaxTopK || K > 32 || n_group > 32 || (n_group > 1 && E % n_group != 0))
    return (int)cudaErrorInvalidValue;
  RouteParams p;
  p.logits = logits; p.bias = (const float*)bias; p.topk_ids = (int32_t*)topk_ids; p.topk_w = (float*)topk_w;
  p.counts = (int32_t*)counts; p.slot = (int32_t*)slot; p.T = T; p.E = E; p.K = K; p.n_group = n_group;
  p.topk_group = topk_group; p.scoring = scoring; p.renorm = renorm; p.logits_fp32 = logits_fp32;
  p.expert_begin = expert_begin; p.expert_end = expert_end; p.scale = scale;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, (cudaStream_t)stream>>>(p);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_moe_offsets(void* counts, void* offsets, void* tile_expert, void* meta, int E, int max_tiles,
                              int expert_begin, void* stream) {
  using namespace xllm;
  moe_offsets_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((int32_t*)counts, (int32_t*)offsets, (int32_t*)tile_expert,
                                                         (int32_t*)meta, E, max_tiles, expert_begin);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_moe_permute(void* xp, void* rows, const void* x, const void* topk_ids, const void* slot,
                              const void* offsets, int T, int K, int H, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  moe_permute_kernel<<<T * K, 256, 0, (cudaStream_t)stream>>>((bf16*)xp, (int32_t*)rows, (const bf16*)x,
                                                             (const int32_t*)topk_ids, (const int32_t*)slot,
                                                             (const int32_t*)offsets, T, K, H);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_moe_finalize(void* out, const void* y, const void* rows, const void* w, const void* shared_out,
                               int T, int K, int H, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  moe_finalize_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)y, (const int32_t*)rows,
                                                          (const float*)w, (const bf16*)shared_out, T, K, H);
  return XLLM_LAUNCH_CHECK();
}
