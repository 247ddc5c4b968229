// Beam attention for fixed-step generative recommendation ("x-attention"): the beams of a request share
// the prompt's KV and differ only in the few tokens they generated.
//
// Parity: xllm/core/kernels/cuda/xattention/{decoder_reshape_and_cache,cache_select,lse_combine}.cu and
// core/layers/cuda/xattention.cpp — there the beams' KV lives in a [request, beam, step] tensor that is
// reordered in place after every beam step, and the two attention partials are combined by a third kernel.
//
// Here the two stages are
//   1. shared stage: the beams of a request are the query rows of ONE non-causal pass of the tcgen05 prefill
//      kernel over the prompt's pages (attn_prefill_tc.cu, with its log-sum-exp output), so the prompt's KV
//      is read once per 128 beams and the scores run on the tensor cores;
//   2. this file: one warp per (beam row, query head) scores the row's own tail of <= kTailMax generated
//      tokens, merges it with the shared stage by log-sum-exp and writes the final output in place.
// The tail cache never moves: a beam finds its ancestors' rows through `anc[t][row]` (the row that held the
// beam's ancestor at step t), which the host-side beam step re-gathers (a few KB) instead of reordering KV.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace xllm {
namespace {

constexpr int kTailMax = 8;

template <int N>
struct alignas(2 * N) BfVec {
  __nv_bfloat16 v[N];
};

template <int N>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float* f) {
  const BfVec<N> t = *reinterpret_cast<const BfVec<N>*>(p);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = __bfloat162float(t.v[i]);
}

template <int D>
__global__ void __launch_bounds__(128)
xattn_tail_merge_kernel(__nv_bfloat16* __restrict__ out, int64_t o_stride, const float* __restrict__ lse,
                        const __nv_bfloat16* __restrict__ q, int64_t q_stride, const __nv_bfloat16* __restrict__ ku,
                        const __nv_bfloat16* __restrict__ vu, const int32_t* __restrict__ anc, int anc_stride,
                        int n_tail, int rows, int nq, int nkv, int tail_cap, float scale_log2) {
  constexpr int PER = D / 32;                         // values per lane
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= rows * nq) return;
  const int row = gw / nq, h = gw % nq;
  const int hk = h / (nq / nkv);
  float qv[PER];
  {
    load_vec<PER>(q + (int64_t)row * q_stride + h * D + lane * PER, qv);
  }
  // scores of the tail tokens (log2 domain)
  float s[kTailMax];
  int src[kTailMax];
  float m = lse[(int64_t)row * nq + h];               // -inf when the prompt gave this row nothing
#pragma unroll
  for (int t = 0; t < kTailMax; ++t) {
    s[t] = -INFINITY;
    src[t] = 0;
    if (t < n_tail) {
      int r = anc[t * anc_stride + row];
      r = r < 0 ? 0 : r;
      src[t] = r;
      const __nv_bfloat16* kp = ku + (((int64_t)r * nkv + hk) * tail_cap + t) * D + lane * PER;
      float kv[PER], acc = 0.f;
      load_vec<PER>(kp, kv);
#pragma unroll
      for (int i = 0; i < PER; ++i) acc += qv[i] * kv[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      s[t] = acc * scale_log2;
      m = fmaxf(m, s[t]);
    }
  }
  const float l_shared = lse[(int64_t)row * nq + h];
  const float w_shared = (l_shared == -INFINITY) ? 0.f : exp2f(l_shared - m);
  float total = w_shared;
  float acc[PER];
  __nv_bfloat16* op = out + (int64_t)row * o_stride + h * D + lane * PER;
  load_vec<PER>(op, acc);
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = w_shared > 0.f ? w_shared * acc[i] : 0.f;
#pragma unroll
  for (int t = 0; t < kTailMax; ++t) {
    if (t < n_tail) {
      const float w = exp2f(s[t] - m);
      total += w;
      const __nv_bfloat16* vp = vu + (((int64_t)src[t] * nkv + hk) * tail_cap + t) * D + lane * PER;
      float vv[PER];
      load_vec<PER>(vp, vv);
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] += w * vv[i];
    }
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
  BfVec<PER> res;
#pragma unroll
  for (int i = 0; i < PER; ++i) res.v[i] = __float2bfloat16(acc[i] * inv);
  *reinterpret_cast<BfVec<PER>*>(op) = res;
}

}  // namespace
}  // namespace xllm

// out [rows, nq, d] bf16 holds the shared-stage result on entry and the merged result on return; lse
// [rows, nq] fp32 is the shared stage's log2-domain log-sum-exp.  ku / vu [tail_rows, nkv, tail_cap, d] hold
// the generated tokens' K / V: token t of the beam in `row` lives in row anc[t * anc_stride + row].
XLLM_API int xllm_xattn_tail_merge(void* out, int64_t o_stride, const void* lse, const void* q, int64_t q_stride,
                                   const void* ku, const void* vu, const void* anc, int anc_stride, int n_tail, int rows,
                                   int nq, int nkv, int d, int tail_cap, float scale, void* stream) {
  using namespace xllm;
  if (rows == 0) return 0;
  if (n_tail < 0 || n_tail > kTailMax || n_tail > tail_cap || nq % nkv != 0 || o_stride % 8 || q_stride % 8 ||
      (((uintptr_t)out | (uintptr_t)q | (uintptr_t)ku | (uintptr_t)vu) & 15))
    return (int)cudaErrorInvalidValue;
  const int warps = rows * nq;
  dim3 grid((warps + 3) / 4), block(128);
  const float sl2 = scale * 1.4426950408889634f;
  auto s = (cudaStream_t)stream;
#define XATTN_LAUNCH(D)                                                                                          \
  xattn_tail_merge_kernel<D><<<grid, block, 0, s>>>((__nv_bfloat16*)out, o_stride, (const float*)lse,             \
                                                   (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)ku,  \
                                                   (const __nv_bfloat16*)vu, (const int32_t*)anc, anc_stride,    \
                                                   n_tail, rows, nq, nkv, tail_cap, sl2)
  if (d == 64) XATTN_LAUNCH(64);
  else if (d == 128) XATTN_LAUNCH(128);
  else if (d == 256) XATTN_LAUNCH(256);
  else return (int)cudaErrorInvalidValue;
#undef XATTN_LAUNCH
  return XLLM_LAUNCH_CHECK();
}
