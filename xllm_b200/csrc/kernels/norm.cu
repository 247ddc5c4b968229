// RMSNorm family for sm_100a (bf16 in, fp32 math; bf16 or e4m3 out).
//
// Parity: rms_norm / fused_add_rms_norm of the reference CUDA backend
// (xllm/core/kernels/cuda/norm.cu:43-174) and the static-fp8 variants (:228-415); the variant that
// emits e4m3 with one scale per 128 columns (the activation format of 128x128 block-scaled fp8
// checkpoints) has no counterpart there.
// Design: a row lives in the registers of a group of 32..256 threads between the sum-of-squares pass
// and the scale pass (one HBM read, one write); a CTA of 256 threads holds 256 / group rows at once
// so that an SM keeps tens of KB of loads in flight even for narrow rows; 128-bit accesses.
#include "rowops.cuh"
#include <cuda_fp8.h>

namespace xllm {

__device__ __forceinline__ uint8_t norm_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(v, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
}

// out = rmsnorm(x [+ residual]) * w ;  if residual != null: residual = x + residual (in place)
// QUANT: 0 bf16 out; 1 e4m3 out with the static per-tensor scale *qscale (out_q = y / scale);
//        2 e4m3 out with one dynamic scale per (row, 128 columns): scales[row, hidden / 128]
template <int TPR, int QUANT>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_kernel(bf16* __restrict__ out, uint8_t* __restrict__ out_q, float* __restrict__ scales,
               const bf16* __restrict__ x, bf16* __restrict__ residual, const bf16* __restrict__ w,
               const float* qscale, int tokens, int hidden, float eps, int64_t x_stride, int64_t out_stride,
               int gemma) {
  __shared__ float red[8];
  constexpr int R = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int64_t row = (int64_t)blockIdx.x * R + threadIdx.x / TPR;
  const bool active = row < tokens;
  const int nvec = hidden >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * x_stride);
  bf16x8* rr = residual ? reinterpret_cast<bf16x8*>(residual + row * (int64_t)hidden) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  // every load of the row is issued before the first store: a store to the residual would otherwise
  // fence the loads behind it (the compiler cannot prove that x and residual do not overlap)
  uint4 rx[kRowMaxVec], rr_in[kRowMaxVec];
#pragma unroll
  for (int i = 0; i < kRowMaxVec; ++i) {
    const int v = t + i * TPR;
    if (active && v < nvec) {
      rx[i] = *reinterpret_cast<const uint4*>(xr + v);
      if (rr) rr_in[i] = *reinterpret_cast<const uint4*>(rr + v);
    }
  }
  float vals[kRowMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kRowMaxVec; ++i) {
    const int v = t + i * TPR;
    if (active && v < nvec) {
      unpack8(*reinterpret_cast<const bf16x8*>(&rx[i]), vals[i]);
      if (rr) {
        float r[8];
        unpack8(*reinterpret_cast<const bf16x8*>(&rr_in[i]), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
        // the residual stream is kept in bf16: round once here so that the norm sees
        // exactly what the next layer will read back
        bf16x8 p = pack8(vals[i]);
        rr[v] = p;
        unpack8(p, vals[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  ss = group_sum<TPR>(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  float qs = 1.f;
  if (QUANT == 1) qs = 1.f / (*qscale);
#pragma unroll
  for (int i = 0; i < kRowMaxVec; ++i) {
    const int v = t + i * TPR;
    const bool on = active && v < nvec;
    float o[8];
    if (on) {
      float wv[8];
      unpack8(wr[v], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * (gemma ? (1.f + wv[j]) : wv[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
    }
    if (QUANT == 0) {
      if (on) reinterpret_cast<bf16x8*>(out + row * out_stride)[v] = pack8(o);
    } else {
      if (QUANT == 2) {
        // 128 columns = 16 consecutive vectors = 16 consecutive lanes: quantise what the bf16
        // output would have held, with the group's own scale
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = __bfloat162float(__float2bfloat16(o[j]));
          amax = fmaxf(amax, fabsf(o[j]));
        }
#pragma unroll
        for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        const float sc = fmaxf(amax, 1e-10f) / 448.f;
        qs = 1.f / sc;
        if (on && (v & 15) == 0) scales[row * (hidden >> 7) + (v >> 4)] = sc;
      }
      if (on) {
        uint2 q;
        uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) qb[j] = norm_to_e4m3(o[j] * qs);
        reinterpret_cast<uint2*>(out_q + row * out_stride)[v] = q;
      }
    }
  }
}

template <int QUANT>
static int launch_rmsnorm(bf16* out, uint8_t* out_q, float* scales, const bf16* x, bf16* residual, const bf16* w,
                          const float* qscale, int tokens, int hidden, float eps, int64_t x_stride,
                          int64_t out_stride, int gemma, cudaStream_t s) {
  // The thread group of a row depends on the row width only, never on the number of rows: the order of the
  // sum-of-squares reduction, and so every rounded output, is then the same whatever batch a row arrives in
  // (spreading a row over more threads for small batches gains ~4 us per launch at 256 rows but makes a request's
  // tokens depend on the batch it shares).
  const int tpr = row_group_threads(hidden);
  if (hidden % 8 != 0 || tpr == 0) return (int)cudaErrorInvalidValue;
  const int rows = kRowThreads / tpr;
  const dim3 grid((unsigned)((tokens + rows - 1) / rows)), block(kRowThreads);
#define XLLM_NORM_CASE(T)                                                                                       \
  case T:                                                                                                       \
    launch_pdl(rmsnorm_kernel<T, QUANT>, grid, block, 0, s, out, out_q, scales, x, residual, w, qscale, tokens, \
               hidden, eps, x_stride, out_stride, gemma);                                                       \
    break;
  switch (tpr) {
    XLLM_NORM_CASE(32)
    XLLM_NORM_CASE(64)
    XLLM_NORM_CASE(128)
    XLLM_NORM_CASE(256)
  }
#undef XLLM_NORM_CASE
  return XLLM_LAUNCH_CHECK();
}

}  // namespace xllm

// x:[tokens, hidden] (row stride x_stride), out likewise (out_stride); residual (optional, in place)
// is dense [tokens, hidden]. hidden % 8 == 0 and hidden <= 16384.
XLLM_API int xllm_rmsnorm(void* out, const void* x, void* residual, const void* w, int tokens,
                          int hidden, float eps, int64_t x_stride, int64_t out_stride, int gemma,
                          void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  return launch_rmsnorm<0>((bf16*)out, nullptr, nullptr, (const bf16*)x, (bf16*)residual, (const bf16*)w, nullptr,
                           tokens, hidden, eps, x_stride, out_stride, gemma, (cudaStream_t)stream);
}

// Same, but the normalised row is written as e4m3 with a static per-tensor scale (out_q = y / scale).
XLLM_API int xllm_rmsnorm_static_fp8(void* out_q, const void* x, void* residual, const void* w,
                                     const void* scale, int tokens, int hidden, float eps,
                                     void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  return launch_rmsnorm<1>(nullptr, (uint8_t*)out_q, nullptr, (const bf16*)x, (bf16*)residual, (const bf16*)w,
                           (const float*)scale, tokens, hidden, eps, hidden, hidden, 0, (cudaStream_t)stream);
}

// Same, but the normalised row is written as e4m3 with one dynamic scale per 128 columns:
// out_q [tokens, hidden] (dense), scales [tokens, hidden / 128] fp32 (scale = group amax / 448).
// hidden % 128 == 0.
XLLM_API int xllm_rmsnorm_group_fp8(void* out_q, void* scales, const void* x, void* residual, const void* w,
                                    int tokens, int hidden, float eps, int64_t x_stride, int gemma, void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (hidden % 128 != 0) return (int)cudaErrorInvalidValue;
  return launch_rmsnorm<2>(nullptr, (uint8_t*)out_q, (float*)scales, (const bf16*)x, (bf16*)residual,
                           (const bf16*)w, nullptr, tokens, hidden, eps, x_stride, hidden, gemma,
                           (cudaStream_t)stream);
}
