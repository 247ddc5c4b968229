// RMSNorm family for sm_100a (bf16 in/out, fp32 math).
//
// Parity: rms_norm / fused_add_rms_norm of the reference CUDA backend
// (xllm/core/kernels/cuda/norm.cu:43-174) and the static-fp8 variants (:228-415).
// Design: one CTA per token row, the row stays in registers between the
// sum-of-squares pass and the scale pass (one HBM read, one write); 128-bit
// vector accesses; rows are independent so the grid is simply `tokens`.
#include "common.cuh"
#include <cuda_fp8.h>

namespace xllm {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;  // 256 threads * 8 vec * 8 elems = hidden <= 16384 in registers

// out = rmsnorm(x [+ residual]) * w ;  if residual != null: residual = x + residual (in place)
// QUANT: 0 none, 1 static per-tensor e4m3 (scale = *qscale, out_q written instead of out)
template <int QUANT>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(bf16* __restrict__ out, uint8_t* __restrict__ out_q, const bf16* __restrict__ x,
               bf16* __restrict__ residual, const bf16* __restrict__ w, const float* qscale,
               int hidden, float eps, int64_t x_stride, int64_t out_stride, int gemma) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = hidden >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * x_stride);
  bf16x8* rr = residual ? reinterpret_cast<bf16x8*>(residual + row * (int64_t)hidden) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  float vals[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      unpack8(xr[v], vals[i]);
      if (rr) {
        float r[8];
        unpack8(rr[v], r);
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
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  float qs = 1.f;
  if (QUANT == 1) qs = 1.f / (*qscale);
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float wv[8];
      unpack8(wr[v], wv);
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * (gemma ? (1.f + wv[j]) : wv[j]);
      if (QUANT == 0) {
        reinterpret_cast<bf16x8*>(out + row * out_stride)[v] = pack8(o);
      } else {
        uint2 q;
        uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float t = fminf(fmaxf(o[j] * qs, -448.f), 448.f);
          qb[j] = (uint8_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
        }
        reinterpret_cast<uint2*>(out_q + row * out_stride)[v] = q;
      }
    }
  }
}

}  // namespace xllm

// x:[tokens, hidden] (row stride x_stride), out likewise (out_stride); residual (optional, in place)
// is dense [tokens, hidden]. hidden % 8 == 0 and hidden <= 16384.
XLLM_API int xllm_rmsnorm(void* out, const void* x, void* residual, const void* w, int tokens,
                          int hidden, float eps, int64_t x_stride, int64_t out_stride, int gemma,
                          void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (hidden % 8 != 0 || hidden > kNormThreads * kNormMaxVec * 8) return (int)cudaErrorInvalidValue;
  launch_pdl(rmsnorm_kernel<0>, dim3(tokens), dim3(kNormThreads), 0, (cudaStream_t)stream, 
      (bf16*)out, nullptr, (const bf16*)x, (bf16*)residual, (const bf16*)w, nullptr, hidden, eps,
      x_stride, out_stride, gemma);
  return XLLM_LAUNCH_CHECK();
}

// Same, but the normalised row is written as e4m3 with a static per-tensor scale (out_q = y / scale).
XLLM_API int xllm_rmsnorm_static_fp8(void* out_q, const void* x, void* residual, const void* w,
                                     const void* scale, int tokens, int hidden, float eps,
                                     void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (hidden % 8 != 0 || hidden > kNormThreads * kNormMaxVec * 8) return (int)cudaErrorInvalidValue;
  launch_pdl(rmsnorm_kernel<1>, dim3(tokens), dim3(kNormThreads), 0, (cudaStream_t)stream, 
      nullptr, (uint8_t*)out_q, (const bf16*)x, (bf16*)residual, (const bf16*)w,
      (const float*)scale, hidden, eps, hidden, hidden, 0);
  return XLLM_LAUNCH_CHECK();
}
