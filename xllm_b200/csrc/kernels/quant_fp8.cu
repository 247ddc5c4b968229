// fp8 (e4m3) quantisation kernels.
//
//   quant_fp8_per_token  : dynamic per-row scale (amax / 448) or a static per-tensor scale
//   quant_fp8_group128   : per-token 1 x 128 group scales (DeepSeek-style activation quantisation)
//   dequant_fp8_block128 : 128 x 128 block-scaled weights -> bf16
//
// Parity: scaled_fp8_quant / fp8_scaled_quantize of the reference (xllm/core/kernels/cuda/fp8_quant.cu:78-151,
// fp8_scaled_quantize.cpp:20-48).  The reference has no block-scaled path on CUDA
// (cutlass_w8a8/scaled_mm_c3x_sm100.cu:34-44); the group / block kernels here are what lets 128x128
// block-scaled checkpoints be loaded and run.
#include "common.cuh"
#include <cuda_fp8.h>

namespace xllm {

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(v, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}

// one CTA per row; static_scale != null => q = x / *static_scale, no scale output
__global__ void __launch_bounds__(256)
quant_per_token_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const bf16* __restrict__ x,
                       const float* __restrict__ static_scale, int H, int64_t x_stride) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * x_stride);
  const int nvec = H >> 3;
  float inv;
  if (static_scale != nullptr) {
    inv = 1.f / *static_scale;
  } else {
    float amax = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
    amax = block_max(amax, red);
    const float s = fmaxf(amax, 1e-10f) / 448.f;
    if (threadIdx.x == 0) scales[row] = s;
    inv = 1.f / s;
  }
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(xr[v], f);
    uint2 o;
    uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) ob[j] = to_e4m3(f[j] * inv);
    reinterpret_cast<uint2*>(q + row * (int64_t)H)[v] = o;
  }
}

// one warp per (row, 128-wide group): 16 lanes x 8 elements
__global__ void __launch_bounds__(256)
quant_group128_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const bf16* __restrict__ x, int64_t T,
                      int H, int64_t x_stride) {
  const int groups = H >> 7;
  const int64_t g = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);  // 16 groups per CTA
  const int l = threadIdx.x & 15;
  const bool active = g < T * groups;
  const int64_t row = active ? g / groups : 0;
  const int gi = active ? (int)(g - row * groups) : 0;
  float f[8];
  if (active) unpack8(reinterpret_cast<const bf16x8*>(x + row * x_stride + gi * 128)[l], f);
  else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(amax, 1e-10f) / 448.f;
  if (!active) return;
  if (l == 0) scales[row * groups + gi] = s;
  const float inv = 1.f / s;
  uint2 o;
  uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
  for (int j = 0; j < 8; ++j) ob[j] = to_e4m3(f[j] * inv);
  reinterpret_cast<uint2*>(q + row * (int64_t)H + gi * 128)[l] = o;
}

// w[n, k] = q[n, k] * scales[n / 128, k / 128]
__global__ void __launch_bounds__(256)
dequant_block128_kernel(bf16* __restrict__ w, const uint8_t* __restrict__ q, const float* __restrict__ scales,
                        int64_t N, int K, int sk) {
  const int kvec = K >> 3;
  const int64_t total = N * kvec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / kvec;
    const int kv = (int)(i - n * kvec);
    const float s = scales[(n >> 7) * sk + ((kv * 8) >> 7)];
    const uint2 v = reinterpret_cast<const uint2*>(q + n * K)[kv];
    const uint8_t* vb = reinterpret_cast<const uint8_t*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = from_e4m3(vb[j]) * s;
    reinterpret_cast<bf16x8*>(w + n * K)[kv] = pack8(f);
  }
}

}  // namespace xllm

XLLM_API int xllm_quant_fp8_per_token(void* q, void* scales, const void* x, const void* static_scale, int64_t T, int H,
                                      int64_t x_stride, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  quant_per_token_kernel<<<(unsigned)T, 256, 0, (cudaStream_t)stream>>>((uint8_t*)q, (float*)scales, (const bf16*)x,
                                                                       (const float*)static_scale, H, x_stride);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_quant_fp8_group128(void* q, void* scales, const void* x, int64_t T, int H, int64_t x_stride,
                                     void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 128) return (int)cudaErrorInvalidValue;
  const int64_t groups = T * (H / 128);
  quant_group128_kernel<<<(unsigned)((groups + 15) / 16), 256, 0, (cudaStream_t)stream>>>(
      (uint8_t*)q, (float*)scales, (const bf16*)x, T, H, x_stride);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_dequant_fp8_block128(void* w, const void* q, const void* scales, int64_t N, int K, void* stream) {
  using namespace xllm;
  if (N == 0) return 0;
  if (K % 8) return (int)cudaErrorInvalidValue;
  dequant_block128_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((bf16*)w, (const uint8_t*)q, (const float*)scales,
                                                                    N, K, (K + 127) / 128);
  return XLLM_LAUNCH_CHECK();
}
