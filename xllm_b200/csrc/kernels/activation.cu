// Gated activations: out[t, :d] = act(x[t, :d]) * x[t, d:2d]   (bf16, fp32 math)
//
// Parity: act_and_mul_kernel (silu/gelu/gelu_tanh) of the reference
// (xllm/core/kernels/cuda/activation.cu:45-159).  Flat grid over 16-byte
// vectors so that small token counts still fill the 148 SMs.
#include "common.cuh"

namespace xllm {

__device__ __forceinline__ float act_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float act_gelu(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678f)); }
__device__ __forceinline__ float act_gelu_tanh(float x) {
  const float k = 0.7978845608f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}

template <int ACT>
__global__ void __launch_bounds__(256)
act_and_mul_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, int64_t tokens, int d,
                   int64_t x_stride, const int32_t* __restrict__ n_rows_dev) {
  const int vec_per_row = d >> 3;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  // the number of rows that hold data may live on the device (expert-parallel receive buffers: the
  // launch is sized for the capacity, the work for what arrived)
  if (n_rows_dev != nullptr) tokens = min(tokens, (int64_t)*n_rows_dev);
  const int64_t total = tokens * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);
    const bf16x8* row = reinterpret_cast<const bf16x8*>(x + t * x_stride);
    float a[8], b[8], o[8];
    unpack8(row[v], a);
    unpack8(row[v + vec_per_row], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = ACT == 0 ? act_silu(a[j]) : (ACT == 1 ? act_gelu(a[j]) : act_gelu_tanh(a[j]));
      o[j] = g * b[j];
    }
    reinterpret_cast<bf16x8*>(out + t * (int64_t)d)[v] = pack8(o);
  }
}

// The same for the interleaved gate|up layout of a fused gate_up projection: every group of 128 input
// columns is [gate of 64 features | up of the same 64 features] (the layout whose GEMM can apply the
// activation in its epilogue, see xllm_gemm_bf16_act_mul).
template <int ACT>
__global__ void __launch_bounds__(256)
act_and_mul_il_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, int64_t tokens, int d, int64_t x_stride) {
  const int vec_per_row = d >> 3;
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = tokens * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);             // output vector: features v*8 .. v*8+7
    const int vin = (v >> 3) * 16 + (v & 7);              // 8 vectors of gate, then 8 of up, per 64 features
    const bf16x8* row = reinterpret_cast<const bf16x8*>(x + t * x_stride);
    float a[8], b[8], o[8];
    unpack8(row[vin], a);
    unpack8(row[vin + 8], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = ACT == 0 ? act_silu(a[j]) : (ACT == 1 ? act_gelu(a[j]) : act_gelu_tanh(a[j]));
      o[j] = g * b[j];
    }
    reinterpret_cast<bf16x8*>(out + t * (int64_t)d)[v] = pack8(o);
  }
}

}  // namespace xllm

// Interleaved layout (groups of 128 columns = 64 gate | 64 up); d % 64 == 0.
XLLM_API int xllm_act_and_mul_interleaved(void* out, const void* x, int64_t tokens, int d, int64_t x_stride, int act,
                                          void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (d % 64 != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = tokens * (d >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  cudaStream_t s = (cudaStream_t)stream;
  if (act == 0) launch_pdl(act_and_mul_il_kernel<0>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride);
  else if (act == 1) launch_pdl(act_and_mul_il_kernel<1>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride);
  else launch_pdl(act_and_mul_il_kernel<2>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride);
  return XLLM_LAUNCH_CHECK();
}

// act: 0 silu, 1 gelu(erf), 2 gelu(tanh).  x:[tokens, 2d] with row stride x_stride, out:[tokens, d].
XLLM_API int xllm_act_and_mul(void* out, const void* x, int64_t tokens, int d, int64_t x_stride,
                              int act, void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (d % 8 != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = tokens * (d >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  cudaStream_t s = (cudaStream_t)stream;
  const int32_t* none = nullptr;
  if (act == 0) launch_pdl(act_and_mul_kernel<0>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride, none);
  else if (act == 1) launch_pdl(act_and_mul_kernel<1>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride, none);
  else launch_pdl(act_and_mul_kernel<2>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, tokens, d, x_stride, none);
  return XLLM_LAUNCH_CHECK();
}

// Same over the first min(max_tokens, *n_rows) rows, n_rows a device int32: for buffers sized for a
// capacity of which only a prefix is in use (the count is not known on the host).
XLLM_API int xllm_act_and_mul_rows(void* out, const void* x, int64_t max_tokens, const void* n_rows, int d,
                                   int64_t x_stride, int act, void* stream) {
  using namespace xllm;
  if (max_tokens == 0) return 0;
  if (d % 8 != 0 || n_rows == nullptr) return (int)cudaErrorInvalidValue;
  const int grid = 148 * 8;
  cudaStream_t s = (cudaStream_t)stream;
  const int32_t* nr = (const int32_t*)n_rows;
  if (act == 0) launch_pdl(act_and_mul_kernel<0>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, max_tokens, d, x_stride, nr);
  else if (act == 1) launch_pdl(act_and_mul_kernel<1>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, max_tokens, d, x_stride, nr);
  else launch_pdl(act_and_mul_kernel<2>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, max_tokens, d, x_stride, nr);
  return XLLM_LAUNCH_CHECK();
}
