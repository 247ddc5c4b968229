// Row-wise helpers for kernels that keep one hidden-state row in the registers of a group of
// threads (RMSNorm family, the fused tensor-parallel reductions).
//
// A CTA of 256 threads is cut into groups of TPR threads (32, 64, 128 or 256); a group owns one row,
// thread t of the group owns the 16-byte vectors t, t + TPR, t + 2 TPR, ... (at most kRowMaxVec of
// them), so a warp reads 512 contiguous bytes per vector index and a CTA keeps 256 / TPR rows in
// flight.  The group size is the smallest one whose threads can hold the row: narrow rows get many
// rows per CTA (more bytes in flight per SM), wide rows still fit.
#pragma once
#include "common.cuh"

namespace xllm {

constexpr int kRowThreads = 256;
constexpr int kRowMaxVec = 8;  // vectors of 8 bf16 per thread -> hidden <= TPR * 64

// smallest thread-group size that holds a row of `hidden` bf16 values; 0 when none does
inline int row_group_threads(int hidden) {
  const int nvec = hidden >> 3;
  for (int tpr = 32; tpr <= kRowThreads; tpr <<= 1)
    if (nvec <= tpr * kRowMaxVec) return tpr;
  return 0;
}

// Sum over the TPR threads of a group.  Every thread of the CTA must call it (it synchronises the
// CTA when a group spans several warps); `red` is shared memory for 8 floats.
template <int TPR>
__device__ __forceinline__ float group_sum(float v, float* red) {
  v = warp_sum(v);
  if constexpr (TPR == 32) {
    return v;
  } else {
    constexpr int W = TPR / 32;
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    const int g = wid / W * W;
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < W; ++i) r += red[g + i];
    return r;
  }
}

}  // namespace xllm
