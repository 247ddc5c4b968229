// Small data-movement kernels: embedding gather, KV block copy, decode metadata update,
// row gather, token feedback.
//
// Parity: block_copy_kernel (xllm/core/kernels/cuda/block_copy.cu:67-207),
// llm_decode_metadata_update_kernel (llm_decode_metadata_update.cu:29-104) and the torch
// embedding / index_select calls of the reference forward path.
#include "common.cuh"

namespace xllm {

// out[t, :] = table[ids[t], :]   (ids outside [vocab_start, vocab_end) give zeros: vocab-parallel)
__global__ void __launch_bounds__(256)
embedding_kernel(bf16* __restrict__ out, const bf16* __restrict__ table,
                 const int64_t* __restrict__ ids, int64_t tokens, int hidden, int64_t vocab_start,
                 int64_t vocab_end) {
  const int vec = hidden >> 3;
  const int64_t total = tokens * vec;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec;
    const int v = (int)(i - t * vec);
    const int64_t id = ids[t];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (id >= vocab_start && id < vocab_end)
      val = reinterpret_cast<const uint4*>(table + (id - vocab_start) * hidden)[v];
    reinterpret_cast<uint4*>(out + t * hidden)[v] = val;
  }
}

// out[i, :] = in[idx[i], :]  (rows of `row_bytes` bytes, multiple of 16)
__global__ void __launch_bounds__(256)
gather_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ in,
                   const int64_t* __restrict__ idx, int64_t rows, int vec_per_row,
                   int64_t in_stride_vec) {
  const int64_t total = rows * vec_per_row;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int v = (int)(i - r * vec_per_row);
    out[i] = in[idx[r] * in_stride_vec + v];
  }
}

// Copy whole KV blocks src -> dst for `n_layers` caches given as a device pointer table.
// pairs: [n_pairs, 2] int32 (src block, dst block).  block_bytes % 16 == 0.
__global__ void __launch_bounds__(256)
block_copy_kernel(void* const* __restrict__ caches, const int32_t* __restrict__ pairs,
                  int64_t block_vec) {
  const int layer = blockIdx.z, pair = blockIdx.y;
  uint4* base = reinterpret_cast<uint4*>(caches[layer]);
  const int64_t src = pairs[2 * pair], dst = pairs[2 * pair + 1];
  const uint4* s = base + src * block_vec;
  uint4* d = base + dst * block_vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < block_vec;
       i += (int64_t)gridDim.x * blockDim.x)
    d[i] = s[i];
}

// One launch that refreshes every persistent decode-graph input for the next step:
//   tokens <- sampled ids of the previous step (device-resident feedback, no host round trip)
//   positions += 1, seq_lens += 1, slot = block_table[b, pos / page] * page + pos % page
// Rows with seq_lens[b] <= 0 are padding and stay untouched.
__global__ void decode_advance_kernel(int64_t* tokens, int64_t* positions, int32_t* seq_lens,
                                      int32_t* slots, const int32_t* block_table, int bt_stride,
                                      const int64_t* sampled, int batch, int page) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int len = seq_lens[b];
  if (len <= 0) return;
  tokens[b] = sampled[b];
  const int64_t pos = positions[b] + 1;
  positions[b] = pos;
  seq_lens[b] = len + 1;
  const int pg = (int)(pos / page);
  slots[b] = block_table[(int64_t)b * bt_stride + pg] * page + (int)(pos - (int64_t)pg * page);
}

// tokens[i] = sampled_prev[-tokens[i] - 1] for every negative entry (placeholders written by a
// scheduler that ran one step ahead of the device).
__global__ void resolve_placeholder_kernel(int64_t* tokens, const int64_t* prev, int64_t n,
                                           int64_t n_prev) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t t = tokens[i];
  if (t < 0) {
    const int64_t j = -t - 1;
    tokens[i] = j < n_prev ? prev[j] : 0;
  }
}

}  // namespace xllm

XLLM_API int xllm_embedding(void* out, const void* table, const void* ids, int64_t tokens,
                            int hidden, int64_t vocab_start, int64_t vocab_end, void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  if (hidden % 8 != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = tokens * (hidden >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  launch_pdl(embedding_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (bf16*)out, (const bf16*)table,
                                                          (const int64_t*)ids, tokens, hidden,
                                                          vocab_start, vocab_end);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_gather_rows(void* out, const void* in, const void* idx, int64_t rows,
                              int64_t row_bytes, int64_t in_stride_bytes, void* stream) {
  using namespace xllm;
  if (rows == 0) return 0;
  if (row_bytes % 16 != 0 || in_stride_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
  const int vec = (int)(row_bytes / 16);
  const int64_t total = rows * vec;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  launch_pdl(gather_rows_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, 
      (uint4*)out, (const uint4*)in, (const int64_t*)idx, rows, vec, in_stride_bytes / 16);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_block_copy(const void* cache_ptr_table, int n_layers, const void* pairs,
                             int n_pairs, int64_t block_bytes, void* stream) {
  using namespace xllm;
  if (n_pairs == 0 || n_layers == 0) return 0;
  if (block_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
  const int64_t vec = block_bytes / 16;
  int gx = (int)((vec + 255) / 256);
  if (gx > 64) gx = 64;
  dim3 grid(gx, n_pairs, n_layers);
  block_copy_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((void* const*)cache_ptr_table,
                                                           (const int32_t*)pairs, vec);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_decode_advance(void* tokens, void* positions, void* seq_lens, void* slots,
                                 const void* block_table, int bt_stride, const void* sampled,
                                 int batch, int page, void* stream) {
  using namespace xllm;
  if (batch == 0) return 0;
  decode_advance_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      (int64_t*)tokens, (int64_t*)positions, (int32_t*)seq_lens, (int32_t*)slots,
      (const int32_t*)block_table, bt_stride, (const int64_t*)sampled, batch, page);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_resolve_placeholders(void* tokens, const void* prev, int64_t n, int64_t n_prev,
                                       void* stream) {
  using namespace xllm;
  if (n == 0) return 0;
  resolve_placeholder_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (int64_t*)tokens, (const int64_t*)prev, n, n_prev);
  return XLLM_LAUNCH_CHECK();
}
