// Paged GQA decode attention (one query token per sequence), split-KV + merge.
//
// Covers the reference's two decode routes — FlashInfer CUDA-core `batch_decode` for GQA group < 4
// and tensor-core `batch_chunked_prefill` used as decode for group >= 4
// (xllm/core/kernels/cuda/batch_decode.cpp:26-86, batch_chunked_prefill.cpp:26-92,
// layers/cuda/flashinfer_attention.cpp:224-337) — with one kernel and no host-side plan step:
// the split count is a launch parameter and every CTA derives its KV range from seq_lens on the
// device, so the launch is CUDA-graph safe.
//
// Work decomposition (decode is HBM-bound: 4 flop/byte at group 4):
//   grid = (kv_heads * ceil(group/16), batch, splits); 4 warps per CTA.
//   Each warp owns a private cp.async ring of 16-token K/V tiles (a tile of one kv head is one
//   contiguous 16*D*2-byte run in the [block, kv_head, slot, D] cache) and walks tiles
//   warp, warp+4, ... of the CTA's range with no CTA-wide barrier in the loop; the 4 partial
//   (m, l, O) states are merged through shared memory at the end.
//   The `group` query heads that share a kv head form the M rows of an m16n8k16 tile.
// Scratch: when splits > 1 the normalised partial outputs and their log2-sum-exp go to
// caller-provided fp32 workspaces and `xllm_attn_merge` combines them.
#include "attn_common.cuh"
#include <atomic>

namespace xllm {

struct DecodeParams {
  const bf16* q;        // [B, nq, D]
  const bf16* k_cache;  // [n_blocks, nkv, page, D]
  const bf16* v_cache;
  const int32_t* block_table;  // [B, bt_stride]
  const int32_t* seq_lens;     // [B]  kv length including the current token
  bf16* out;                   // [B, nq, D]
  float* o_part;               // [B, nq, splits, D]
  float* lse_part;             // [B, nq, splits]   (log2 domain)
  int64_t q_stride;            // elements between sequences in q
  int bt_stride, nq, nkv, group, page_size, splits;
  int window;                  // 0 = attend to the whole sequence
  float scale_log2;
};

template <int D, int STAGES>
__global__ void __launch_bounds__(128) paged_decode_kernel(DecodeParams p) {
  constexpr int CH = D / 8;               // 16-byte chunks per row
  constexpr int TILE_BYTES = 16 * D * 2;  // one 16-token K (or V) tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int KS = D / 16;
  extern __shared__ __align__(128) uint8_t smem[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qtiles = (p.group + 15) >> 4;
  const int kvh = blockIdx.x / qtiles, qt = blockIdx.x - kvh * qtiles;
  const int b = blockIdx.y, split = blockIdx.z;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  const int seq_len = p.seq_lens[b];
  // sliding window: only the last `window` positions take part; tiles before them are never
  // touched (their cache blocks may have been given back already)
  const int win_start = p.window > 0 ? max(0, seq_len - p.window) : 0;
  const int tile_first = win_start >> 4;
  const int tiles_total = (seq_len + 15) >> 4;
  const int tps = (tiles_total - tile_first + p.splits - 1) / p.splits;
  const int t_begin = tile_first + split * tps;
  const int t_end = min(t_begin + tps, tiles_total);
  const int my_n = (t_end - t_begin - warp + 3) >> 2;  // tiles of this warp (may be <= 0)
  const int rows_valid = min(16, p.group - qt * 16);
  const int head0 = kvh * p.group + qt * 16;

  // ---- Q fragments (A operand), rows beyond the group are zero
  uint32_t qa[KS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const bf16* qb = p.q + (int64_t)b * p.q_stride + (int64_t)head0 * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int col = ks * 16 + (lane & 3) * 2;
      qa[ks][0] = r0 < rows_valid ? *reinterpret_cast<const uint32_t*>(qb + r0 * D + col) : 0u;
      qa[ks][1] = r1 < rows_valid ? *reinterpret_cast<const uint32_t*>(qb + r1 * D + col) : 0u;
      qa[ks][2] = r0 < rows_valid ? *reinterpret_cast<const uint32_t*>(qb + r0 * D + col + 8) : 0u;
      qa[ks][3] = r1 < rows_valid ? *reinterpret_cast<const uint32_t*>(qb + r1 * D + col + 8) : 0u;
    }
  }

  const uint32_t ring = smem_u32(smem) + warp * (STAGES * STAGE_BYTES);
  const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;

  auto load_tile = [&](int i) {  // i-th tile of this warp -> stage i % STAGES
    if (i < my_n) {
      const int tok0 = (t_begin + warp + 4 * i) << 4;
      const int page = tok0 / p.page_size;
      const int off = tok0 - page * p.page_size;
      const int64_t blk = bt[page];
      const int64_t base = ((blk * p.nkv + kvh) * p.page_size + off) * (int64_t)D;
      const bf16* kb = p.k_cache + base;
      const bf16* vb = p.v_cache + base;
      const uint32_t ks = ring + (i % STAGES) * STAGE_BYTES;
      const uint32_t vs = ks + TILE_BYTES;
#pragma unroll
      for (int j = 0; j < (16 * CH) / 32; ++j) {
        const int id = lane + j * 32;
        const int r = id / CH, c = id - r * CH;
        const bool valid = tok0 + r < seq_len && tok0 + r >= win_start;
        const int64_t go = valid ? (int64_t)r * D + c * 8 : 0;
        cp_async16(ks + swz<CH>(r, c), kb + go, valid);
        cp_async16(vs + swz<CH>(r, c), vb + go, valid);
      }
    }
    cp_async_commit();
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) load_tile(s);

  for (int i = 0; i < my_n; ++i) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    // the stage consumed in the previous iteration is free: refill it
    load_tile(i + STAGES - 1);
    const uint32_t ks_addr = ring + (i % STAGES) * STAGE_BYTES;
    const uint32_t vs_addr = ks_addr + TILE_BYTES;
    const int tok0 = (t_begin + warp + 4 * i) << 4;

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int row = (lane & 7) + ((lane >> 4) << 3);
      const int cb = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks_addr + swz<CH>(row, ks * 2 + cb));
        mma_bf16_16816(s[0], qa[ks], b0, b1);
        mma_bf16_16816(s[1], qa[ks], b2, b3);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tok = tok0 + nt * 8 + (lane & 3) * 2 + (j & 1);
        float v = s[nt][j] * p.scale_log2;
        if (tok >= seq_len || tok < win_start) v = -INFINITY;
        s[nt][j] = v;
        if (j < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - mn0); s[nt][1] = exp2f(s[nt][1] - mn0);
      s[nt][2] = exp2f(s[nt][2] - mn1); s[nt][3] = exp2f(s[nt][3] - mn1);
      rs0 += s[nt][0] + s[nt][1];
      rs1 += s[nt][2] + s[nt][3];
    }
    l0 = l0 * a0 + rs0;
    l1 = l1 * a1 + rs1;
#pragma unroll
    for (int i2 = 0; i2 < D / 8; ++i2) {
      o[i2][0] *= a0; o[i2][1] *= a0; o[i2][2] *= a1; o[i2][3] *= a1;
    }
    uint32_t pa[4];
    pa[0] = pack_bf162(s[0][0], s[0][1]);
    pa[1] = pack_bf162(s[0][2], s[0][3]);
    pa[2] = pack_bf162(s[1][0], s[1][1]);
    pa[3] = pack_bf162(s[1][2], s[1][3]);
    {
      const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int cb = lane >> 4;
#pragma unroll
      for (int jn = 0; jn < D / 16; ++jn) {
        uint32_t v0, v1, v2, v3;
        ldmatrix_x4_trans(v0, v1, v2, v3, vs_addr + swz<CH>(row, jn * 2 + cb));
        mma_bf16_16816(o[jn * 2], pa, v0, v1);
        mma_bf16_16816(o[jn * 2 + 1], pa, v2, v3);
      }
    }
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();  // every warp is done with its ring; reuse it for the merge

  float* sm_m = reinterpret_cast<float*>(smem);  // [4][16]
  float* sm_l = sm_m + 64;                       // [4][16]
  float* sm_o = sm_l + 64;                       // [4][16][D]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    if ((lane & 3) == 0) {
      sm_m[warp * 16 + r0] = m0; sm_m[warp * 16 + r1] = m1;
      sm_l[warp * 16 + r0] = l0; sm_l[warp * 16 + r1] = l1;
    }
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const int col = nt * 8 + (lane & 3) * 2;
      if (r0 < rows_valid)
        *reinterpret_cast<float2*>(sm_o + (warp * 16 + r0) * D + col) = make_float2(o[nt][0], o[nt][1]);
      if (r1 < rows_valid)
        *reinterpret_cast<float2*>(sm_o + (warp * 16 + r1) * D + col) = make_float2(o[nt][2], o[nt][3]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_valid * D; idx += 128) {
    const int r = idx / D, d = idx - r * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
    float acc = 0.f, L = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float wgt = exp2f(sm_m[w * 16 + r] - M);
        acc += sm_o[(w * 16 + r) * D + d] * wgt;
        L += sm_l[w * 16 + r] * wgt;
      }
    }
    const float val = L > 0.f ? acc / L : 0.f;
    const int64_t head = (int64_t)b * p.nq + head0 + r;
    if (p.splits == 1) {
      p.out[head * D + d] = __float2bfloat16(val);
    } else {
      p.o_part[(head * p.splits + split) * D + d] = val;
      if (d == 0) p.lse_part[head * p.splits + split] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
}

// out[row, :] = sum_s o_part[row, s, :] * 2^(lse[row, s] - max) / sum_s 2^(lse[row, s] - max)
__global__ void attn_merge_kernel(bf16* __restrict__ out, const float* __restrict__ o_part,
                                  const float* __restrict__ lse, int splits, int D) {
  const int64_t row = blockIdx.x;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, lse[row * splits + s]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
    if (M > -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float w = exp2f(lse[row * splits + s] - M);
        acc += o_part[(row * splits + s) * D + d] * w;
        L += w;
      }
    }
    out[row * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
  }
}

template <int D, int STAGES>
static int launch_decode(const DecodeParams& p, int batch, cudaStream_t s) {
  constexpr int SMEM = 4 * STAGES * 2 * 16 * D * 2;
  static std::atomic<bool> attr_done[64] = {};   // first calls from several host threads may coincide
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<D, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63].store(true, std::memory_order_release);
  }
  const int qtiles = (p.group + 15) / 16;
  dim3 grid(p.nkv * qtiles, batch, p.splits);
  launch_pdl(paged_decode_kernel<D, STAGES>, dim3(grid), dim3(128), SMEM, s, p);
  return XLLM_LAUNCH_CHECK();
}

}  // namespace xllm

// Number of bytes of fp32 scratch the split path needs: o_part then lse_part.
XLLM_API int64_t xllm_decode_attn_workspace_bytes(int batch, int nq, int d, int splits) {
  if (splits <= 1) return 0;
  return (int64_t)batch * nq * splits * (d + 1) * 4;
}

// q:[B,nq,D] (q_stride elements between sequences), caches [n_blocks, nkv, page, D], out:[B,nq,D] dense.
// workspace: fp32 scratch of xllm_decode_attn_workspace_bytes() bytes when splits > 1 (else may be null).
static int decode_attn_impl(void* out, const void* q, int64_t q_stride, const void* k_cache,
                            const void* v_cache, const void* block_table, int bt_stride,
                            const void* seq_lens, int batch, int nq, int nkv, int d,
                            int page_size, float scale, int splits, void* workspace, int window,
                            void* stream) {
  using namespace xllm;
  if (batch == 0) return 0;
  if (nq % nkv != 0 || page_size % 16 != 0 || splits < 1 || window < 0) return (int)cudaErrorInvalidValue;
  if (splits > 1 && workspace == nullptr) return (int)cudaErrorInvalidValue;
  DecodeParams p;
  p.q = (const bf16*)q; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_table = (const int32_t*)block_table; p.seq_lens = (const int32_t*)seq_lens;
  p.out = (bf16*)out; p.q_stride = q_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv;
  p.group = nq / nkv; p.page_size = page_size; p.splits = splits; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o_part = (float*)workspace;
  p.lse_part = p.o_part ? p.o_part + (int64_t)batch * nq * splits * d : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (d == 128) rc = launch_decode<128, 3>(p, batch, s);
  else if (d == 64) rc = launch_decode<64, 4>(p, batch, s);
  else if (d == 256) rc = launch_decode<256, 2>(p, batch, s);
  else return (int)cudaErrorInvalidValue;
  if (rc != 0 || splits == 1) return rc;
  launch_pdl(attn_merge_kernel, dim3(batch * nq), dim3(d < 128 ? d : 128), 0, s, p.out, p.o_part, p.lse_part, splits, d);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_paged_decode_attn(void* out, const void* q, int64_t q_stride, const void* k_cache,
                                    const void* v_cache, const void* block_table, int bt_stride,
                                    const void* seq_lens, int batch, int nq, int nkv, int d,
                                    int page_size, float scale, int splits, void* workspace,
                                    void* stream) {
  return decode_attn_impl(out, q, q_stride, k_cache, v_cache, block_table, bt_stride, seq_lens, batch, nq, nkv, d,
                          page_size, scale, splits, workspace, 0, stream);
}

// The same with a sliding window: every query attends to its last `window` positions only, and the
// block-table entries of pages entirely before the window are never read.
XLLM_API int xllm_paged_decode_attn_window(void* out, const void* q, int64_t q_stride, const void* k_cache,
                                           const void* v_cache, const void* block_table, int bt_stride,
                                           const void* seq_lens, int batch, int nq, int nkv, int d,
                                           int page_size, float scale, int splits, void* workspace,
                                           int window, void* stream) {
  return decode_attn_impl(out, q, q_stride, k_cache, v_cache, block_table, bt_stride, seq_lens, batch, nq, nkv, d,
                          page_size, scale, splits, workspace, window, stream);
}

// Standalone merge of `splits` normalised partials (also used by context-parallel decode).
XLLM_API int xllm_attn_merge(void* out, const void* o_part, const void* lse_part, int64_t rows,
                             int splits, int d, void* stream) {
  using namespace xllm;
  if (rows == 0) return 0;
  launch_pdl(attn_merge_kernel, dim3((unsigned)rows), dim3(d < 128 ? d : 128), 0, (cudaStream_t)stream, 
      (bf16*)out, (const float*)o_part, (const float*)lse_part, splits, d);
  return XLLM_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in no_alloc.h, which states who needs it and the contract).
// The split-KV partials live in this file-scope array instead of a caller-provided workspace.
#include "no_alloc.h"
#include <atomic>
#include <cstdio>

namespace xllm {
static __device__ __align__(256) unsigned char g_noalloc_scratch[XLLM_NO_ALLOC_SCRATCH_BYTES];
// Device address of the array, per device.  In host code `g_noalloc_scratch` is only a handle of
// the symbol — passing it to a kernel would hand the GPU a host address — so the address is
// resolved once per device with cudaGetSymbolAddress and cached here.
// Published with release / read with acquire: two host threads may make their first call on a device
// at the same time; both would store the same address.
static std::atomic<float*> g_noalloc_ptr[64] = {};
static thread_local char g_noalloc_msg[192] = "";
}  // namespace xllm

XLLM_API const char* xllm_no_alloc_last_error(void) { return xllm::g_noalloc_msg; }

XLLM_API int xllm_paged_decode_attn_noalloc(void* out, const void* q, int64_t q_stride, const void* k_cache,
                                            const void* v_cache, const void* block_table, int bt_stride,
                                            const void* seq_lens, int batch, int nq, int nkv, int d,
                                            int page_size, float scale, int splits, void* stream) {
  using namespace xllm;
  g_noalloc_msg[0] = 0;
  if (batch == 0) return 0;
  // every argument is checked before the first CUDA call
  if (batch < 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || page_size % 16 != 0 || splits < 1 ||
      (d != 64 && d != 128 && d != 256)) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "bad argument: batch %d, heads %d / %d, head_dim %d (64, 128 or 256), page %d, splits %d", batch, nq, nkv,
             d, page_size, splits);
    return (int)cudaErrorInvalidValue;
  }
  const long long need = splits > 1 ? (long long)batch * nq * splits * (d + 1) * 4 : 0;
  if (need > (long long)XLLM_NO_ALLOC_SCRATCH_BYTES) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "decode attention needs %lld bytes of split-KV scratch (batch %d x heads %d x splits %d), the "
             "built-in array holds %u; lower `splits` or the batch",
             need, batch, nq, splits, (unsigned)XLLM_NO_ALLOC_SCRATCH_BYTES);
    return XLLM_NO_ALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "no current CUDA device (or device index >= 64)");
    return XLLM_NO_ALLOC_SETUP_FAILED;
  }
  float* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // set-up, once per device, with that device current.  With CUDA's lazy module loading this is
    // also the moment the driver loads the kernel image and gives the array its device memory.
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return XLLM_NO_ALLOC_SETUP_FAILED;
    }
    scratch = static_cast<float*>(p);
    g_noalloc_ptr[dev].store(scratch, std::memory_order_release);
  }
  DecodeParams p;
  p.q = (const bf16*)q; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_table = (const int32_t*)block_table; p.seq_lens = (const int32_t*)seq_lens;
  p.out = (bf16*)out; p.q_stride = q_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv;
  p.group = nq / nkv; p.page_size = page_size; p.splits = splits; p.window = 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o_part = splits > 1 ? scratch : nullptr;
  p.lse_part = p.o_part ? p.o_part + (int64_t)batch * nq * splits * d : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (d == 128) rc = launch_decode<128, 3>(p, batch, s);
  else if (d == 64) rc = launch_decode<64, 4>(p, batch, s);
  else if (d == 256) rc = launch_decode<256, 2>(p, batch, s);
  else return (int)cudaErrorInvalidValue;
  if (rc != 0 || splits == 1) return rc;
  launch_pdl(attn_merge_kernel, dim3(batch * nq), dim3(d < 128 ? d : 128), 0, s, p.out, p.o_part, p.lse_part, splits, d);
  return XLLM_LAUNCH_CHECK();
}
