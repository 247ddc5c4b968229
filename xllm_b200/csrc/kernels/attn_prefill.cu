// Variable-length causal GQA attention over the paged KV cache (prefill and chunked prefill).
//
// One kernel covers the reference's `batch_prefill` (ragged K/V) and `batch_chunked_prefill`
// (paged K/V) routes (xllm/core/kernels/cuda/batch_prefill.cpp:21-229,
// batch_chunked_prefill.cpp:26-92): K/V of the new tokens are already in the cache (written by
// the fused rope/KV-write kernel), so a prompt chunk simply attends to cache positions
// [0, kv_len) with the causal frontier shifted by kv_len - q_len.  No host-side plan.
//
// grid = (max q tiles of 64 rows, q heads, sequences); 4 warps, 16 query rows each; K/V tiles of
// 64 tokens double-buffered through cp.async; online softmax in registers.
#include "attn_common.cuh"

namespace xllm {

struct PrefillParams {
  const bf16* q;       // [T, nq, D]
  bf16* out;           // [T, nq, D]
  const bf16* k_cache; // [n_blocks, nkv, page, D]
  const bf16* v_cache;
  const int32_t* block_table;  // [B, bt_stride]
  const int32_t* cu_q;         // [B+1] query start offsets
  const int32_t* kv_lens;      // [B]
  int64_t q_stride;            // elements between tokens in q
  int64_t o_stride;
  int bt_stride, nq, nkv, page_size, causal, window;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(128) paged_prefill_kernel(PrefillParams p) {
  constexpr int CH = D / 8;
  constexpr int BM = 64, BN = 64;
  constexpr int KS = D / 16;
  constexpr int Q_BYTES = BM * D * 2;
  constexpr int KV_TILE = BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sq = smem_u32(smem);
  const uint32_t sk = sq + Q_BYTES;           // 2 stages
  const uint32_t sv = sk + 2 * KV_TILE;       // 2 stages

  const int b = blockIdx.z, h = blockIdx.y;
  const int group = p.nq / p.nkv;
  const int kvh = h / group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int q_start = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_start;
  const int kv_len = p.kv_lens[b];
  const int tile = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int m0 = tile * BM;
  if (m0 >= q_len) return;
  const int shift = kv_len - q_len;  // query i sits at cache position shift + i
  int kv_end = p.causal ? min(kv_len, shift + m0 + BM) : kv_len;
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, shift + m0 - p.window + 1) & ~(BN - 1);
  const int n_tiles = (kv_end - kv_begin + BN - 1) / BN;
  const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;

  // Q tile -> smem
  {
    const bf16* qb = p.q + (int64_t)(q_start + m0) * p.q_stride + (int64_t)h * D;
#pragma unroll
    for (int j = 0; j < (BM * CH) / 128; ++j) {
      const int id = threadIdx.x + j * 128;
      const int r = id / CH, c = id - r * CH;
      const bool valid = m0 + r < q_len;
      cp_async16(sq + swz<CH>(r, c), qb + (valid ? (int64_t)r * p.q_stride + c * 8 : 0), valid);
    }
  }
  auto load_kv = [&](int it) {
    const int n0 = kv_begin + it * BN;
    const uint32_t ks = sk + (it & 1) * KV_TILE, vs = sv + (it & 1) * KV_TILE;
#pragma unroll
    for (int j = 0; j < (BN * CH) / 128; ++j) {
      const int id = threadIdx.x + j * 128;
      const int r = id / CH, c = id - r * CH;
      const int tok = n0 + r;
      const bool valid = tok < kv_len;
      int64_t go = 0;
      if (valid) {
        const int page = tok / p.page_size;
        const int off = tok - page * p.page_size;
        go = (((int64_t)bt[page] * p.nkv + kvh) * p.page_size + off) * (int64_t)D + c * 8;
      }
      cp_async16(ks + swz<CH>(r, c), p.k_cache + go, valid);
      cp_async16(vs + swz<CH>(r, c), p.v_cache + go, valid);
    }
    cp_async_commit();
  };
  load_kv(0);  // group 0 = Q + first K/V tile

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mr0 = -INFINITY, mr1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  uint32_t qa[KS][4];
  const int qrow0 = m0 + warp * 16 + (lane >> 2);  // query index (within the sequence chunk) of row r0
  const int qpos0 = shift + qrow0, qpos1 = qpos0 + 8;

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) {
      load_kv(it + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
      const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int cb = lane >> 4;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], sq + swz<CH>(row, ks * 2 + cb));
    }
    const uint32_t ks_addr = sk + (it & 1) * KV_TILE, vs_addr = sv + (it & 1) * KV_TILE;
    const int n0 = kv_begin + it * BN;

    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int rr = (lane & 7) + ((lane >> 4) << 3);
      const int cb = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, ks_addr + swz<CH>(np * 16 + rr, ks * 2 + cb));
          mma_bf16_16816(s[np * 2], qa[ks], b0, b1);
          mma_bf16_16816(s[np * 2 + 1], qa[ks], b2, b3);
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tok = n0 + nt * 8 + (lane & 3) * 2 + (j & 1);
        const int qpos = j < 2 ? qpos0 : qpos1;
        float v = s[nt][j] * p.scale_log2;
        bool masked = tok >= kv_len;
        if (p.causal) masked |= tok > qpos;
        if (p.window > 0) masked |= tok <= qpos - p.window;
        if (masked) v = -INFINITY;
        s[nt][j] = v;
        if (j < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(mr0, mx0), mn1 = fmaxf(mr1, mx1);
    // a row with nothing visible so far keeps m = -inf; use 0 as the reference to avoid inf-inf
    const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    const float a0 = exp2f(mr0 - ref0), a1 = exp2f(mr1 - ref1);
    mr0 = mn0; mr1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - ref0); s[nt][1] = exp2f(s[nt][1] - ref0);
      s[nt][2] = exp2f(s[nt][2] - ref1); s[nt][3] = exp2f(s[nt][3] - ref1);
      rs0 += s[nt][0] + s[nt][1];
      rs1 += s[nt][2] + s[nt][3];
    }
    l0 = l0 * a0 + rs0;
    l1 = l1 * a1 + rs1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
    }
    {
      const int rr = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int cb = lane >> 4;
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf162(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf162(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf162(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf162(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int jn = 0; jn < D / 16; ++jn) {
          uint32_t v0, v1, v2, v3;
          ldmatrix_x4_trans(v0, v1, v2, v3, vs_addr + swz<CH>(kk * 16 + rr, jn * 2 + cb));
          mma_bf16_16816(o[jn * 2], pa, v0, v1);
          mma_bf16_16816(o[jn * 2 + 1], pa, v2, v3);
        }
      }
    }
    __syncthreads();  // the stage just read is refilled at the top of the next iteration
  }
  pdl_launch_dependents();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = qrow0, r1 = qrow0 + 8;
  bf16* ob = p.out + (int64_t)q_start * p.o_stride + (int64_t)h * D;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + (lane & 3) * 2;
    if (r0 < q_len)
      *reinterpret_cast<uint32_t*>(ob + (int64_t)r0 * p.o_stride + col) = pack_bf162(o[nt][0] * i0, o[nt][1] * i0);
    if (r1 < q_len)
      *reinterpret_cast<uint32_t*>(ob + (int64_t)r1 * p.o_stride + col) = pack_bf162(o[nt][2] * i1, o[nt][3] * i1);
  }
}

template <int D>
static int launch_prefill(const PrefillParams& p, int batch, int max_q_len, cudaStream_t s) {
  constexpr int SMEM = 64 * D * 2 + 4 * 64 * D * 2;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  dim3 grid((max_q_len + 63) / 64, p.nq, batch);
  paged_prefill_kernel<D><<<grid, 128, SMEM, s>>>(p);
  return XLLM_LAUNCH_CHECK();
}

}  // namespace xllm

// q/out: [T, nq, D] with q_stride / o_stride elements between tokens.  cu_q:[B+1], kv_lens:[B].
// causal: query i of a sequence sees cache positions <= kv_len - q_len + i.  window > 0 adds a
// sliding window of that many positions (including the current one).
XLLM_API int xllm_paged_prefill_attn(void* out, int64_t o_stride, const void* q, int64_t q_stride,
                                     const void* k_cache, const void* v_cache,
                                     const void* block_table, int bt_stride, const void* cu_q,
                                     const void* kv_lens, int batch, int max_q_len, int nq, int nkv,
                                     int d, int page_size, float scale, int causal, int window,
                                     void* stream) {
  using namespace xllm;
  if (batch == 0 || max_q_len == 0) return 0;
  if (nq % nkv != 0) return (int)cudaErrorInvalidValue;
  PrefillParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.k_cache = (const bf16*)k_cache;
  p.v_cache = (const bf16*)v_cache; p.block_table = (const int32_t*)block_table;
  p.cu_q = (const int32_t*)cu_q; p.kv_lens = (const int32_t*)kv_lens; p.q_stride = q_stride;
  p.o_stride = o_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
  p.causal = causal; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  if (d == 128) return launch_prefill<128>(p, batch, max_q_len, s);
  if (d == 64) return launch_prefill<64>(p, batch, max_q_len, s);
  if (d == 256) return launch_prefill<256>(p, batch, max_q_len, s);
  return (int)cudaErrorInvalidValue;
}
