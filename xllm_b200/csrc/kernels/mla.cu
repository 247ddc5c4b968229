// Multi-head latent attention (MLA, DeepSeek-V2/V3) over a paged latent cache.
//
// The cache holds one row per token, shared by all heads: [c_kv (kv_lora = 512) | k_pe (64)] = 576
// bf16 values.  With the up-projections absorbed into the query (q_abs = q_nope . W_UK) and into the
// output (W_UV applied afterwards), attention over that cache is multi-QUERY attention with
//   score(h, t) = q[h, :576] . row[t, :576],   out[h, :512] = sum_t p(h, t) row[t, :512],
// i.e. one "KV head" of width 576 whose first 512 values double as V.  A decode step therefore reads
// 1152 bytes per cached token instead of nh * (192 + 128) * 2.
//
// Reference: the absorbed decode path of the DCU backend
// (xllm/core/layers/dcu/deepseek_v2_attention.cpp:242-433); the reference has no MLA on CUDA.
//
//   xllm_mla_cache_write : RMSNorm(c_kv) * w | RoPE(k_pe) -> cache row of the token's slot, and RoPE
//                          of the rotary part of every query head, in one pass over the token
//   xllm_mla_decode      : split-KV attention of N query rows (nh heads each) against the cache.
//                          A query row names its own visible length and block-table row, so decode
//                          tokens (one per sequence) and the tokens of prompt chunks (each sees the
//                          cache up to its own position) run through the same launch; nothing is
//                          read back to the host, so the launch can be captured in a CUDA graph.
//
// Work decomposition of the decode kernel: grid = (ceil(nh / 16), N, splits), 8 warps per CTA.  The
// 16 heads of a CTA are the M rows of m16n8k16 tiles.  Warps work in pairs: a pair owns a cp.async
// ring of 16-token tiles (one tile = 16 rows x 1152 bytes, contiguous in a page) and walks tiles
// pair, pair + 4, ...  Inside a pair the 576-wide dot product is cut in two (each warp multiplies 288
// columns, the halves meet through shared memory), and each warp accumulates 256 of the 512 output
// columns, which keeps the accumulators at 128 registers per thread.  The four pairs' (m, l, O) states
// are merged through shared memory at the end; splits > 1 write normalised partials for
// xllm_attn_merge.
#include "attn_common.cuh"
#include <atomic>

namespace xllm {
namespace mla {

constexpr int kDQK = 576;         // latent + rope width of a cache row
constexpr int kDV = 512;          // latent width (the part that is V)
constexpr int kCH = kDQK / 8;     // 16-byte chunks per row
constexpr int kTileBytes = 16 * kDQK * 2;
constexpr int kStages = 2;
constexpr int kPairs = 4;
constexpr int kThreads = kPairs * 64;
constexpr int kQBytes = kTileBytes;                               // 16 heads x 576
constexpr int kRingBytes = kPairs * kStages * kTileBytes;         // 147456
constexpr int kXchgBytes = kPairs * 2 * 256 * 4;                  // partial scores of the two halves
constexpr int kSmem = kQBytes + kRingBytes + kXchgBytes;

struct DecodeParams {
  const bf16* q;               // [N, nh, 576]
  const bf16* cache;           // [n_blocks, page, 576]
  const int32_t* block_table;  // [B, bt_stride]
  const int32_t* seq_lens;     // [N] tokens visible to the row, or null: positions[row] + 1
  const int64_t* positions;    // [N] (used when seq_lens is null)
  const int32_t* bt_rows;      // [N] block-table row of the query row, or null: identity
  bf16* out;                   // [N, nh, 512]
  float* o_part;               // [N, nh, splits, 512]
  float* lse_part;             // [N, nh, splits] (log2 domain)
  int64_t q_stride;            // elements between query rows
  int bt_stride, nh, page_size, splits;
  float scale_log2;
};

__device__ __forceinline__ void pair_sync(int pair) {
  asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

__global__ void __launch_bounds__(kThreads) mla_decode_kernel(DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = warp >> 1, half = warp & 1;
  const int qt = blockIdx.x, n = blockIdx.y, split = blockIdx.z;
  pdl_wait();
  pdl_launch_dependents();
  const int seq_len = p.seq_lens ? p.seq_lens[n] : (int)p.positions[n] + 1;
  const int tiles_total = (seq_len + 15) >> 4;
  const int tps = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = split * tps;
  const int t_end = min(t_begin + tps, tiles_total);
  const int my_n = (t_end - t_begin - pair + kPairs - 1) / kPairs;  // tiles of this pair (may be <= 0)
  const int rows_valid = min(16, p.nh - qt * 16);
  const int head0 = qt * 16;

  // ---- the 16 query rows go to shared memory once (rows beyond nh are zero)
  const uint32_t q_smem = smem_u32(smem);
  {
    const bf16* qb = p.q + (int64_t)n * p.q_stride + (int64_t)head0 * kDQK;
    for (int id = threadIdx.x; id < 16 * kCH; id += kThreads) {
      const int r = id / kCH, c = id - r * kCH;
      cp_async16(q_smem + swz<kCH>(r, c), qb + (int64_t)(r < rows_valid ? r : 0) * kDQK + c * 8, r < rows_valid);
    }
    cp_async_commit();
  }
  const uint32_t ring = q_smem + kQBytes + pair * (kStages * kTileBytes);
  float* xchg = reinterpret_cast<float*>(smem + kQBytes + kRingBytes) + pair * 512;
  const int32_t* bt = p.block_table + (int64_t)(p.bt_rows ? p.bt_rows[n] : n) * p.bt_stride;

  auto load_tile = [&](int i) {  // i-th tile of this pair -> stage i % kStages; both warps copy half of it
    if (i < my_n) {
      const int tok0 = (t_begin + pair + kPairs * i) << 4;
      const int page = tok0 / p.page_size;
      const int off = tok0 - page * p.page_size;
      const bf16* kb = p.cache + ((int64_t)bt[page] * p.page_size + off) * kDQK;
      const uint32_t dst = ring + (i % kStages) * kTileBytes;
#pragma unroll
      for (int j = 0; j < (16 * kCH) / 64; ++j) {
        const int id = (half * 32 + lane) + j * 64;
        const int r = id / kCH, c = id - r * kCH;
        const bool valid = tok0 + r < seq_len;
        cp_async16(dst + swz<kCH>(r, c), kb + (valid ? (int64_t)r * kDQK + c * 8 : 0), valid);
      }
    }
    cp_async_commit();
  };

  float o[kDV / 16][4];   // this warp's 256 output columns: 32 n8 tiles
#pragma unroll
  for (int i = 0; i < kDV / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  load_tile(0);
  cp_async_wait<1>();   // the query rows (the first group); tile 0 may still be in flight
  __syncthreads();      // they were copied by all warps of the CTA
  for (int i = 0; i < my_n; ++i) {
    cp_async_wait<0>();
    pair_sync(pair);               // tile i is complete; both warps are done with tile i - 1
    load_tile(i + 1);
    const uint32_t k_addr = ring + (i % kStages) * kTileBytes;
    const int tok0 = (t_begin + pair + kPairs * i) << 4;

    // ---- partial scores over this warp's half of the 576 columns (18 k-steps of 16)
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int brow = (lane & 7) + ((lane >> 4) << 3);
      const int bcb = (lane >> 3) & 1;
      const int arow = lane & 15, acb = lane >> 4;
#pragma unroll 6
      for (int ks = half * 18; ks < half * 18 + 18; ++ks) {
        uint32_t a[4], b0, b1, b2, b3;
        ldmatrix_x4(a[0], a[1], a[2], a[3], q_smem + swz<kCH>(arow, ks * 2 + acb));
        ldmatrix_x4(b0, b1, b2, b3, k_addr + swz<kCH>(brow, ks * 2 + bcb));
        mma_bf16_16816(s[0], a, b0, b1);
        mma_bf16_16816(s[1], a, b2, b3);
      }
    }
    // ---- the two halves meet: each warp publishes its partial tile and adds the other's
    {
      float* mine = xchg + half * 256;
      const float* other = xchg + (half ^ 1) * 256;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[(nt * 4 + j) * 32 + lane] = s[nt][j];
      pair_sync(pair);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[nt][j] += other[(nt * 4 + j) * 32 + lane];
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tok = tok0 + nt * 8 + (lane & 3) * 2 + (j & 1);
        float v = s[nt][j] * p.scale_log2;
        if (tok >= seq_len) v = -INFINITY;
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
    for (int i2 = 0; i2 < kDV / 16; ++i2) {
      o[i2][0] *= a0; o[i2][1] *= a0; o[i2][2] *= a1; o[i2][3] *= a1;
    }
    uint32_t pa[4];
    pa[0] = pack_bf162(s[0][0], s[0][1]);
    pa[1] = pack_bf162(s[0][2], s[0][3]);
    pa[2] = pack_bf162(s[1][0], s[1][1]);
    pa[3] = pack_bf162(s[1][2], s[1][3]);
    {
      // V = the first 512 columns of the same tile; this warp takes columns [256 half, 256 half + 256)
      const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int cb = lane >> 4;
#pragma unroll
      for (int jn = 0; jn < kDV / 32; ++jn) {
        uint32_t v0, v1, v2, v3;
        ldmatrix_x4_trans(v0, v1, v2, v3, k_addr + swz<kCH>(row, (half * (kDV / 32) + jn) * 2 + cb));
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
  __syncthreads();  // every pair is done with its ring; reuse it for the merge

  float* sm_m = reinterpret_cast<float*>(smem + kQBytes);  // [4][16]
  float* sm_l = sm_m + 64;                                 // [4][16]
  float* sm_o = sm_l + 64;                                 // [4][16][512]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    if (half == 0 && (lane & 3) == 0) {
      sm_m[pair * 16 + r0] = m0; sm_m[pair * 16 + r1] = m1;
      sm_l[pair * 16 + r0] = l0; sm_l[pair * 16 + r1] = l1;
    }
#pragma unroll
    for (int nt = 0; nt < kDV / 16; ++nt) {
      const int col = half * (kDV / 2) + nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(sm_o + (pair * 16 + r0) * kDV + col) = make_float2(o[nt][0], o[nt][1]);
      *reinterpret_cast<float2*>(sm_o + (pair * 16 + r1) * kDV + col) = make_float2(o[nt][2], o[nt][3]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_valid * kDV; idx += kThreads) {
    const int r = idx / kDV, d = idx - r * kDV;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPairs; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
    float acc = 0.f, L = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kPairs; ++w) {
        const float wgt = exp2f(sm_m[w * 16 + r] - M);
        acc += sm_o[(w * 16 + r) * kDV + d] * wgt;
        L += sm_l[w * 16 + r] * wgt;
      }
    }
    const float val = L > 0.f ? acc / L : 0.f;
    const int64_t head = (int64_t)n * p.nh + head0 + r;
    if (p.splits == 1) {
      p.out[head * kDV + d] = __float2bfloat16(val);
    } else {
      p.o_part[(head * p.splits + split) * kDV + d] = val;
      if (d == 0) p.lse_part[head * p.splits + split] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
}

}  // namespace mla
}  // namespace xllm

namespace xllm {
namespace mla {

// One CTA per token: cache row = [rmsnorm(c_kv) * w | rope(k_pe)], and rope of every head's rotary
// query part.  RoPE acts on adjacent pairs (x[2i], x[2i+1]) with cos_sin[pos] = [cos(rot/2) | sin(rot/2)].
struct WriteParams {
  const bf16* kv_a;        // [T, 576] (row stride kv_stride): c_kv | k_pe, straight from the projection
  const bf16* norm_w;      // [512]
  const float* cos_sin;    // [max_pos, rot]
  const int64_t* positions;
  const int32_t* slots;    // [T], -1: no cache write
  bf16* cache;             // rows of 576
  const bf16* q_rope_in;   // rotary part of head 0 of token 0; head stride q_in_hs, token stride q_in_ts
  bf16* q_out;             // [T, nh, 576]: the rotary part lands in columns [512, 576)
  int64_t kv_stride, q_in_ts, q_in_hs;
  int nh;
  float eps;
};

__global__ void __launch_bounds__(128) mla_cache_write_kernel(WriteParams p) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  constexpr int ROT = kDQK - kDV;   // 64
  pdl_wait();
  pdl_launch_dependents();
  const int64_t pos = p.positions[t];
  const float* cs = p.cos_sin + pos * ROT;
  const int slot = p.slots ? p.slots[t] : -1;
  const bf16* row = p.kv_a + t * p.kv_stride;
  // ---- latent part: 64 threads x 8 values
  float v[8];
  float ss = 0.f;
  if (threadIdx.x < 64) {
    unpack8(reinterpret_cast<const bf16x8*>(row)[threadIdx.x], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  }
  ss = block_sum(ss, red);
  if (slot >= 0) {
    bf16* dst = p.cache + (int64_t)slot * kDQK;
    if (threadIdx.x < 64) {
      const float inv = rsqrtf(ss / (float)kDV + p.eps);
      float w[8], o[8];
      unpack8(reinterpret_cast<const bf16x8*>(p.norm_w)[threadIdx.x], w);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[j] * inv * w[j];
      reinterpret_cast<bf16x8*>(dst)[threadIdx.x] = pack8(o);
    } else if (threadIdx.x < 64 + ROT / 2) {
      const int i = threadIdx.x - 64;
      const float x1 = __bfloat162float(row[kDV + 2 * i]), x2 = __bfloat162float(row[kDV + 2 * i + 1]);
      const float c = cs[i], sn = cs[ROT / 2 + i];
      *reinterpret_cast<bf162*>(dst + kDV + 2 * i) = __floats2bfloat162_rn(x1 * c - x2 * sn, x2 * c + x1 * sn);
    }
  }
  // ---- rotary part of the queries
  if (p.q_out != nullptr) {
    for (int id = threadIdx.x; id < p.nh * (ROT / 2); id += blockDim.x) {
      const int h = id / (ROT / 2), i = id - h * (ROT / 2);
      const bf16* src = p.q_rope_in + t * p.q_in_ts + (int64_t)h * p.q_in_hs;
      const float x1 = __bfloat162float(src[2 * i]), x2 = __bfloat162float(src[2 * i + 1]);
      const float c = cs[i], sn = cs[ROT / 2 + i];
      *reinterpret_cast<bf162*>(p.q_out + (t * p.nh + h) * kDQK + kDV + 2 * i) =
          __floats2bfloat162_rn(x1 * c - x2 * sn, x2 * c + x1 * sn);
    }
  }
}

}  // namespace mla
}  // namespace xllm

extern "C" int xllm_attn_merge(void* out, const void* o_part, const void* lse_part, int64_t rows, int splits, int d,
                               void* stream);

// fp32 elements of workspace xllm_mla_decode needs for `splits` > 1 (0 otherwise).
XLLM_API int64_t xllm_mla_decode_workspace(int64_t n_rows, int nh, int splits) {
  return splits > 1 ? n_rows * nh * splits * (int64_t)(xllm::mla::kDV + 1) : 0;
}

// out [N, nh, 512] = absorbed-MLA attention of query rows q [N, nh, 576] (row stride q_stride
// elements) over the latent cache [n_blocks, page, 576].  seq_lens [N] int32: tokens visible to each
// row; when null, positions [N] int64 gives it as position + 1 (rows of a prompt chunk).  bt_rows [N]
// int32: block-table row of each query row (null: row n uses table row n).  page_size % 16 == 0.
// workspace: xllm_mla_decode_workspace() floats when splits > 1.
XLLM_API int xllm_mla_decode(void* out, const void* q, int64_t q_stride, const void* cache, const void* block_table,
                             int bt_stride, const void* seq_lens, const void* positions, const void* bt_rows,
                             int n_rows, int nh, int page_size, float scale, int splits, void* workspace,
                             void* stream) {
  using namespace xllm;
  using namespace xllm::mla;
  if (n_rows == 0) return 0;
  if (nh <= 0 || page_size <= 0 || page_size % 16 != 0 || splits < 1 || (seq_lens == nullptr && positions == nullptr) ||
      (splits > 1 && workspace == nullptr) || q_stride % 8 || (((uintptr_t)q | (uintptr_t)cache) & 15))
    return (int)cudaErrorInvalidValue;
  static std::atomic<bool> attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63].store(true, std::memory_order_release);
  }
  DecodeParams p;
  p.q = (const bf16*)q; p.cache = (const bf16*)cache; p.block_table = (const int32_t*)block_table;
  p.seq_lens = (const int32_t*)seq_lens; p.positions = (const int64_t*)positions; p.bt_rows = (const int32_t*)bt_rows;
  p.out = (bf16*)out; p.q_stride = q_stride; p.bt_stride = bt_stride; p.nh = nh; p.page_size = page_size;
  p.splits = splits; p.scale_log2 = scale * 1.4426950408889634f;
  p.o_part = splits > 1 ? (float*)workspace : nullptr;
  p.lse_part = p.o_part ? p.o_part + (int64_t)n_rows * nh * splits * kDV : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  launch_pdl(mla_decode_kernel, dim3((nh + 15) / 16, n_rows, splits), dim3(kThreads), (size_t)kSmem, s, p);
  int rc = XLLM_LAUNCH_CHECK();
  if (rc != 0 || splits == 1) return rc;
  return xllm_attn_merge(out, p.o_part, p.lse_part, (int64_t)n_rows * nh, splits, kDV, stream);
}

// Latent-cache write fused with the rotary embeddings of a step's tokens (see the kernel's comment).
// kv_a [T, 576] bf16 (row stride kv_stride), norm_w [512], cos_sin fp32 [max_pos, 64], positions [T]
// int64, slots [T] int32 (-1: skip the write; null: no cache write at all), cache rows of 576 bf16.
// q_rope_in: address of the rotary part of (token 0, head 0) of the query projection, with token and
// head strides in elements; q_out [T, nh, 576] receives it in columns [512, 576).  q_out may be null.
XLLM_API int xllm_mla_cache_write(const void* kv_a, int64_t kv_stride, const void* norm_w, float eps,
                                  const void* cos_sin, const void* positions, const void* slots, void* cache,
                                  const void* q_rope_in, int64_t q_in_ts, int64_t q_in_hs, void* q_out, int T, int nh,
                                  void* stream) {
  using namespace xllm;
  using namespace xllm::mla;
  if (T == 0) return 0;
  if (kv_stride % 8 || ((uintptr_t)kv_a & 15) || ((uintptr_t)cache & 15)) return (int)cudaErrorInvalidValue;
  WriteParams p;
  p.kv_a = (const bf16*)kv_a; p.norm_w = (const bf16*)norm_w; p.cos_sin = (const float*)cos_sin;
  p.positions = (const int64_t*)positions; p.slots = (const int32_t*)slots; p.cache = (bf16*)cache;
  p.q_rope_in = (const bf16*)q_rope_in; p.q_out = (bf16*)q_out; p.kv_stride = kv_stride; p.q_in_ts = q_in_ts;
  p.q_in_hs = q_in_hs; p.nh = nh; p.eps = eps;
  launch_pdl(mla_cache_write_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, p);
  return XLLM_LAUNCH_CHECK();
}
