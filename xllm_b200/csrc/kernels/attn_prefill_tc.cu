// Varlen causal prefill attention over the paged KV cache on the 5th-generation tensor cores.
//
// One CTA = (sequence, query head, tile of 128 query tokens), head_dim 128, 320 threads:
//   warp 0      TMA producer: the Q tile once, then K and V tiles of 128 tokens into a two-stage
//               shared-memory ring; a tile is gathered page by page through the block table (one
//               [page x 64]-element box per page and half of the head dimension)
//   warp 1      MMA issuer: S = Q K^T (tcgen05.mma, both operands K-major) into one of two S
//               accumulators in TMEM; then, once the softmax warps have written P, O_tile = P V
//               with V as an MN-major operand (the cache keeps head_dim contiguous), into one of two
//               O accumulators.  QK of tile j+1 is issued before PV of tile j, so the tensor pipe
//               works while the softmax of tile j runs.
//   warps 2-9   softmax: two threads per query row, 64 columns each (tcgen05.ld gives a thread its
//               own row; the two halves exchange their row maximum through shared memory); P goes to
//               shared memory as bf16 in the 128-byte swizzled K-major layout; the finished O tile
//               of the previous step is added with the usual rescaling O = (O + O_tile) * alpha.
// The reference reaches the same op through FlashInfer's fa2 kernels
// (xllm/core/kernels/cuda/flashinfer_attention.cpp:239-301); the mma.sync kernel of attn_prefill.cu
// stays as the path for other head sizes, sliding windows and small pages.
//
// Every mbarrier wait is bounded; on expiry all roles leave, TMEM is released and an error word
// is set (xllm_fmha_error_status).
#include "common.cuh"
#include <cuda.h>

namespace xllm {
namespace fmha {

constexpr int kD = 128;
constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // kv tokens per tile
constexpr int kHalf = kBM * 128;          // bytes of one [128 rows x 64 elements] swizzled half tile
constexpr int kTile = 2 * kHalf;          // 32 KB: a [128 x 128] bf16 operand tile
constexpr long long kWaitBudget = 4000000000LL;

constexpr int Q_OFF = 0;
constexpr int KV_OFF = kTile;                       // 2 stages x (K, V)
constexpr int P_OFF = KV_OFF + 4 * kTile;
constexpr int BAR_OFF = P_OFF + kTile;
constexpr int XCH_OFF = BAR_OFF + 24 * 8 + 16;          // row-max / row-sum exchange between the two halves of a row
constexpr int SMEM_TOTAL = XCH_OFF + (2 * 2 + 2) * kBM * 4 + 1024;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if ((++spins & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudget) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// shared-memory operand descriptor, 128-byte swizzle; lbo / sbo in bytes
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D = f32, A = B = bf16, M = 128, N = 128; b_mn: B is MN-major (bit 16)
__host__ __device__ constexpr uint32_t idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct Params {
  bf16* out;
  const int32_t* block_table;
  const int32_t* cu_q;
  const int32_t* kv_lens;
  int64_t o_stride;
  int bt_stride, nq, nkv, page, causal;
  float scale_log2;
  int* err;
  float* lse;                  // optional [total_q, nq]: log2-domain log-sum-exp of every row's scaled scores
};

__global__ void __launch_bounds__(320, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                  const __grid_constant__ CUtensorMap tma_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + BAR_OFF;
  // barrier slots
  // K and V have rings of their own: a K slot is free again as soon as the QK product that read it
  // has completed, a V slot after its PV product, so the load of K_{j+2} starts a whole tile earlier
  // than with a joint slot and the loads stay off the critical path.
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int b) { return bar0 + 8u * (9 + b); };
  auto s_free = [&](int b) { return bar0 + 8u * (11 + b); };
  const uint32_t p_full = bar0 + 8u * 13, p_free = bar0 + 8u * 14;
  const uint32_t o_full = bar0 + 8u * 15;             // the last PV product has completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + BAR_OFF + 24 * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int hk = h / (p.nq / p.nkv);
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int n_q_tiles = (q_len + kBM - 1) / kBM;
  if ((int)blockIdx.x >= n_q_tiles) return;          // uniform for the whole CTA: nothing allocated yet
  const int m0 = (n_q_tiles - 1 - (int)blockIdx.x) * kBM;  // heavy (late) tiles first
  const int kv_len = p.kv_lens[b];
  const int ctx_off = kv_len - q_len;                 // absolute position of this chunk's first query
  const int kv_hi = p.causal ? min(kv_len, ctx_off + m0 + kBM) : kv_len;
  const int n_tiles = (kv_hi + kBN - 1) / kBN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(o_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(s_free(s), 8);
    }
    mbar_init(p_full, 8);
    mbar_init(p_free, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  const uint32_t TS0 = tmem, TO0 = tmem + 256;        // S[b] = TS0 + 128 b; O accumulates at TO0 over all tiles

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, kTile);
      tma_load_2d(sbase + Q_OFF, &tma_q, h * kD, q_begin + m0, q_full);
      tma_load_2d(sbase + Q_OFF + kHalf, &tma_q, h * kD + 64, q_begin + m0, q_full);
    }
    const int pages = kBN / p.page;                   // pages per kv tile (page is 16, 32, 64 or 128)
    const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
    const int n_blk = (kv_len + p.page - 1) / p.page;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const int pg = j * pages + lane;
      const int myblk = (lane < pages && pg < n_blk) ? bt[pg] : 0;   // pages past the sequence read block 0 (masked)
      const int y = (myblk * p.nkv + hk) * p.page;
      const uint32_t off = (uint32_t)(lane * p.page * 128);
      const uint32_t kdst = sbase + KV_OFF + st * 2 * kTile, vdst = kdst + kTile;
      // every lane gathers its own page: the copies of all pages issue together
      if (!mbar_wait_warp(k_empty(st), ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
      if (lane == 0) mbar_expect_tx(k_full(st), kTile);
      __syncwarp();
      if (lane < pages) {
        tma_load_2d(kdst + off, &tma_k, 0, y, k_full(st));
        tma_load_2d(kdst + kHalf + off, &tma_k, 64, y, k_full(st));
      }
      if (!mbar_wait_warp(v_empty(st), ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
      if (lane == 0) mbar_expect_tx(v_full(st), kTile);
      __syncwarp();
      if (lane < pages) {
        tma_load_2d(vdst + off, &tma_v, 0, y, v_full(st));
        tma_load_2d(vdst + kHalf + off, &tma_v, 64, y, v_full(st));
      }
      __syncwarp();
    }
    if (!ok) {
      const long long t0 = clock64();
      while (clock64() - t0 < 20000000LL) {}          // bounded grace period for copies in flight
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t ID_QK = idesc(false), ID_PV = idesc(true);
    bool ok = mbar_wait_warp(q_full, 0, abort_flag);
    auto issue_qk = [&](int j) {
      // S[j & 1] = Q K_j^T : 8 steps of 16 along head_dim, two 64-element halves
      const uint32_t kaddr = sbase + KV_OFF + (j & 1) * 2 * kTile;
      if (lane == 0) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * kHalf + (ks & 3) * 32;
          umma(TS0 + (j & 1) * 128, smem_desc(sbase + Q_OFF + o, 16, 1024), smem_desc(kaddr + o, 16, 1024), ID_QK, ks != 0);
        }
        umma_commit(s_full(j & 1));
        umma_commit(k_empty(j & 1));   // the K slot may be refilled once these MMAs have read it
      }
      __syncwarp();
    };
    if (ok && n_tiles > 0) {
      ok = mbar_wait_warp(k_full(0), 0, abort_flag);
      tc_fence_after();
      if (ok) issue_qk(0);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) {
        const int nb = (j + 1) & 1, use = (j + 1) >> 1;
        if (!mbar_wait_warp(k_full(nb), use & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait_warp(s_free(nb), (use & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        issue_qk(j + 1);
      }
      if (!mbar_wait_warp(v_full(j & 1), (j >> 1) & 1, abort_flag)) { ok = false; break; }
      if (!mbar_wait_warp(p_full, j & 1, abort_flag)) { ok = false; break; }   // also: O has been rescaled if need be
      tc_fence_after();
      if (lane == 0) {
        // O += P V_j : 8 steps of 16 kv tokens; V is MN-major (rows = tokens, 128-byte rows of
        // 64 head_dim elements, second half of head_dim one half-tile further)
        const uint32_t vaddr = sbase + KV_OFF + (j & 1) * 2 * kTile + kTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t pa = sbase + P_OFF + (ks >> 2) * kHalf + (ks & 3) * 32;
          umma(TO0, smem_desc(pa, 16, 1024), smem_desc(vaddr + ks * 16 * 128, kHalf, 1024), ID_PV, (j | ks) != 0);
        }
        umma_commit(p_free);
        if (j == n_tiles - 1) umma_commit(o_full);
        umma_commit(v_empty(j & 1));
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax / output (warps 2..9)
    // Two threads per query row: warps 2-5 take kv columns / head_dim columns 0..63 of the row, warps
    // 6-9 take 64..127 (two warps per scheduler hide each other's TMEM round trips, and 64 instead of
    // 128 output values per thread leave room to keep the S row in registers: S is read once).
    const int quarter = warp & 3;                     // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;                 // which 64 columns
    const int row = quarter * 32 + lane;              // query row inside the tile
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int q_pos = ctx_off + m0 + row;             // absolute position of this query token
    const int limit = p.causal ? min(kv_len - 1, q_pos) : kv_len - 1;   // last kv index this row may see
    float* smax = reinterpret_cast<float*>(smem + XCH_OFF);             // [2 tile parities][2 halves][128 rows]
    float* lsum = smax + 2 * 2 * kBM;                                   // [2 halves][128 rows]
    // O stays in TMEM and the MMAs accumulate into it over all kv tiles.  The exponent uses a row
    // maximum m that lags the true one: it moves (and O and l are rescaled) only when the true
    // maximum has grown by more than 2^kLag, so after the first tiles the rescale is rare and the
    // common tile costs no pass over O at all.  P stays below 2^kLag, well inside bf16 and fp32 range.
    constexpr float kLag = 8.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    const uint32_t oaddr = TO0 + half * 64 + lane_addr;
    // Every thread runs every iteration and every named barrier even after a wait has given up (the
    // waits then fail at once): a thread that left early would strand its partners in bar.sync.
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = ok && mbar_wait(s_full(sb), (j >> 1) & 1, abort_flag);
      tc_fence_after();
      const uint32_t saddr = TS0 + sb * 128 + half * 64 + lane_addr;
      const int kv0 = j * kBN + half * 64;
      const bool full_tile = kv0 + 63 <= limit;
      uint32_t sv[64];
      tmem_ld32(saddr, sv);
      tmem_ld32(saddr + 32, sv + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free(sb));         // S has been read out: the next QK may overwrite it
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (full_tile || kv0 + i <= limit) mx = fmaxf(mx, __uint_as_float(sv[i]));
      smax[(sb * 2 + half) * kBM + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, smax[(sb * 2 + (half ^ 1)) * kBM + row]);
      const float m_true = fmaxf(m, mx * p.scale_log2);
      float factor = 1.f;
      if (m_true - m > kLag) {                        // also the first tile that shows this row a key (m = -inf)
        factor = exp2f(m - m_true);                   // 0 when m was -inf: nothing accumulated yet
        m = m_true;
      }
      const float m_use = m == -INFINITY ? 0.f : m;
      // P may be overwritten, and O touched, once the PV product of the previous tile has completed
      ok = ok && mbar_wait(p_free, (j & 1) ^ 1, abort_flag);
      if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(oaddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
          tmem_st32(oaddr + c * 32, r);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      float rs = 0.f;
      const uint32_t pbase = sbase + P_OFF + half * kHalf + row * 128;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const int i = u * 8 + e;
          float p0 = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - m_use);
          float p1 = exp2f(__uint_as_float(sv[i + 1]) * p.scale_log2 - m_use);
          if (!full_tile) {
            if (kv0 + i > limit) p0 = 0.f;
            if (kv0 + i + 1 > limit) p1 = 0.f;
          }
          rs += p0 + p1;
          const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        const uint32_t dst = pbase + ((u ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]),
                     "r"(packed[3])
                     : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      l = l * factor + rs;
    }
    float o[64];
    if (n_tiles > 0) {
      ok = ok && mbar_wait(o_full, 0, abort_flag);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(oaddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(r[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) o[i] = 0.f;
    }
    // ---- output: the two halves of a row add their sums, normalise, stage the tile in shared memory
    // (the Q buffer is free now), store rows
    lsum[half * kBM + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += lsum[(half ^ 1) * kBM + row];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (p.lse != nullptr && half == 0 && ok && m0 + row < q_len)
      p.lse[(int64_t)(q_begin + m0 + row) * p.nq + h] = l > 0.f ? m + log2f(l) : -INFINITY;
    uint8_t* stage = smem + Q_OFF;                    // [128 rows][256 bytes], 16-byte units XOR-swizzled by row
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = o[u * 8 + e] * inv;
      const bf16x8 v = pack8(f);
      *reinterpret_cast<uint4*>(stage + row * 256 + (((half * 8 + u) ^ (row & 15)) << 4)) = *reinterpret_cast<const uint4*>(&v);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (ok) {
      const int t = threadIdx.x - 64;                 // 0..255
      const int u = t & 15;
      for (int r0 = t >> 4; r0 < kBM; r0 += 16) {     // 16 rows per pass, 16 threads x 16 bytes per row
        if (m0 + r0 < q_len) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r0 * 256 + ((u ^ (r0 & 15)) << 4));
          *reinterpret_cast<uint4*>(p.out + (int64_t)(q_begin + m0 + r0) * p.o_stride + h * kD + u * 8) = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.err != nullptr) atomicExch(p.err, 1);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// bf16 [rows, cols] with row stride ld elements; box = [box_rows, 64 cols], 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static int* g_err[64] = {};

}  // namespace fmha
}  // namespace xllm

// Same contract as xllm_paged_prefill_attn for head_dim 128, no sliding window, page_size in
// {16, 32, 64, 128}: q [total_q, nq, 128] (row stride q_stride elements), caches
// [n_blocks, nkv, page, 128], cu_q absolute row offsets [batch + 1], kv_lens [batch].
// `lse` (optional, fp32 [total_q, nq]) receives every row's log-sum-exp in the log2 domain, so that the
// result can be merged with attention over other keys (xllm_attn_merge, the beam-tail kernel).
XLLM_API int xllm_paged_prefill_attn_tc_lse(void* out, int64_t o_stride, const void* q, int64_t q_stride, int64_t total_q,
                                            const void* k_cache, const void* v_cache, int64_t n_blocks,
                                            const void* block_table, int bt_stride, const void* cu_q,
                                            const void* kv_lens, int batch, int max_q_len, int nq, int nkv,
                                            int page_size, float scale, int causal, void* lse, void* stream) {
  using namespace xllm;
  using namespace xllm::fmha;
  if (batch == 0 || max_q_len == 0) return 0;
  if (nq % nkv != 0 || (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) || q_stride % 8 ||
      o_stride % 8 || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15))
    return (int)cudaErrorInvalidValue;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {};
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  if (g_err[dev & 63] == nullptr) {
    if (cudaMalloc(&g_err[dev & 63], sizeof(int)) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    cudaMemset(g_err[dev & 63], 0, sizeof(int));
  }
  CUtensorMap tq, tk, tv;
  const int64_t cache_rows = n_blocks * nkv * page_size;
  if (!make_map(&tq, q, total_q, (int64_t)nq * kD, q_stride, kBM) || !make_map(&tk, k_cache, cache_rows, kD, kD, page_size) ||
      !make_map(&tv, v_cache, cache_rows, kD, kD, page_size))
    return (int)cudaErrorInvalidValue;
  Params p;
  p.out = (bf16*)out; p.block_table = (const int32_t*)block_table; p.cu_q = (const int32_t*)cu_q;
  p.kv_lens = (const int32_t*)kv_lens; p.o_stride = o_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv;
  p.page = page_size; p.causal = causal; p.scale_log2 = scale * 1.4426950408889634f; p.err = g_err[dev & 63];
  p.lse = (float*)lse;
  dim3 grid((max_q_len + kBM - 1) / kBM, nq, batch);
  prefill_tc_kernel<<<grid, 320, SMEM_TOTAL, (cudaStream_t)stream>>>(tq, tk, tv, p);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_paged_prefill_attn_tc(void* out, int64_t o_stride, const void* q, int64_t q_stride, int64_t total_q,
                                        const void* k_cache, const void* v_cache, int64_t n_blocks,
                                        const void* block_table, int bt_stride, const void* cu_q, const void* kv_lens,
                                        int batch, int max_q_len, int nq, int nkv, int page_size, float scale,
                                        int causal, void* stream) {
  return xllm_paged_prefill_attn_tc_lse(out, o_stride, q, q_stride, total_q, k_cache, v_cache, n_blocks, block_table,
                                        bt_stride, cu_q, kv_lens, batch, max_q_len, nq, nkv, page_size, scale, causal,
                                        nullptr, stream);
}

// 0 = no bounded wait expired in the prefill kernel on this device since the last call.
XLLM_API int xllm_fmha_error_status() {
  using namespace xllm::fmha;
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_err[dev & 63] == nullptr) return 0;
  int v = 0;
  cudaMemcpy(&v, g_err[dev & 63], sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) cudaMemset(g_err[dev & 63], 0, sizeof(int));
  return v;
}
