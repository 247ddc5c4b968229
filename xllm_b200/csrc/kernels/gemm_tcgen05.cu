// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] · W[N,K]^T (+ bias[N])
//
// This is the engine's dense linear (qkv / o / gate_up / down / lm_head / router); the reference
// sends all of these to cuBLAS through torch::nn::functional::linear
// (xllm/core/kernels/cuda/matmul.cpp:21-25).
//
// Structure (one persistent CTA per SM, 192 threads, warp-specialised):
//   warp 0   TMA producer : cp.async.bulk.tensor 2-D tiles of A (128 x 64) and W (BN x 64) into a
//                           STAGES-deep shared-memory ring, 128-byte swizzle, completion on mbarriers
//   warp 1   MMA issuer   : one elected thread issues tcgen05.mma (cta_group::1, kind::f16,
//                           M = 128, N = BN, K = 16) straight from shared-memory descriptors into a
//                           TMEM accumulator; tcgen05.commit releases ring slots and publishes the
//                           finished accumulator
//   warps 2-5 epilogue    : tcgen05.ld the fp32 accumulator (each warp owns its 32 TMEM lanes),
//                           add bias, convert to bf16, stage 32 x 64 chunks in swizzled shared
//                           memory and write them out with TMA stores (full 128-byte rows)
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the main loop of tile i+1.  Both operands are K-major, which is exactly the layout of activations
// [tokens, in] and of nn.Linear weights [out, in]: no transposes anywhere.
//
// Every mbarrier wait is bounded (clock64 budget); on expiry the kernel raises an error word in
// global memory, all roles leave their loops, TMEM is released and the kernel returns normally.
#include "common.cuh"
#include <cuda.h>
#include <cstdlib>

namespace xllm {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr long long kWaitBudgetCycles = 4000000000LL;

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
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the budget ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if ((++spins & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024
// bytes apart (the layout TMA writes with CU_TENSOR_MAP_SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f8f6f4 with A = B = e4m3 (format code 0), D = f32; K per instruction is 32 elements (32 bytes)
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}
__device__ __forceinline__ void umma_fp8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Operand type and output scaling of a launch.  fp8 == 0: bf16 operands, no scaling.
// fp8 == 1: e4m3 operands, C = acc * a_scale[row or 0] * b_scale[col or 0] (+ bias).
// ks > 1: split-K.  Work unit = (tile, K slice).  Every unit adds its fp32 partial tile into the
// zero-filled scratch `ws` ([m_pad][N]) with TMA reduce-add (the adds happen in L2), waits for
// them to complete and bumps the tile's counter; the unit that arrives last reads the sum once,
// writes zeros back (the scratch is clean again for the next launch), adds the bias and stores the
// bf16 rows.  Nobody waits for anybody, so the scheme cannot deadlock.
struct GemmMode {
  const float* a_scale;
  const float* b_scale;
  int fp8, a_per_row, b_per_col;
  int ks;
  float* ws;
  int* counters;
  bf16* c;      // output base and row stride (elements) for the split-K finishing pass
  int64_t ldc;
  // Push mode (the reduce-scatter half of a tensor-parallel row-linear, fused into the GEMM): the
  // token rows are sharded over the ranks, S rows each; the epilogue stores every finished
  // 32-row slice of this rank's partial product straight into the owner rank's inbox
  // [world][S][N] over NVLink (plain 16-byte peer stores) and then releases the owner's arrival
  // counter (system-scope red.add of the row count), so the transfer of tile i overlaps the MMAs of
  // tile i+1 and the owner can start reducing as soon as its counter is full.
  void* const* push_bufs;  // [world] base pointers of the symmetric buffer; null = mode off
  void* const* push_sigs;  // [world] base pointers of the signal pads
  int64_t push_off;        // byte offset of the inbox inside the symmetric buffer
  int64_t push_sig_idx;    // uint32 index of the arrival counter inside a signal pad
  int push_S, push_rank, push_world;
  // Gated-activation epilogue: the weight rows are interleaved in groups of 128 output columns =
  // [gate of 64 features | up of the same 64 features]; the epilogue writes act(gate) * up, 64 columns per
  // group, into an output of N / 2 columns.  0 = off, 1 = SiLU, 2 = GELU(erf), 3 = GELU(tanh).
  int act_mul;
};
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
// One lane of a converged warp.  The producer and MMA warps run their loops with all 32 lanes and
// only predicate the TMA / tcgen05 instructions on the elected lane: loop state, shared-memory
// addresses and descriptors then stay warp-uniform, which is what these instructions take as
// operands (a loop run by a single lane under divergence pays a register-file round trip per
// operand: measured ~120 cycles per tcgen05.mma issue against ~30 here).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// Whole-warp bounded wait: every lane polls, the verdict is made uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
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


__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// r[i] += TMEM[taddr2 + i] for 32 columns: the second accumulator of a dual-issuer tile.
__device__ __forceinline__ void tmem_add32(uint32_t taddr2, uint32_t* r) {
  uint32_t t[32];
  tmem_ld32(taddr2, t);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(t[i]));
}

// TMEM is allocated in powers of two (32..512 columns).
__host__ __device__ constexpr int tmem_alloc_cols(int need) {
  return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}

constexpr int kEpiCols = 64;                       // columns per epilogue chunk (128 bytes of bf16)
constexpr int kEpiBufBytes = 32 * kEpiCols * 2;    // one warp's chunk: 32 rows x 64 cols
constexpr int kEpiBytes = 4 * 2 * kEpiBufBytes;    // 4 warps x 2 buffers

// Drain one warp's 32 x BN slice of a TMEM accumulator: tcgen05.ld -> (+bias) -> bf16 -> 128-byte
// swizzled shared memory -> TMA store (full 128-byte rows, clipped at the M / N edges by the
// tensor map).  Two chunk buffers per warp keep a store in flight while the next chunk is built.
template <int BN>
__device__ __forceinline__ void epilogue_slice(uint32_t taddr, const CUtensorMap* tmap_c, uint32_t warp_stage,
                                               int row0, int n0, const bf16* __restrict__ bias, int N, int lane,
                                               int& buf, const GemmMode mode = GemmMode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0},
                                               int M = 0, uint32_t taddr2 = 0) {
  if (mode.act_mul != 0) {
    if constexpr (BN % 128 == 0) {
#pragma unroll 1
      for (int c = 0; c < BN / 128; ++c) {
        uint32_t g[64], u[64];
        tmem_ld32(taddr + c * 128, g);
        tmem_ld32(taddr + c * 128 + 32, g + 32);
        tmem_ld32(taddr + c * 128 + 64, u);
        tmem_ld32(taddr + c * 128 + 96, u + 32);
        tmem_ld_wait();
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        const uint32_t sb = warp_stage + buf * kEpiBufBytes;
        const int col0 = (n0 >> 1) + c * kEpiCols;       // output column: half of the interleaved one
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            // gate and up are rounded to bf16 first, as the two-launch form stores them: a request's tokens
            // must not depend on which of the two forms its batch size selects
            const float x = __bfloat162float(__float2bfloat16(__uint_as_float(g[j * 8 + e])));
            float a;
            if (mode.act_mul == 1) a = x / (1.f + __expf(-x));
            else if (mode.act_mul == 2) a = 0.5f * x * (1.f + erff(x * 0.70710678f));
            else a = 0.5f * x * (1.f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
            f[e] = a * __bfloat162float(__float2bfloat16(__uint_as_float(u[j * 8 + e])));
          }
          const bf16x8 v = pack8(f);
          const uint4 w4 = *reinterpret_cast<const uint4*>(&v);
          const uint32_t dst = sb + lane * 128 + ((j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w4.x), "r"(w4.y), "r"(w4.z), "r"(w4.w)
                       : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tmap_c, sb, col0, row0);
          bulk_commit();
        }
        buf ^= 1;
      }
    }
    return;
  }
  float a_s = 1.f;
  if (mode.fp8 && mode.a_scale != nullptr) {
    const int r = row0 + lane;
    a_s = mode.a_per_row ? (r < M ? mode.a_scale[r] : 0.f) : mode.a_scale[0];
  }
#pragma unroll 1
  for (int c = 0; c < BN / kEpiCols; ++c) {
    uint32_t r[64];
    tmem_ld32(taddr + c * kEpiCols, r);
    tmem_ld32(taddr + c * kEpiCols + 32, r + 32);
    tmem_ld_wait();
    if (taddr2 != 0) {
      tmem_add32(taddr2 + c * kEpiCols, r);
      tmem_add32(taddr2 + c * kEpiCols + 32, r + 32);
    }
    if (lane == 0) bulk_wait_read<1>();  // the store that last read this buffer has finished reading
    __syncwarp();
    const uint32_t sb = warp_stage + buf * kEpiBufBytes;
    const int col0 = n0 + c * kEpiCols;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j * 8 + e]);
      if (mode.fp8 && col0 + j * 8 < N) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float b_s = mode.b_scale == nullptr ? 1.f : (mode.b_per_col ? mode.b_scale[col0 + j * 8 + e] : mode.b_scale[0]);
          f[e] *= a_s * b_s;
        }
      }
      if (bias != nullptr && col0 + j * 8 < N) {
        float bv[8];
        unpack8(*reinterpret_cast<const bf16x8*>(bias + col0 + j * 8), bv);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += bv[e];
      }
      const bf16x8 v = pack8(f);
      const uint4 u = *reinterpret_cast<const uint4*>(&v);
      const uint32_t dst = sb + lane * 128 + ((j ^ (lane & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                   : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmap_c, sb, col0, row0);
      bulk_commit();
    }
    buf ^= 1;
  }
}

// Push-mode epilogue of one warp (see GemmMode): tcgen05.ld -> bf16 -> swizzled shared memory ->
// coalesced 16-byte stores into the owners' inboxes (4 rows x 128 bytes per warp instruction),
// then one system-scope red.add per owner present in the slice.
template <int BN>
__device__ __forceinline__ void epilogue_push(uint32_t taddr, uint32_t warp_stage, int row0, int n0, int M, int N,
                                              int lane, const GemmMode& mode, uint32_t taddr2 = 0) {
  const int S = mode.push_S;
#pragma unroll 1
  for (int c = 0; c < BN / kEpiCols; ++c) {
    uint32_t r[64];
    tmem_ld32(taddr + c * kEpiCols, r);
    tmem_ld32(taddr + c * kEpiCols + 32, r + 32);
    tmem_ld_wait();
    if (taddr2 != 0) {
      tmem_add32(taddr2 + c * kEpiCols, r);
      tmem_add32(taddr2 + c * kEpiCols + 32, r + 32);
    }
    __syncwarp();  // the copy-out of the previous chunk has finished reading the staging buffer
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j * 8 + e]);
      const bf16x8 v = pack8(f);
      const uint4 u = *reinterpret_cast<const uint4*>(&v);
      const uint32_t dst = warp_stage + lane * 128 + ((j ^ (lane & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                   : "memory");
    }
    __syncwarp();
    const int unit = lane & 7;
    const int col = n0 + c * kEpiCols + unit * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      const int row = row0 + rr;
      if (row < M && col < N) {
        uint4 u;
        const uint32_t src = warp_stage + rr * 128 + ((unit ^ (rr & 7)) << 4);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(src));
        const int owner = row / S;
        uint8_t* base = reinterpret_cast<uint8_t*>(mode.push_bufs[owner]) + mode.push_off;
        const int64_t slot = (int64_t)mode.push_rank * S + (row - owner * S);
        *reinterpret_cast<uint4*>(base + (slot * N + col) * 2) = u;
      }
    }
  }
  __threadfence_system();
  __syncwarp();
  const int row = row0 + lane;
  const int owner = row < M ? row / S : -1;
  const unsigned grp = __match_any_sync(0xffffffffu, owner);
  if (owner >= 0 && lane == __ffs(grp) - 1) {
    uint32_t* cnt = reinterpret_cast<uint32_t*>(mode.push_sigs[owner]) + mode.push_sig_idx;
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"((uint32_t)__popc(grp)) : "memory");
  }
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}

// Split-K epilogue of one warp: add its 32 x BN fp32 slice into the scratch (32 x 32 chunks staged
// in swizzled shared memory, one TMA reduce-add each), then (all four epilogue warps together)
// bump the tile counter; returns true in the warps of the unit that arrived last.
template <int BN>
__device__ __forceinline__ bool splitk_dump(uint32_t taddr, const CUtensorMap* tmap_ws, uint32_t warp_stage,
                                            const GemmMode& mode, int counter_idx, int row0, int n0, int lane,
                                            int q, int& buf, volatile int* s_last, uint32_t taddr2 = 0) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    if (taddr2 != 0) tmem_add32(taddr2 + c * 32, r);
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
    const uint32_t sb = warp_stage + buf * kEpiBufBytes;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t dst = sb + lane * 128 + ((j ^ (lane & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(r[4 * j]), "r"(r[4 * j + 1]),
                   "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                   : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_reduce_add_2d(tmap_ws, sb, n0 + c * 32, row0);
      bulk_commit();
    }
    buf ^= 1;
  }
  if (lane == 0) {
    bulk_wait_all();  // the adds have been performed, not merely read from shared memory
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
  if (q == 0 && lane == 0) {
    const int old = atomicAdd(mode.counters + counter_idx, 1);
    const int last = old == mode.ks - 1;
    if (last) mode.counters[counter_idx] = 0;  // ready for the next launch
    *s_last = last;
    __threadfence();
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  return *s_last != 0;
}

// Finishing pass of the last arriver, one warp per 32 rows: read the summed fp32 rows (coalesced,
// from L2), put zeros back, add the bias and store bf16.  16 rows are in flight per step.
template <int BN>
__device__ __forceinline__ void splitk_finish(const GemmMode& mode, const bf16* __restrict__ bias, int row0, int n0,
                                              int M, int N, int lane) {
  constexpr int RB = 16;
#pragma unroll 1
  for (int cc = 0; cc < BN; cc += 128) {
    const int col = n0 + cc + lane * 4;
    if (cc + lane * 4 >= BN || col >= N) continue;
    float bv[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias != nullptr) {
      const uint2 b = *reinterpret_cast<const uint2*>(bias + col);
      const __nv_bfloat162 b0 = *reinterpret_cast<const __nv_bfloat162*>(&b.x);
      const __nv_bfloat162 b1 = *reinterpret_cast<const __nv_bfloat162*>(&b.y);
      bv[0] = __low2float(b0); bv[1] = __high2float(b0); bv[2] = __low2float(b1); bv[3] = __high2float(b1);
    }
#pragma unroll 1
    for (int r0 = 0; r0 < 32; r0 += RB) {
      float4 v[RB];
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int row = row0 + r0 + i;
        v[i] = row < M ? __ldcg(reinterpret_cast<const float4*>(mode.ws + (int64_t)row * N + col))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int row = row0 + r0 + i;
        if (row < M) {
          __stcg(reinterpret_cast<float4*>(mode.ws + (int64_t)row * N + col), make_float4(0.f, 0.f, 0.f, 0.f));
          const __nv_bfloat162 o0 = __floats2bfloat162_rn(v[i].x + bv[0], v[i].y + bv[1]);
          const __nv_bfloat162 o1 = __floats2bfloat162_rn(v[i].z + bv[2], v[i].w + bv[3]);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t*>(&o0);
          o.y = *reinterpret_cast<const uint32_t*>(&o1);
          *reinterpret_cast<uint2*>(mode.c + (int64_t)row * mode.ldc + col) = o;
        }
      }
    }
  }
}

// KS = 64-element K blocks per ring stage.  A stage costs one barrier wait, one commit and one
// producer round trip whatever it holds (~600 cycles measured); narrow tiles, whose MMAs are short,
// take two K blocks per stage so that this fixed cost is paid half as often.
template <int BN, int STAGES, int KS = 1>
struct GemmSmem {
  static constexpr int A_KB = kBM * kBK * 2;  // one K block of A
  static constexpr int B_KB = BN * kBK * 2;
  static constexpr int A_BYTES = KS * A_KB;
  static constexpr int B_BYTES = KS * B_KB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;  // 1024-byte aligned: stages are multiples of 1 KB
  static constexpr int BAR_OFF = EPI_OFF + kEpiBytes;
  static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory per CTA");
};

template <int BN, int STAGES, int KS, bool DUAL>
__global__ void __launch_bounds__(DUAL ? 224 : 192, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_ws,
                         const bf16* __restrict__ bias, int M, int N, int K, int a_box_rows, int w_packed, const int32_t* __restrict__ tile_expert, int expert_rows,
                         const GemmMode mode, int* __restrict__ err_word) {
  using S = GemmSmem<BN, STAGES, KS>;
  // DUAL: a second MMA-issuing warp (warp 6) owns the odd ring stages and accumulates them into an
  // accumulator of its own; the epilogue adds the two.  One issuing warp spends ~500 cycles per stage
  // on waits, commits and issue latency, which hides under 256-wide MMAs but not under narrow ones.
  // Ownership goes by STAGE, not by step within a tile: a warp then waits on each of its barriers
  // every pass of the ring, and a parity wait is only meaningful for a waiter that never skips a
  // phase of the barrier (with an even ring, stage parity = parity of the global step count).
  constexpr int NACC = DUAL ? 2 : 1;
  static_assert(!DUAL || STAGES % 2 == 0, "stage ownership by parity needs an even ring");
  static_assert(2 * NACC * BN <= 512 && BN % 64 == 0, "TMEM has 512 columns; the epilogue works in 64-column chunks");
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles need 1024-byte aligned bases
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + S::BAR_OFF;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_elems = mode.fp8 ? 2 * kBK : kBK;  // elements per 128-byte K block
  const int k_blocks = (K + k_elems - 1) / k_elems;
  const int ks = mode.ks;
  const int k_steps = (k_blocks + KS - 1) / KS;  // ring stages along K (a tail block past K reads as zeros)
  const int kbs = (k_steps + ks - 1) / ks;       // stages per split
  const int total_units = total_tiles * ks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), NACC);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(tmem_alloc_cols(2 * NACC * BN)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()

  if (warp == 0) {
    {
      // ------------------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int armed = 0;  // loads issued so far (for the drain on an aborted run)
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit % total_tiles, kslice = unit / total_tiles;
        const int kb0 = kslice * kbs, kb1 = min(k_steps, kb0 + kbs);
        const int m0 = (tile % m_tiles) * kBM;
        int n0 = (tile / m_tiles) * BN;
        if (tile_expert != nullptr) {
          // grouped (MoE) mode: the row tile belongs to one expert, whose weights start
          // expert_rows * e rows into W; unused tail tiles are skipped by every role alike
          const int e = tile_expert[tile % m_tiles];
          if (e < 0) continue;
          n0 += e * expert_rows;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_warp(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = sbase + stage * S::STAGE_BYTES;
          if (elect_one()) {
            // for M < 128 the A box only covers the rows that exist; the rest of the 128-row operand
            // is whatever the slot held before and only feeds output rows that are never stored
            mbar_expect_tx(full_bar(stage), S::B_BYTES + KS * a_box_rows * kBK * 2);
#pragma unroll
            for (int s = 0; s < KS; ++s)
              tma_load_2d(a_dst + s * S::A_KB, &tma_a, (kb * KS + s) * k_elems, m0, full_bar(stage));
            if (!w_packed) {
#pragma unroll
              for (int s = 0; s < KS; ++s)
                tma_load_2d(a_dst + S::A_BYTES + s * S::B_KB, &tma_b, (kb * KS + s) * k_elems, n0, full_bar(stage));
            } else {
              // tile-packed weights: every 64 x 64 block is one contiguous 8 KB run
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(a_dst + S::A_BYTES + j * 8192, &tma_b, 0, ((n0 / 64 + j) * k_blocks + kb) * 64,
                            full_bar(stage));
            }
          }
          __syncwarp();
          ++armed;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // give the copies that are still in flight a bounded chance to land before the CTA exits
        const int pending = armed < STAGES ? armed : STAGES;
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i;
          uint32_t ph = phase;
          if (s < 0) { s += STAGES; ph ^= 1; }
          const long long t0 = clock64();
          while (!mbar_try(full_bar(s), ph) && clock64() - t0 < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1 || (DUAL && warp == 6)) {
    {
      // ------------------------------------------------------------------ MMA issuer(s)
      const int mw = warp == 1 ? 0 : 1;  // which issuer this warp is
      const uint32_t idesc = mode.fp8 ? umma_idesc_e4m3(BN) : umma_idesc_bf16(BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit % total_tiles, kslice = unit / total_tiles;
        const int kb0 = kslice * kbs, kb1 = min(k_steps, kb0 + kbs);
        if (tile_expert != nullptr && tile_expert[tile % m_tiles] < 0) continue;
        const int acc = t & 1;
        const uint32_t use = (uint32_t)(t >> 1);
        ++t;
        if (!mbar_wait_warp(tempty_bar(acc), (use & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc * NACC + mw) * BN;
        bool fresh = true;  // this issuer has not written its accumulator for this unit yet
        for (int kb = kb0; kb < kb1; ++kb) {
          if (DUAL && (stage & 1) != mw) {  // the other issuer's stage
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (!mbar_wait_warp(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = sbase + stage * S::STAGE_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int s = 0; s < KS; ++s) {
              const uint64_t adesc = umma_smem_desc(a_addr + s * S::A_KB);
              const uint64_t bdesc = umma_smem_desc(a_addr + S::A_BYTES + s * S::B_KB);
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k) {
                // +32 bytes (2 x 16-byte units) along K inside the swizzled row per UMMA_K = 16
                if (mode.fp8) umma_fp8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, !fresh || (s | k) != 0);
                else umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, !fresh || (s | k) != 0);
              }
            }
            umma_commit(empty_bar(stage));  // slot reusable once these MMAs have read it
          }
          __syncwarp();
          fresh = false;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) umma_commit(tfull_bar(acc));  // accumulator complete
        __syncwarp();
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    bool ok = true;
    int t = 0, ebuf = 0;
    int steps_done = 0;  // ring steps of the units before this one: its parity says who owns the first stage
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const int tile = unit % total_tiles, kslice = unit / total_tiles;
      if (tile_expert != nullptr && tile_expert[tile % m_tiles] < 0) continue;
      const int m0 = (tile % m_tiles) * kBM, n0 = (tile / m_tiles) * BN;
      const int n_steps = min(k_steps, kslice * kbs + kbs) - kslice * kbs;
      const int acc = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      ++t;
      if (!mbar_wait(tfull_bar(acc), use & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t taddr = tmem_base + acc * NACC * BN + ((uint32_t)(q * 32) << 16);
      uint32_t taddr2 = 0u;
      if (DUAL) {
        // which accumulators this unit wrote: both from two steps on, else the owner of its only stage
        if (n_steps >= 2) taddr2 = taddr + BN;
        else if (steps_done & 1) taddr += BN;
        steps_done += n_steps;
      }
      if (mode.push_bufs != nullptr) {
        epilogue_push<BN>(taddr, sbase + S::EPI_OFF + q * 2 * kEpiBufBytes, m0 + q * 32, n0, M, N, lane, mode, taddr2);
      } else if (ks == 1) {
        epilogue_slice<BN>(taddr, &tma_c, sbase + S::EPI_OFF + q * 2 * kEpiBufBytes, m0 + q * 32, n0, bias, N, lane, ebuf, mode, M, taddr2);
      } else {
        const bool last = splitk_dump<BN>(taddr, &tma_ws, sbase + S::EPI_OFF + q * 2 * kEpiBufBytes, mode, tile,
                                          m0 + q * 32, n0, lane, q, ebuf, s_last, taddr2);
        // the accumulator has been read out: release it before the (longer) finishing pass
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        if (last) splitk_finish<BN>(mode, bias, m0 + q * 32, n0, M, N, lane);
        continue;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (lane == 0) bulk_wait_all();  // every output store has completed before the CTA exits
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && err_word != nullptr) atomicExch(err_word, 1);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_alloc_cols(2 * NACC * BN)));
  }
}

// ===================================================================================== 2-CTA
// cta_group::2 variant: a cluster of two CTAs (a pair of SMs) computes one 256 x BN tile.  Each
// CTA loads its own 128 rows of A and its own BN/2 rows of W, so every operand byte is fetched
// once per pair and a ring stage costs 16 KB + BN*64 bytes per CTA — deeper pipelines than the
// 1-CTA kernel at the same tile area.  The leader CTA (cluster rank 0) issues
// tcgen05.mma.cta_group::2 (M = 256); the accumulator rows 0-127 live in the leader's TMEM and
// rows 128-255 in the peer's.  Loads of both CTAs complete on the leader's "full" barrier;
// tcgen05.commit signals the "empty" / "accumulator full" barriers of both CTAs at once; the
// epilogue warps of both CTAs arrive on the leader's "accumulator empty" barrier.
__device__ __forceinline__ bool mbar_wait_cluster_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag);
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (true) {
    if (mbar_try_cluster(bar, parity)) return true;
    if ((++spins & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_cluster_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait_cluster(bar, parity, abort_flag));
}
// TMA tile load issued by either CTA of the pair; completion bytes are counted on the barrier of
// the pair's leader (bit 24 of a shared-window address selects the CTA inside the pair).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar) {
  const uint32_t leader_bar = bar & 0xFEFFFFFFu;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_bf16_m256(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int BN, int STAGES, int KS = 1>
struct GemmSmem2 {
  static constexpr int A_KB = kBM * kBK * 2;            // this CTA's 128 rows of A, one K block
  static constexpr int B_KB = (BN / 2) * kBK * 2;       // this CTA's half of the W tile
  static constexpr int A_BYTES = KS * A_KB;
  static constexpr int B_BYTES = KS * B_KB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = EPI_OFF + kEpiBytes;
  static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory per CTA");
};

template <int BN, int STAGES, int KS, bool DUAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DUAL ? 224 : 192, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                              const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_ws,
                              const bf16* __restrict__ bias, int M, int N, int K, int w_packed, const GemmMode mode, int* __restrict__ err_word) {
  using S = GemmSmem2<BN, STAGES, KS>;
  constexpr int NACC = DUAL ? 2 : 1;  // accumulators per tile: one per MMA-issuing warp of the leader
  static_assert(2 * NACC * BN <= 512 && BN % 64 == 0, "TMEM has 512 columns; the epilogue works in 64-column chunks");
  static_assert(!DUAL || STAGES % 2 == 0, "stage ownership by parity needs an even ring");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + S::BAR_OFF;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM), n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kBK - 1) / kBK;
  const int ks = mode.ks;
  const int k_steps = (k_blocks + KS - 1) / KS;
  const int kbs = (k_steps + ks - 1) / ks;
  const int total_units = total_tiles * ks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), NACC);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(tmem_alloc_cols(2 * NACC * BN)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()

  if (warp == 0) {
    {
      // ------------------------------------------------------------------ TMA producer (both CTAs)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = pair; unit < total_units && ok; unit += n_pairs) {
        const int tile = unit % total_tiles, kslice = unit / total_tiles;
        const int kb0 = kslice * kbs, kb1 = min(k_steps, kb0 + kbs);
        const int m0 = (tile % m_tiles) * (2 * kBM) + (int)rank * kBM;
        const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_cluster_warp(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = sbase + stage * S::STAGE_BYTES;
          if (elect_one()) {
            if (leader) mbar_expect_tx(full_bar(stage), 2 * S::STAGE_BYTES);
#pragma unroll
            for (int s = 0; s < KS; ++s)
              tma_load_2d_pair(a_dst + s * S::A_KB, &tma_a, (kb * KS + s) * kBK, m0, full_bar(stage));
            if (!w_packed) {
#pragma unroll
              for (int s = 0; s < KS; ++s)
                tma_load_2d_pair(a_dst + S::A_BYTES + s * S::B_KB, &tma_b, (kb * KS + s) * kBK, n0, full_bar(stage));
            } else {
              constexpr int ROWS = BN / 2 < 64 ? BN / 2 : 64;  // rows per packed-block load
#pragma unroll
              for (int j = 0; j < (BN / 2) / ROWS; ++j) {
                const int n = n0 + j * ROWS;
                tma_load_2d_pair(a_dst + S::A_BYTES + j * ROWS * 128, &tma_b, 0,
                                 ((n / 64) * k_blocks + kb) * 64 + (n % 64), full_bar(stage));
              }
            }
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) {}  // bounded grace period for copies still in flight
      }
    }
  } else if (warp == 1 || (DUAL && warp == 6)) {
    if (leader) {
      // ------------------------------------------------------------------ MMA issuer(s) (leader only)
      const int mw = warp == 1 ? 0 : 1;
      constexpr uint32_t idesc = umma_idesc_bf16_m256(BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int unit = pair; unit < total_units && ok; unit += n_pairs, ++t) {
        const int kslice = unit / total_tiles;
        const int kb0 = kslice * kbs, kb1 = min(k_steps, kb0 + kbs);
        const int acc = t & 1;
        const uint32_t use = (uint32_t)(t >> 1);
        if (!mbar_wait_cluster_warp(tempty_bar(acc), (use & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc * NACC + mw) * BN;
        bool fresh = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (DUAL && (stage & 1) != mw) {
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (!mbar_wait_cluster_warp(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = sbase + stage * S::STAGE_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int s = 0; s < KS; ++s) {
              const uint64_t adesc = umma_smem_desc(a_addr + s * S::A_KB);
              const uint64_t bdesc = umma_smem_desc(a_addr + S::A_BYTES + s * S::B_KB);
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k)
                umma_bf16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, !fresh || (s | k) != 0);
            }
            umma_commit_pair(empty_bar(stage));
          }
          __syncwarp();
          fresh = false;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) umma_commit_pair(tfull_bar(acc));
        __syncwarp();
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    const uint32_t leader_tempty0 = map_to_cta(tempty_bar(0), 0);
    bool ok = true;
    int t = 0, ebuf = 0;
    int steps_done = 0;
    for (int unit = pair; unit < total_units && ok; unit += n_pairs, ++t) {
      const int tile = unit % total_tiles, kslice = unit / total_tiles;
      const int m0 = (tile % m_tiles) * (2 * kBM) + (int)rank * kBM, n0 = (tile / m_tiles) * BN;
      const int n_steps = min(k_steps, kslice * kbs + kbs) - kslice * kbs;
      const int acc = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      if (!mbar_wait_cluster(tfull_bar(acc), use & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t taddr = tmem_base + acc * NACC * BN + ((uint32_t)(q * 32) << 16);
      uint32_t taddr2 = 0u;
      if (DUAL) {
        if (n_steps >= 2) taddr2 = taddr + BN;
        else if (steps_done & 1) taddr += BN;
        steps_done += n_steps;
      }
      if (ks == 1) {
        GemmMode pm{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0};
        pm.act_mul = mode.act_mul;
        epilogue_slice<BN>(taddr, &tma_c, sbase + S::EPI_OFF + q * 2 * kEpiBufBytes, m0 + q * 32, n0, bias, N, lane, ebuf,
                           pm, 0, taddr2);
      } else {
        // one counter per (tile, CTA of the pair): each CTA finishes its own 128 rows
        const bool last = splitk_dump<BN>(taddr, &tma_ws, sbase + S::EPI_OFF + q * 2 * kEpiBufBytes, mode,
                                          tile * 2 + (int)rank, m0 + q * 32, n0, lane, q, ebuf, s_last, taddr2);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(leader_tempty0 + 8u * acc);
        if (last) splitk_finish<BN>(mode, bias, m0 + q * 32, n0, M, N, lane);
        continue;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(leader_tempty0 + 8u * acc);
    }
    if (lane == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && err_word != nullptr) atomicExch(err_word, 1);
  cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers / smem
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_alloc_cols(2 * NACC * BN)));
  }
}

// ------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] (row stride ld elements), box = [box_rows, 64 cols], 128B swizzle.
static bool make_tmap(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows,
                      bool promote = true, bool bytes = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (bytes ? 1 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)(bytes ? 2 * kBK : kBK), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  promote ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// fp32 row-major [rows, cols], box 32 x 32 (128-byte rows), 128B swizzle: the split-K scratch.
static bool make_tmap_f32(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int* g_err_word[64] = {};
// Two MMA-issuing warps for the narrow-tile kernels.  Off by default: measured on B200 the decode-size
// GEMMs are bound by what one SM can pull from L2/HBM (~100 GB/s), not by MMA issue, and the second
// issuer changes nothing (16.8 vs 16.4 us at 256 x 4096 x 4096).
static int g_dual = 0;
static int g_k_per_stage = 2;  // preferred K blocks per ring stage for tiles narrower than 256

// Split-K scratch of one device: the zero-filled fp32 accumulation area and the per-tile arrival counters.  Allocated
// once (never during stream capture); split-K GEMMs of one device must be stream-ordered with
// respect to one another, which holds for the single compute stream of the engine.
constexpr size_t kSplitWsBytes = 64u << 20;
constexpr int kSplitCounters = 16384;
static float* g_split_ws[64] = {};
static int* g_split_cnt[64] = {};

static bool split_scratch_ready(int dev, cudaStream_t s) {
  if (g_split_ws[dev & 63] != nullptr) return true;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return false;
  float* ws = nullptr;
  int* cnt = nullptr;
  if (cudaMalloc(&ws, kSplitWsBytes) != cudaSuccess) return false;
  if (cudaMalloc(&cnt, kSplitCounters * sizeof(int)) != cudaSuccess) {
    cudaFree(ws);
    return false;
  }
  cudaMemset(cnt, 0, kSplitCounters * sizeof(int));
  cudaMemset(ws, 0, kSplitWsBytes);  // every launch leaves the scratch zero-filled again
  g_split_ws[dev & 63] = ws;
  g_split_cnt[dev & 63] = cnt;
  return true;
}

// Clamp a requested split so that every K slice is non-empty and the scratch is large enough.
static int usable_split(int ks, int M, int N, int K, int k_per_stage, int counters_needed, int dev, cudaStream_t s) {
  const int k_blocks = (K + kBK * k_per_stage - 1) / (kBK * k_per_stage);  // ring stages along K
  if (ks > k_blocks) ks = k_blocks;
  if (ks <= 1 || N % 4) return 1;
  const int kbs = (k_blocks + ks - 1) / ks;
  ks = (k_blocks + kbs - 1) / kbs;
  if (ks <= 1 || counters_needed > kSplitCounters) return 1;
  if ((size_t)M * (size_t)N * sizeof(float) > kSplitWsBytes) return 1;
  if (!split_scratch_ready(dev, s)) return 1;
  return ks;
}

template <int BN, int STAGES, int KS = 1, bool DUAL = false>
static int launch_gemm(const void* a, const void* w, void* c, const void* bias, int M, int N, int K, int64_t lda,
                       int64_t ldw, int64_t ldc, int max_ctas, int w_packed, cudaStream_t s,
                       const int32_t* tile_expert = nullptr, int n_experts = 1,
                       GemmMode mode = GemmMode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0}, int split_k = 1) {
  using S = GemmSmem<BN, STAGES, KS>;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {};
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, STAGES, KS, DUAL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  if (g_err_word[dev & 63] == nullptr) {
    // one 4-byte status word per device, allocated on first use (not during stream capture)
    if (cudaMalloc(&g_err_word[dev & 63], sizeof(int)) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    cudaMemset(g_err_word[dev & 63], 0, sizeof(int));
  }
  CUtensorMap ta, tb, tc;
  const int a_box = M >= kBM ? kBM : ((M + 7) & ~7);
  const bool okb = w_packed ? make_tmap(&tb, w, (int64_t)N * (K / 64), 64, 64, 64)
                            : make_tmap(&tb, w, (int64_t)N * n_experts, K, ldw, BN, true, mode.fp8 != 0);
  if (!make_tmap(&ta, a, M, K, lda, a_box, true, mode.fp8 != 0) || !okb) return (int)cudaErrorInvalidValue;
  if (mode.push_bufs != nullptr) tc = ta;  // push mode stores through peer pointers, the map is unused
  // gated-activation epilogue: the output has one column per (gate, up) pair, half of the GEMM's N
  else if (!make_tmap(&tc, c, M, mode.act_mul ? N / 2 : N, ldc, 32, false)) return (int)cudaErrorInvalidValue;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  if (split_k > 1 && tile_expert == nullptr && !mode.fp8) {
    mode.ks = usable_split(split_k, M, N, K, KS, tiles, dev, s);
    mode.ws = g_split_ws[dev & 63];
    mode.counters = g_split_cnt[dev & 63];
    mode.c = (bf16*)c;
    mode.ldc = ldc;
  }
  CUtensorMap tws = tc;
  if (mode.ks > 1 && !make_tmap_f32(&tws, mode.ws, M, N)) return (int)cudaErrorInvalidValue;
  const int units = tiles * mode.ks;
  int grid = units < max_ctas ? units : max_ctas;
  launch_pdl(gemm_bf16_tcgen05_kernel<BN, STAGES, KS, DUAL>, dim3(grid), dim3(DUAL ? 224 : 192), S::TOTAL, s, ta, tb, tc, tws, (const bf16*)bias, M, N, K, a_box,
                                                                 w_packed, tile_expert, N, mode, g_err_word[dev & 63]);
  return XLLM_LAUNCH_CHECK();
}

template <int BN, int STAGES, int KS = 1, bool DUAL = false>
static int launch_gemm_pair(const void* a, const void* w, void* c, const void* bias, int M, int N, int K, int64_t lda,
                            int64_t ldw, int64_t ldc, int max_ctas, int w_packed, cudaStream_t s, int split_k = 1,
                            int act_mul = 0) {
  using S = GemmSmem2<BN, STAGES, KS>;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {};
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_pair_kernel<BN, STAGES, KS, DUAL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  if (g_err_word[dev & 63] == nullptr) {
    if (cudaMalloc(&g_err_word[dev & 63], sizeof(int)) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    cudaMemset(g_err_word[dev & 63], 0, sizeof(int));
  }
  CUtensorMap ta, tb, tc;
  const bool okb = w_packed ? make_tmap(&tb, w, (int64_t)N * (K / 64), 64, 64, BN / 2 < 64 ? BN / 2 : 64)
                            : make_tmap(&tb, w, N, K, ldw, BN / 2);
  if (!make_tmap(&ta, a, M, K, lda, kBM) || !okb || !make_tmap(&tc, c, M, act_mul ? N / 2 : N, ldc, 32, false))
    return (int)cudaErrorInvalidValue;
  const int tiles = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + BN - 1) / BN);
  GemmMode mode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0};
  mode.act_mul = act_mul;
  if (act_mul) split_k = 1;
  if (split_k > 1) {
    mode.ks = usable_split(split_k, M, N, K, KS, 2 * tiles, dev, s);
    mode.ws = g_split_ws[dev & 63];
    mode.counters = g_split_cnt[dev & 63];
    mode.c = (bf16*)c;
    mode.ldc = ldc;
  }
  CUtensorMap tws = tc;
  if (mode.ks > 1 && !make_tmap_f32(&tws, mode.ws, M, N)) return (int)cudaErrorInvalidValue;
  const int units = tiles * mode.ks;
  int pairs = units < max_ctas / 2 ? units : max_ctas / 2;
  launch_pdl(gemm_bf16_tcgen05_pair_kernel<BN, STAGES, KS, DUAL>, dim3(2 * pairs), dim3(DUAL ? 224 : 192), S::TOTAL, s, ta, tb, tc, tws, (const bf16*)bias, M, N, K,
                                                                            w_packed, mode, g_err_word[dev & 63]);
  return XLLM_LAUNCH_CHECK();
}

// C[M, N / 2] = act(A W_gate^T) * (A W_up^T) in one launch.  W [N, K] holds the fused gate|up projection with its
// rows interleaved in groups of 128 = [64 gate rows | the 64 up rows of the same features] (N % 256 == 0); the
// 256-wide tiles of the CTA-pair kernel then hold both halves of 128 features and the epilogue applies the gated
// activation on the fp32 accumulators before anything is written.  act: 1 SiLU, 2 GELU(erf), 3 GELU(tanh).
XLLM_API int xllm_gemm_bf16_act_mul(const void* a, const void* w, void* c, int M, int N, int K, int64_t lda, int64_t ldw,
                                    int64_t ldc, int act, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 8 || N % 256 || lda % 8 || ldw % 8 || ldc % 8 || act < 1 || act > 3) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) return (int)cudaErrorInvalidValue;
  return launch_gemm_pair<256, 6>(a, w, c, nullptr, M, N, K, lda, ldw, ldc, 148, 0, (cudaStream_t)stream, 1, act);
}

// ===================================================================================== block-scaled fp8
// C[M,N] (bf16) = sum over 128-wide K blocks kb of
//     (A_q[:, kb] . W_q[:, kb]^T) * a_scale[m, kb] * w_scale[n / 128, kb]
// with A_q, W_q e4m3: the format of DeepSeek-V3-style checkpoints (weights quantised in 128 x 128
// blocks, activations per token in groups of 128).  The reference has no such kernel on CUDA: its
// CUTLASS sm100 scaled_mm refuses block scales
// (xllm/core/kernels/cuda/cutlass_w8a8/scaled_mm_c3x_sm100.cu:34-44).
//
// The scales differ from one K block to the next, so the products of different K blocks cannot be
// summed inside the tensor core's accumulator.  Each K block (4 x tcgen05.mma kind::f8f6f4, K = 32) is
// accumulated FRESH into one of four 128-column TMEM buffers (all 512 columns: with two, the round trip
// MMA -> commit -> tcgen05.ld -> release of a buffer, ~1000 cycles, is longer than the ~260 cycles of a
// K block's MMAs and the tensor pipe idles half the time); the four epilogue warps read a buffer back
// (tcgen05.ld), multiply by the block's scales and add into fp32 registers (eight warps: one output row
// and 64 of the 128 columns per thread) while the MMA warp already fills the other buffer.  One tile is 128 x 128, so
// the weight scale is one number per (tile, K block) and the activation scale one per (row, K block).
// Grouped form (MoE experts): `tile_expert[row tile]` names the expert of each 128-row tile (-1:
// skip); expert e's weights start e * expert_rows rows into W and its scale rows e * expert_rows / 128
// rows into w_scale.
constexpr int kFbStages = 6;
constexpr int kFbAcc = 4;        // TMEM accumulators of 128 columns
struct FbSmem {
  static constexpr int A_BYTES = kBM * 128;        // 128 rows x 128 bytes (one K block of e4m3)
  static constexpr int B_BYTES = 128 * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFF = kFbStages * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + (2 * kFbStages + 2 * kFbAcc) * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(320, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      bf16* __restrict__ c, int64_t ldc, const float* __restrict__ a_scale,
                      const float* __restrict__ w_scale, int M, int N, int K, int a_box_rows,
                      const int32_t* __restrict__ tile_expert, int expert_rows, int* __restrict__ err_word) {
  using S = FbSmem;
  constexpr int BN = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + S::BAR_OFF;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kFbStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kFbStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kFbStages + kFbAcc + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + (2 * kFbStages + 2 * kFbAcc) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = K / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFbStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kFbAcc; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int armed = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % m_tiles) * kBM;
      int n0 = (tile / m_tiles) * BN;
      if (tile_expert != nullptr) {
        const int e = tile_expert[tile % m_tiles];
        if (e < 0) continue;
        n0 += e * expert_rows;
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_warp(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
        const uint32_t a_dst = sbase + stage * S::STAGE_BYTES;
        if (elect_one()) {
          mbar_expect_tx(full_bar(stage), S::B_BYTES + a_box_rows * 128);
          tma_load_2d(a_dst, &tma_a, kb * 128, m0, full_bar(stage));
          tma_load_2d(a_dst + S::A_BYTES, &tma_b, kb * 128, n0, full_bar(stage));
        }
        __syncwarp();
        ++armed;
        if (++stage == kFbStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok) {
      const int pending = armed < kFbStages ? armed : kFbStages;
      for (int i = 0; i < pending; ++i) {
        int s = stage - 1 - i;
        uint32_t ph = phase;
        if (s < 0) { s += kFbStages; ph ^= 1; }
        const long long t0 = clock64();
        while (!mbar_try(full_bar(s), ph) && clock64() - t0 < 20000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = umma_idesc_e4m3(BN);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    uint32_t g = 0;  // K blocks issued so far: block g uses accumulator g % 4 for the (g / 4)-th time
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      if (tile_expert != nullptr && tile_expert[tile % m_tiles] < 0) continue;
      for (int kb = 0; kb < k_blocks; ++kb, ++g) {
        const int acc = g & (kFbAcc - 1);
        if (!mbar_wait_warp(tempty_bar(acc), ((g / kFbAcc) & 1) ^ 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait_warp(full_bar(stage), phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = sbase + stage * S::STAGE_BYTES;
        if (elect_one()) {
          const uint64_t adesc = umma_smem_desc(a_addr);
          const uint64_t bdesc = umma_smem_desc(a_addr + S::A_BYTES);
          const uint32_t d_tmem = tmem_base + acc * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_fp8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, k != 0);
          umma_commit(empty_bar(stage));   // the ring slot is free once these MMAs have read it
          umma_commit(tfull_bar(acc));     // ... and the block's product is complete in TMEM
        }
        __syncwarp();
        if (++stage == kFbStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // -------------------------------------------------------------------- promote + store (warps 2..9)
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int ch0 = ((warp - 2) >> 2) * (BN / 2);   // its half of the tile's columns
    bool ok = true;
    uint32_t g = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int e = 0;
      if (tile_expert != nullptr) {
        e = tile_expert[tile % m_tiles];
        if (e < 0) continue;
      }
      const int m0 = (tile % m_tiles) * kBM, n0 = (tile / m_tiles) * BN;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < M;
      const float* as = a_scale + (int64_t)(row_ok ? row : 0) * k_blocks;
      const float* ws = w_scale + ((int64_t)(e * expert_rows + n0) / 128) * k_blocks;
      float accum[BN / 2];
#pragma unroll
      for (int i = 0; i < BN / 2; ++i) accum[i] = 0.f;
      float sc_next = row_ok ? as[0] * ws[0] : 0.f;
      for (int kb = 0; kb < k_blocks; ++kb, ++g) {
        const int acc = g & (kFbAcc - 1);
        const float sc = sc_next;
        if (kb + 1 < k_blocks) sc_next = row_ok ? as[kb + 1] * ws[kb + 1] : 0.f;   // in flight during the wait
        if (!mbar_wait(tfull_bar(acc), (g / kFbAcc) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * BN + ch0 + ((uint32_t)(q * 32) << 16);
        uint32_t r0[32], r1[32];
        tmem_ld32(taddr, r0);
        tmem_ld32(taddr + 32, r1);
        tmem_ld_wait();
        // the buffer has been read: hand it back before the arithmetic
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
#pragma unroll
        for (int i = 0; i < 32; ++i) accum[i] = fmaf(__uint_as_float(r0[i]), sc, accum[i]);
#pragma unroll
        for (int i = 0; i < 32; ++i) accum[32 + i] = fmaf(__uint_as_float(r1[i]), sc, accum[32 + i]);
      }
      if (ok && row_ok) {
        bf16* dst = c + (int64_t)row * ldc + n0 + ch0;
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
          if (n0 + ch0 + j * 8 < N) reinterpret_cast<bf16x8*>(dst)[j] = pack8(accum + j * 8);   // N % 8 == 0
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && err_word != nullptr) atomicExch(err_word, 1);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

static int launch_fp8_block(const void* a, const void* w, void* c, const void* a_scale, const void* w_scale, int M,
                            int N, int K, int64_t lda, int64_t ldw, int64_t ldc, const int32_t* tile_expert,
                            int n_experts, cudaStream_t s) {
  using S = FbSmem;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {};
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  if (g_err_word[dev & 63] == nullptr) {
    if (cudaMalloc(&g_err_word[dev & 63], sizeof(int)) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    cudaMemset(g_err_word[dev & 63], 0, sizeof(int));
  }
  CUtensorMap ta, tb;
  const int a_box = M >= kBM ? kBM : ((M + 7) & ~7);
  if (!make_tmap(&ta, a, M, K, lda, a_box, true, true) ||
      !make_tmap(&tb, w, (int64_t)N * n_experts, K, ldw, 128, true, true))
    return (int)cudaErrorInvalidValue;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + 127) / 128);
  const int grid = tiles < 148 ? tiles : 148;
  launch_pdl(gemm_fp8_block_kernel, dim3(grid), dim3(320), (size_t)S::TOTAL, s, ta, tb, (bf16*)c, ldc,
             (const float*)a_scale, (const float*)w_scale, M, N, K, a_box, tile_expert, N, g_err_word[dev & 63]);
  return XLLM_LAUNCH_CHECK();
}

}  // namespace xllm

// Block-scaled fp8 GEMM: C[M,N] (bf16, row stride ldc) = sum_kb (A_q[:, kb] . W_q[:, kb]^T) * a_scale[m, kb] *
// w_scale[n / 128, kb].  A_q [M, K] and W_q [N, K] are e4m3 (row strides lda / ldw bytes); a_scale [M, K / 128]
// and w_scale [ceil(N / 128), K / 128] are fp32, row-major.  K % 128 == 0, N % 8 == 0, 16-byte aligned
// bases, lda / ldw % 16 == 0, ldc % 8 == 0.
XLLM_API int xllm_gemm_fp8_block(const void* a, const void* w, void* c, const void* a_scale, const void* w_scale, int M,
                                 int N, int K, int64_t lda, int64_t ldw, int64_t ldc, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 128 || K == 0 || N % 8 || lda % 16 || ldw % 16 || ldc % 8 || (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15))
    return (int)cudaErrorInvalidValue;
  return launch_fp8_block(a, w, c, a_scale, w_scale, M, N, K, lda, ldw, ldc, nullptr, 1, (cudaStream_t)stream);
}

// Grouped form for MoE experts: the rows of A are sorted by expert and padded so that every 128-row
// tile belongs to one expert, tile_expert[row tile] (device int32, -1 = unused tile).  W_q is
// [n_experts * N, K], w_scale [n_experts * ceil(N / 128), K / 128]; N % 128 == 0.
XLLM_API int xllm_gemm_fp8_block_grouped(const void* a, const void* w, void* c, const void* a_scale,
                                         const void* w_scale, const void* tile_expert, int n_experts, int M, int N,
                                         int K, int64_t lda, int64_t ldw, int64_t ldc, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 128 || K == 0 || N % 128 || lda % 16 || ldw % 16 || ldc % 8 || tile_expert == nullptr ||
      (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15))
    return (int)cudaErrorInvalidValue;
  return launch_fp8_block(a, w, c, a_scale, w_scale, M, N, K, lda, ldw, ldc, (const int32_t*)tile_expert, n_experts,
                          (cudaStream_t)stream);
}

namespace xllm {
}  // namespace xllm

// C[M,N] = A[M,K] · W[N,K]^T (+ bias).  bf16 row-major, leading dimensions in elements.
// Requirements: K % 8 == 0, N % 8 == 0, lda/ldw/ldc % 8 == 0, 16-byte aligned base pointers.
// tile_n: 0 = choose from the problem shape; else one of 64, 128, 192, 256.
// pair: -1 = choose; 0 = one CTA per 128 x tile_n tile; 1 = a CTA pair (cta_group::2) per 256 x tile_n tile.
// w_packed: W is stored tile-packed as [N/64][K/64][64][64] (see xllm_pack_weight_bf16); needs
// N % 64 == 0 and K % 64 == 0.  Each 64 x 64 block is then one contiguous 8 KB run, which is what
// lets a weight-streaming (small M) GEMM pull HBM at full rate.
// split_k: 0 = choose; 1 = off; n > 1 = cut K into (at most) n slices whose fp32 partial tiles meet
// in a per-device scratch; the CTA that arrives last at a tile reduces and stores it.  This is what
// fills all 148 SMs when M x N alone gives fewer tiles than SMs (decode-size batches).
XLLM_API int xllm_gemm_bf16(const void* a, const void* w, void* c, const void* bias, int M, int N, int K,
                            int64_t lda, int64_t ldw, int64_t ldc, int tile_n, int pair, int w_packed,
                            int split_k, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 8 || N % 8 || lda % 8 || ldw % 8 || ldc % 8) return (int)cudaErrorInvalidValue;
  if (w_packed && (N % 64 || K % 64)) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  static int sms = 0;
  if (sms == 0) {
    // XLLM_GEMM_MAX_CTAS caps the persistent grid (for experiments and for leaving SMs to a
    // concurrent communication kernel); default: every SM of a B200
    const char* e = getenv("XLLM_GEMM_MAX_CTAS");
    sms = e ? atoi(e) : 148;
    if (sms < 2 || sms > 148) sms = 148;
  }
  // Split-K sums its fp32 partial tiles with reduce-adds that land in L2 in whatever order the slices finish, so
  // the last bits of a result can differ from run to run.  XLLM_GEMM_DETERMINISTIC=1 turns split-K off (one fixed
  // summation order per output) at the cost of idle SMs on decode-size GEMMs.
  static int deterministic = -1;
  if (deterministic < 0) {
    const char* e = getenv("XLLM_GEMM_DETERMINISTIC");
    deterministic = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  if (deterministic) split_k = 1;
  if ((pair < 0 || tile_n == 0 || split_k == 0) && M <= 512) {
    // Decode-size batches (few row tiles).  Measured on B200: an MMA instruction costs ~75 cycles
    // whatever its width below 128 columns, so tiles narrower than 128 waste the tensor pipe; a
    // 128-wide tile is used while that gives every SM (or SM pair) at most one tile, else 256;
    // left-over SMs are filled by cutting K, as long as a slice keeps enough K to amortise the
    // reduce (~6 us for the scratch round trip).
    const int p = pair >= 0 ? pair : (M > kBM ? 1 : 0);
    const int rows = p ? 2 * kBM : kBM, slots = p ? sms / 2 : sms;
    const int m_t = (M + rows - 1) / rows;
    int tn = tile_n;
    if (tn == 0) {
      // one wave of 128-wide tiles if that fits; else the width (128 / 192 / 256) with the least
      // waves x time per tile, the measured time of a K block growing as ~0.18 + 0.0008 * width us
      if (m_t * ((N + 127) / 128) <= slots) {
        tn = 128;
      } else {
        double best = 1e30;
        for (int cand : {128, 192, 256}) {
          if (cand == 192 && w_packed) continue;
          const long tiles = (long)m_t * ((N + cand - 1) / cand);
          const double cost = (double)((tiles + slots - 1) / slots) * (0.18 + 0.0008 * cand);
          if (cost < best - 1e-9) { best = cost; tn = cand; }
        }
      }
    }
    int sk = split_k;
    if (sk == 0) {
      const int tiles = m_t * ((N + tn - 1) / tn);
      const int min_k = p ? 3072 : 1024;
      sk = slots / tiles;
      if (sk > 8) sk = 8;
      while (sk > 1 && K / sk < min_k) --sk;
      if (sk < 1 || (size_t)M * N * 4 > kSplitWsBytes) sk = 1;
      // pairs, no split, and even 64-wide tiles fit in one wave: the narrower tile is quicker
      // (256 x 4096 x 4096: 15.0 us against 16.4)
      if (tile_n == 0 && p == 1 && sk == 1 && tn == 128 && !w_packed && m_t * ((N + 63) / 64) <= slots) tn = 64;
    }
    pair = p;
    tile_n = tn;
    split_k = sk;
  } else if (pair < 0 || tile_n == 0 || split_k == 0) {
    // Cost model: a tile costs max(operand bytes its SM must pull from L2 at ~85 GB/s per SM,
    // tensor-core time of its MMAs); a launch costs that times the number of waves.
    double best = 1e30;
    int bp = 0, bt = 256;
    for (int p = 0; p < 2; ++p) {
      if (pair >= 0 && p != pair) continue;
      if (p == 1 && M <= kBM) continue;
      for (int tn : {64, 128, 192, 256}) {
        if (tile_n != 0 && tn != tile_n) continue;
        if (tn == 192 && w_packed) continue;
        const int rows = p ? 2 * kBM : kBM, units = p ? sms / 2 : sms;
        const long tiles = (long)((M + rows - 1) / rows) * ((N + tn - 1) / tn);
        const long waves = (tiles + units - 1) / units;
        const double b_rows = p ? tn / 2 : tn;
        const double t_in = ((double)kBM + b_rows) * K * 2.0 / 85e9;
        const double t_mma = (K / 16.0) * (tn > 150 ? tn / 2.0 : 75.0) / 1.8e9;
        const double t_epi = 128.0 * tn * 2.0 / 200e9;
        const double cost = waves * ((t_in > t_mma ? t_in : t_mma) + 0.3 * t_epi) + t_epi;
        if (cost < best) { best = cost; bp = p; bt = tn; }
      }
    }
    pair = bp;
    tile_n = bt;
    if (split_k == 0) split_k = 1;
  }
  // narrow tiles take two K blocks per ring stage unless the weight is tile-packed (whose block
  // addressing has no zero-filled tail) or the caller asked for the one-block form
  const bool two = g_k_per_stage != 1 && !w_packed && K > kBK;
  if (tile_n == 192 && w_packed) tile_n = 256;  // packed blocks are 64 rows: a 96-row half tile would straddle them
  if (pair) {
    switch (tile_n) {
      case 256: return launch_gemm_pair<256, 6>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
      case 192: return launch_gemm_pair<192, 6>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
      case 128:
        if (two && g_dual) return launch_gemm_pair<128, 4, 2, true>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
        if (two) return launch_gemm_pair<128, 4, 2>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
        return launch_gemm_pair<128, 8>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
      case 64:
        if (two && g_dual) return launch_gemm_pair<64, 4, 2, true>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
        if (two) return launch_gemm_pair<64, 4, 2>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
        return launch_gemm_pair<64, 9>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, split_k);
      default: return (int)cudaErrorInvalidValue;
    }
  }
  const GemmMode plain{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0};
  if (two && g_dual && tile_n == 128)
    return launch_gemm<128, 6, 1, true>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1, plain, split_k);
  if (two && g_dual && tile_n == 64)
    return launch_gemm<64, 4, 2, true>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1, plain, split_k);
  if (two && tile_n == 128)
    return launch_gemm<128, 3, 2>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1, plain, split_k);
  if (two && tile_n == 64)
    return launch_gemm<64, 4, 2>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1, plain, split_k);
  switch (tile_n) {
    case 192: return launch_gemm<192, 4>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1, plain, split_k);
    case 256: return launch_gemm<256, 4>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1,
                                          GemmMode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0}, split_k);
    case 128: return launch_gemm<128, 6>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1,
                                          GemmMode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0}, split_k);
    case 64: return launch_gemm<64, 8>(a, w, c, bias, M, N, K, lda, ldw, ldc, sms, w_packed, s, nullptr, 1,
                                          GemmMode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0}, split_k);
    default: return (int)cudaErrorInvalidValue;
  }
}

// Row-parallel linear fused with the scatter half of a reduce-scatter (see GemmMode "push mode").
// a [M, K] and w [N, K] are this rank's operands; nothing is written locally: row r of the partial
// product goes to rank r / S, into inbox[rank][r % S][:] at byte offset `inbox_off` of that rank's
// symmetric buffer, and the rank's arrival counter (uint32 `sig_idx` of its signal pad) grows by
// one per (row, column tile).  The owner therefore expects rows_owned * ceil(N / tile_n) * world
// arrivals.  tile_n: 128 or 256.  peer_bufs / signal_pads: device arrays of `world` pointers.
XLLM_API int xllm_gemm_bf16_push(const void* a, const void* w, const void* peer_bufs, const void* signal_pads,
                                 int64_t inbox_off, int64_t sig_idx, int M, int N, int K, int64_t lda, int64_t ldw,
                                 int S, int rank, int world, int tile_n, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 8 || N % 8 || lda % 8 || ldw % 8 || (inbox_off & 15) || S <= 0 || (int64_t)S * world < M)
    return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)w) & 15) return (int)cudaErrorInvalidValue;
  GemmMode mode{nullptr, nullptr, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, (void* const*)peer_bufs,
                (void* const*)signal_pads, inbox_off, sig_idx, S, rank, world};
  cudaStream_t s = (cudaStream_t)stream;
  if (tile_n == 256)
    return launch_gemm<256, 4>(a, w, const_cast<void*>(a), nullptr, M, N, K, lda, ldw, lda, 148, 0, s, nullptr, 1, mode);
  if (tile_n == 128)
    return launch_gemm<128, 3, 2>(a, w, const_cast<void*>(a), nullptr, M, N, K, lda, ldw, lda, 148, 0, s, nullptr, 1, mode);
  return (int)cudaErrorInvalidValue;
}

// Grouped (mixture-of-experts) GEMM: rows of A are grouped by expert in 128-row tiles
// (tile_expert[i] = expert of row tile i, -1 = unused); W is [n_experts, N, K].
// C[rows of tile i, :] = A[rows of tile i, :] · W[tile_expert[i]]^T.  M is the padded row count.
// N must be a multiple of the tile width so that a tile never mixes two experts' weights.
XLLM_API int xllm_gemm_bf16_grouped(const void* a, const void* w, void* c, const void* tile_expert, int M, int N,
                                    int K, int n_experts, int64_t lda, int64_t ldc, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 8 || N % 64 || lda % 8 || ldc % 8 || M % kBM) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const int32_t* te = (const int32_t*)tile_expert;
  if (N % 256 == 0) return launch_gemm<256, 4>(a, w, c, nullptr, M, N, K, lda, K, ldc, 148, 0, s, te, n_experts);
  if (N % 128 == 0) return launch_gemm<128, 6>(a, w, c, nullptr, M, N, K, lda, K, ldc, 148, 0, s, te, n_experts);
  return launch_gemm<64, 8>(a, w, c, nullptr, M, N, K, lda, K, ldc, 148, 0, s, te, n_experts);
}

// Grouped GEMM with the gated activation in the epilogue: every expert's N rows (gate | up) are stored
// interleaved in groups of 128 = [64 gate rows | the 64 up rows of the same features], as for
// xllm_gemm_bf16_act_mul; C is [M, N / 2] = act(gate) * up, and the [M, N] intermediate is never written.
XLLM_API int xllm_gemm_bf16_grouped_act_mul(const void* a, const void* w, void* c, const void* tile_expert, int M,
                                            int N, int K, int n_experts, int64_t lda, int64_t ldc, int act,
                                            void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 8 || N % 128 || lda % 8 || ldc % 8 || M % kBM || act < 1 || act > 3) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const int32_t* te = (const int32_t*)tile_expert;
  GemmMode mode{};
  mode.ks = 1;
  mode.act_mul = act;
  if (N % 256 == 0) return launch_gemm<256, 4>(a, w, c, nullptr, M, N, K, lda, K, ldc, 148, 0, s, te, n_experts, mode);
  return launch_gemm<128, 6>(a, w, c, nullptr, M, N, K, lda, K, ldc, 148, 0, s, te, n_experts, mode);
}

// fp8 (e4m3) scaled GEMM: C[M,N] (bf16) = (A_fp8[M,K] · W_fp8[N,K]^T) * a_scale * b_scale (+ bias).
// a_scale: one float (per tensor) or M floats (per token, a_per_row = 1); b_scale: one float or N
// floats (per output channel, b_per_col = 1).  K % 16 == 0; leading dimensions in elements (= bytes).
// Same capability as the reference's CUTLASS scaled_mm for sm_100
// (xllm/core/kernels/cuda/cutlass_w8a8/c3x/scaled_mm_sm100_fp8_dispatch.cuh:34-429).
XLLM_API int xllm_gemm_fp8(const void* a, const void* w, void* c, const void* bias, const void* a_scale,
                           const void* b_scale, int a_per_row, int b_per_col, int M, int N, int K, int64_t lda,
                           int64_t ldw, int64_t ldc, void* stream) {
  using namespace xllm;
  if (M == 0 || N == 0) return 0;
  if (K % 16 || N % 8 || lda % 16 || ldw % 16 || ldc % 8) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) return (int)cudaErrorInvalidValue;
  GemmMode mode{(const float*)a_scale, (const float*)b_scale, 1, a_per_row, b_per_col, 1, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0, 0};
  cudaStream_t s = (cudaStream_t)stream;
  const int mt = (M + kBM - 1) / kBM;
  int tile_n = 256;
  while (tile_n > 64 && mt * ((N + tile_n - 1) / tile_n) < 148) tile_n >>= 1;
  if (tile_n == 256) return launch_gemm<256, 4>(a, w, c, bias, M, N, K, lda, ldw, ldc, 148, 0, s, nullptr, 1, mode);
  if (tile_n == 128) return launch_gemm<128, 6>(a, w, c, bias, M, N, K, lda, ldw, ldc, 148, 0, s, nullptr, 1, mode);
  return launch_gemm<64, 8>(a, w, c, bias, M, N, K, lda, ldw, ldc, 148, 0, s, nullptr, 1, mode);
}

namespace xllm {
// dst[(n/64), (k/64), n%64, k%64] = src[n, k]; one thread moves 16 bytes
__global__ void pack_weight_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int N, int K, int64_t ld) {
  const int kc = K >> 3;  // 16-byte chunks per source row
  const int64_t total = (int64_t)N * kc;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / kc;
    const int c = (int)(i - n * kc);
    const int kb = c >> 3, cc = c & 7;
    const int64_t d = (((n >> 6) * (K >> 6) + kb) * 64 + (n & 63)) * 8 + cc;
    dst[d] = src[n * (ld >> 3) + c];
  }
}
}  // namespace xllm

// Re-lay a row-major bf16 weight [N, K] (row stride ld) into the tile-packed form.  dst != src.
XLLM_API int xllm_pack_weight_bf16(void* dst, const void* src, int N, int K, int64_t ld, void* stream) {
  using namespace xllm;
  if (N % 64 || K % 64 || ld % 8 || dst == src) return (int)cudaErrorInvalidValue;
  pack_weight_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, N, K, ld);
  return XLLM_LAUNCH_CHECK();
}

// 1 = one 64-element K block per ring stage everywhere; 2 (default) = two for tiles narrower than 256.
XLLM_API void xllm_gemm_set_k_per_stage(int n) { xllm::g_k_per_stage = n == 1 ? 1 : 2; }
// 1 = the narrow-tile kernels use two MMA-issuing warps; 0 (default) = one.
XLLM_API void xllm_gemm_set_dual_issue(int on) { xllm::g_dual = on ? 1 : 0; }

// Allocate the per-device split-K scratch now (call once per device before capturing CUDA graphs).
XLLM_API int xllm_gemm_prepare() {
  using namespace xllm;
  int dev = 0;
  cudaGetDevice(&dev);
  return split_scratch_ready(dev, nullptr) ? 0 : (int)cudaErrorMemoryAllocation;
}

// 0 = no bounded wait has expired on this device since the last call; the word is cleared.
XLLM_API int xllm_gemm_error_status() {
  using namespace xllm;
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_err_word[dev & 63] == nullptr) return 0;
  int v = 0;
  cudaMemcpy(&v, g_err_word[dev & 63], sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) {
    cudaMemset(g_err_word[dev & 63], 0, sizeof(int));
    // an aborted split-K launch may have left arrival counters half-way
    if (g_split_cnt[dev & 63] != nullptr) {
      cudaMemset(g_split_cnt[dev & 63], 0, kSplitCounters * sizeof(int));
      cudaMemset(g_split_ws[dev & 63], 0, kSplitWsBytes);
    }
  }
  return v;
}
