// Tensor-parallel communication kernels over NVLink / NVSwitch peer memory.
//
//   xllm_tp_allreduce_norm : out = RMSNorm(sum_ranks(x) + residual) * w   (or plain sum)
//
// This is the all-reduce that follows every row-parallel linear (o_proj, down_proj) fused with the
// residual add and the RMSNorm that always comes next.  The reference issues an NCCL all-reduce
// from RowParallelLinear (xllm/core/layers/common/linear.cpp:1938-1940) and then a separate
// fused_add_rms_norm launch; its Python path replaces small all-reduces by torch's symmetric-memory
// one-shot kernel (xllm/python/distributed/collectives.py:258-312).
//
// Algorithm (two-shot, sequence-sharded): every rank's partial x lives at the same offset of a
// symmetric buffer.  Rank r owns rows [r*S, (r+1)*S), S = ceil(T / world).
//   barrier 1  all partials are complete and visible
//   reduce     owner pulls its rows: one `multimem.ld_reduce` per 16 bytes when the buffer is bound
//              to an NVSwitch multicast object (the switch adds the replicas), else plain loads from
//              every peer pointer, fp32 accumulation
//   epilogue   + residual shard (kept only by the owner, updated in place), RMSNorm, * weight
//   broadcast  the normalised rows go to every rank's `out`: one `multimem.st`, or a store per peer
//   barrier 2  every rank's `out` is complete; partial buffers may be overwritten
// A barrier is a flag exchange through the symmetric signal pad: a growing epoch stored into slot
// [my rank] of every peer by one CTA, then a wait on the own slots.  For the opening barrier EVERY CTA
// polls the own slots (local memory), so no CTA waits for another CTA of its grid and the grid may be
// of any size; the closing one is run by the last CTA to finish.  Rows are spread over thread groups
// (rowops.cuh), several rows per CTA.  Every wait is bounded;
// when the budget runs out the kernel sets an error word and carries on (results are then
// undefined, the GPU stays healthy and the host can see the error).  Epoch counters live in device
// memory and are advanced by the kernel itself, so the launch can be replayed from a CUDA graph.
//
//   xllm_tp_inbox_norm : the owner's half of the fused GEMM -> reduce-scatter.  The row-parallel GEMM
// of every rank has pushed its partial rows into this rank's inbox [world][S][H] (gemm_tcgen05.cu,
// push mode) and bumped this rank's arrival counter.  This kernel waits (bounded) for the counter to
// reach the expected count, sums the `world` inbox slices of each owned row in fp32, adds the
// residual shard, applies RMSNorm and broadcasts the normalised rows to every rank's `out`
// (`multimem.st` or peer stores), then runs the closing flag exchange.  There is no opening
// barrier: an arrival from a peer already proves that the peer's earlier kernels have finished.
#include "rowops.cuh"
#include <algorithm>

namespace xllm {

constexpr int kCommThreads = 256;
constexpr int kCommMaxVec = 8;
constexpr int kMaxRanks = 16;
// Budget of every flag wait, in SM clock cycles (about two seconds by default).  It is a launch
// parameter: the launchers copy this host value into the kernel parameters, and
// xllm_comm_set_wait_budget() changes it (tests make a wait run out with a short budget).
static long long g_wait_budget_cycles = 4000000000LL;

struct TpNormParams {
  void* const* peer_bufs;     // [world] base pointers of the symmetric buffer on every rank
  void* const* signal_pads;   // [world] base pointers of the signal pads
  uint64_t mc_base;           // multicast address of the symmetric buffer, 0 = none
  int64_t x_off, out_off;     // byte offsets inside the symmetric buffer
  int64_t sig_off;            // uint32 offset of this op's flag area inside the signal pad
  uint32_t* epochs;           // local state: [0] epoch, [1] go flag, [2] arrival counter
  bf16* residual;             // [S, H] local shard, updated in place; null for plain all-reduce
  const bf16* weight;         // [H]; null for plain all-reduce
  int* err;                   // error word
  int T, H, rank, world, mode;  // mode 0: out = sum ; 1: out = rmsnorm(sum + residual) * w
  float eps;
  long long budget;           // cycles a flag wait may take before the error word is set
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Cross-rank flag exchange done by ONE CTA (threads 0..world-1): store `epoch` into my slot of
// every peer's signal pad, then wait until every peer's slot in my pad has reached it.
__device__ __forceinline__ void exchange_flags(const TpNormParams& p, uint32_t epoch) {
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    uint32_t* remote = reinterpret_cast<uint32_t*>(p.signal_pads[peer]) + p.sig_off + p.rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.signal_pads[p.rank]) + p.sig_off + peer;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > p.budget) {
        atomicExch(p.err, 1 + peer);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(uint64_t mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16(uint64_t mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Closing exchange shared by both kernels: the last CTA to finish tells the peers and waits for
// theirs, so that the completion of the kernel means `out` is complete on this rank.
__device__ __forceinline__ void closing_barrier(const TpNormParams& p, volatile uint32_t* state, uint32_t e0,
                                                int* s_last, uint32_t* reset_word) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(const_cast<uint32_t*>(&state[2]), 1u);
    *s_last = prev == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (*s_last) {
    // every CTA of this rank has consumed the inbox: the counter may restart before any peer is
    // told that this rank is done (a peer only pushes again after it has seen that flag)
    if (reset_word != nullptr && threadIdx.x == 0) {
      *reset_word = 0u;
      __threadfence_system();
    }
    __syncthreads();
    exchange_flags(p, e0 + 2);
    if (threadIdx.x == 0) {
      state[2] = 0;
      state[0] = e0 + 2;
      __threadfence();
    }
  }
}

__global__ void __launch_bounds__(kCommThreads) tp_inbox_norm_kernel(TpNormParams p, int64_t counter_idx,
                                                                     uint32_t expected) {
  __shared__ float red[32];
  __shared__ int s_last;
  volatile uint32_t* state = p.epochs;
  const uint32_t e0 = state[0];
  const int S = (p.T + p.world - 1) / p.world;
  const int row_begin = p.rank * S;
  const int row_end = min(row_begin + S, p.T);
  const int nvec = p.H >> 3;
  uint32_t* counter = reinterpret_cast<uint32_t*>(p.signal_pads[p.rank]) + counter_idx;
  pdl_wait();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    while (ld_acquire_sys(counter) < expected) {
      if (clock64() - t0 > p.budget) {
        atomicExch(p.err, 200);
        break;
      }
    }
  }
  __syncthreads();
  const uint8_t* inbox = reinterpret_cast<const uint8_t*>(p.peer_bufs[p.rank]) + p.x_off;
  for (int row = row_begin + blockIdx.x; row < row_end; row += gridDim.x) {
    float vals[kCommMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kCommMaxVec; ++i) {
      const int v = threadIdx.x + i * kCommThreads;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
        for (int k = 0; k < p.world; ++k) {
          const int64_t off = (((int64_t)k * S + (row - row_begin)) * p.H) * 2 + (int64_t)v * 16;
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(inbox + off));
          float f[8];
          unpack8(*reinterpret_cast<const bf16x8*>(&raw), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += f[j];
        }
        if (p.mode == 1) {
          bf16x8* rr = reinterpret_cast<bf16x8*>(p.residual + (int64_t)(row - row_begin) * p.H) + v;
          float r[8];
          unpack8(*rr, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
          const bf16x8 nr = pack8(vals[i]);
          *rr = nr;
          unpack8(nr, vals[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
      }
    }
    float inv = 1.f;
    if (p.mode == 1) {
      ss = block_sum(ss, red);
      inv = rsqrtf(ss / (float)p.H + p.eps);
    }
    const int64_t row_byte = (int64_t)row * p.H * 2;
#pragma unroll
    for (int i = 0; i < kCommMaxVec; ++i) {
      const int v = threadIdx.x + i * kCommThreads;
      if (v < nvec) {
        float o[8];
        if (p.mode == 1) {
          float w[8];
          unpack8(reinterpret_cast<const bf16x8*>(p.weight)[v], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * w[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j];
        }
        const bf16x8 ob = pack8(o);
        const uint4 u = *reinterpret_cast<const uint4*>(&ob);
        const int64_t off = p.out_off + row_byte + (int64_t)v * 16;
        if (p.mc_base != 0) {
          multimem_st_16(p.mc_base + off, u);
        } else {
          for (int k = 0; k < p.world; ++k) {
            const int peer = (p.rank + k) % p.world;
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_bufs[peer]) + off) = u;
          }
        }
      }
    }
  }
  closing_barrier(p, state, e0, &s_last, counter);
  pdl_launch_dependents();
}


// ------------------------------------------------------------------------------------------------
//   xllm_tp_oneshot_norm : one-shot form of the fused all-reduce for messages of a few MB.
//
// Every rank reduces ALL rows itself: with the buffer bound to an NVSwitch multicast object one
// `multimem.ld_reduce` per 16 bytes returns the sum over the ranks (the switch adds the replicas, so
// the bytes that enter this GPU are those of one copy of the message); without it the rank reads the
// row from every peer.  Residual add, RMSNorm and the store are local: the residual stream is
// replicated, nothing is broadcast and there is no closing barrier.
//   signal   CTA 0 stores the call's epoch into this rank's slot of every peer's signal pad
//   wait     EVERY CTA polls the `world` slots of its own pad (local memory) until they reach the
//            epoch - no CTA waits for another CTA of the grid, so the grid need not be co-resident
//   reduce   rows are spread over thread groups (rowops.cuh): several rows per CTA
// What makes the missing closing barrier safe: the caller alternates between two partial buffers
// (`x_off` of consecutive calls differ).  A rank can only pass the wait of call n+1 after every rank
// has entered call n+1, i.e. finished reading in call n; so when a rank overwrites the buffer of call
// n (for call n+2) nobody reads it any more.
struct TpOneShotParams {
  void* const* peer_bufs;
  void* const* signal_pads;
  uint64_t mc_base;
  int64_t x_off;              // byte offset of this call's partial buffer in the symmetric buffer
  int64_t sig_off;            // uint32 offset of the flag slots [world] in the signal pad
  uint32_t* state;            // local: [0] epoch of the last finished call, [1] CTA arrival counter
  const bf16* residual_in;    // [T, H] or null (treated as zero)
  bf16* residual_out;         // [T, H] or null; may alias residual_in
  const bf16* weight;         // [H] or null: no normalisation, out = sum (+ residual)
  bf16* out;                  // [T, H] local
  int* err;
  int T, H, rank, world;
  float eps;
  long long budget;
};

__device__ __forceinline__ bool wait_flags(void* const* signal_pads, int64_t sig_off, int rank, int world,
                                           uint32_t epoch, long long budget, int* err, int code) {
  bool ok = true;
  if (threadIdx.x < world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(signal_pads[rank]) + sig_off + threadIdx.x;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > budget) {
        atomicExch(err, code + (int)threadIdx.x);
        ok = false;
        break;
      }
    }
  }
  return ok;
}

template <int TPR>
__global__ void __launch_bounds__(kRowThreads) tp_oneshot_norm_kernel(TpOneShotParams p) {
  __shared__ float red[8];
  constexpr int R = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = p.H >> 3;
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;
  if (blockIdx.x == 0 && threadIdx.x < p.world)   // the release store orders the earlier kernels' writes before the flag
    st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, epoch);
  bool waited = false;
  for (int64_t row0 = (int64_t)blockIdx.x * R; row0 < p.T; row0 += (int64_t)gridDim.x * R) {
    const int64_t row = row0 + threadIdx.x / TPR;
    const bool active = row < p.T;
    const int64_t row_byte = row * p.H * 2;
    // what is local goes first: the residual rows are in flight while the flags travel
    uint4 rres[kRowMaxVec];
    if (p.residual_in != nullptr) {
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) rres[i] = __ldg(reinterpret_cast<const uint4*>(p.residual_in + row * p.H) + v);
      }
    }
    if (!waited) {
      wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, epoch, p.budget, p.err, 300);
      __syncthreads();
      waited = true;
    }
    float vals[kRowMaxVec][8];
    float ss = 0.f;
    if (p.mc_base != 0) {
      // all loads of the row in flight before the first use
      uint4 raw[kRowMaxVec];
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) raw[i] = multimem_ld_reduce_bf16x8(p.mc_base + p.x_off + row_byte + (int64_t)v * 16);
      }
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) unpack8(*reinterpret_cast<const bf16x8*>(&raw[i]), vals[i]);
      }
    } else {
      for (int k = 0; k < p.world; ++k) {
        // fixed order (rank 0 first) so that every rank adds the same numbers in the same order
        uint4 raw[kRowMaxVec];
#pragma unroll
        for (int i = 0; i < kRowMaxVec; ++i) {
          const int v = t + i * TPR;
          if (active && v < nvec)
            raw[i] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.peer_bufs[k]) + p.x_off +
                                                           row_byte + (int64_t)v * 16));
        }
#pragma unroll
        for (int i = 0; i < kRowMaxVec; ++i) {
          const int v = t + i * TPR;
          if (active && v < nvec) {
            float f[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&raw[i]), f);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] = (k == 0 ? 0.f : vals[i][j]) + f[j];
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      const int v = t + i * TPR;
      if (active && v < nvec) {
        if (p.residual_in != nullptr) {
          float r[8];
          unpack8(*reinterpret_cast<const bf16x8*>(&rres[i]), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
        }
        const bf16x8 nr = pack8(vals[i]);  // the residual stream is bf16: round once
        if (p.residual_out != nullptr) reinterpret_cast<bf16x8*>(p.residual_out + row * p.H)[v] = nr;
        unpack8(nr, vals[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    float inv = 1.f;
    if (p.weight != nullptr) {
      ss = group_sum<TPR>(ss, red);
      inv = rsqrtf(ss / (float)p.H + p.eps);
    }
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      const int v = t + i * TPR;
      if (active && v < nvec) {
        float o[8];
        if (p.weight != nullptr) {
          float w[8];
          unpack8(reinterpret_cast<const bf16x8*>(p.weight)[v], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * w[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j];
        }
        reinterpret_cast<bf16x8*>(p.out + row * p.H)[v] = pack8(o);
      }
    }
  }
  // the last CTA to finish publishes the epoch for the next call of this communicator
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(p.state + 1, 1u);
    if (prev == gridDim.x - 1) {
      p.state[1] = 0u;
      *reinterpret_cast<volatile uint32_t*>(p.state) = epoch;
      __threadfence();
    }
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
//   two-shot kernel of xllm_tp_allreduce_norm (algorithm in the header of this file)
template <int TPR>
__global__ void __launch_bounds__(kRowThreads) tp_twoshot_norm_kernel(TpNormParams p) {
  __shared__ float red[8];
  __shared__ int s_last;
  constexpr int R = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = p.H >> 3;
  const int S = (p.T + p.world - 1) / p.world;
  const int row_begin = p.rank * S;
  const int row_end = min(row_begin + S, p.T);
  pdl_wait();
  const uint32_t e0 = *reinterpret_cast<volatile uint32_t*>(p.epochs);
  if (blockIdx.x == 0 && threadIdx.x < p.world)
    st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, e0 + 1);
  bool waited = false;
  for (int64_t row0 = row_begin + (int64_t)blockIdx.x * R; row0 < row_end; row0 += (int64_t)gridDim.x * R) {
    const int64_t row = row0 + threadIdx.x / TPR;
    const bool active = row < row_end;
    const int64_t row_byte = row * p.H * 2;
    uint4 rres[kRowMaxVec];
    if (p.mode == 1) {
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) rres[i] = *(reinterpret_cast<const uint4*>(p.residual + (row - row_begin) * p.H) + v);
      }
    }
    if (!waited) {
      wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, e0 + 1, p.budget, p.err, 1);
      __syncthreads();
      waited = true;
    }
    float vals[kRowMaxVec][8];
    float ss = 0.f;
    if (p.mc_base != 0) {
      uint4 raw[kRowMaxVec];
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) raw[i] = multimem_ld_reduce_bf16x8(p.mc_base + p.x_off + row_byte + (int64_t)v * 16);
      }
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) unpack8(*reinterpret_cast<const bf16x8*>(&raw[i]), vals[i]);
      }
    } else {
      for (int k = 0; k < p.world; ++k) {
        const int peer = (p.rank + k) % p.world;  // start at home, spread the link load
        uint4 raw[kRowMaxVec];
#pragma unroll
        for (int i = 0; i < kRowMaxVec; ++i) {
          const int v = t + i * TPR;
          if (active && v < nvec)
            raw[i] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.peer_bufs[peer]) +
                                                           p.x_off + row_byte + (int64_t)v * 16));
        }
#pragma unroll
        for (int i = 0; i < kRowMaxVec; ++i) {
          const int v = t + i * TPR;
          if (active && v < nvec) {
            float f[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&raw[i]), f);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] = (k == 0 ? 0.f : vals[i][j]) + f[j];
          }
        }
      }
    }
    if (p.mode == 1) {
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i) {
        const int v = t + i * TPR;
        if (active && v < nvec) {
          float r[8];
          unpack8(*reinterpret_cast<const bf16x8*>(&rres[i]), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
          const bf16x8 nr = pack8(vals[i]);  // the residual stream is bf16: round once
          reinterpret_cast<bf16x8*>(p.residual + (row - row_begin) * p.H)[v] = nr;
          unpack8(nr, vals[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
      }
    }
    float inv = 1.f;
    if (p.mode == 1) {
      ss = group_sum<TPR>(ss, red);
      inv = rsqrtf(ss / (float)p.H + p.eps);
    }
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      const int v = t + i * TPR;
      if (active && v < nvec) {
        float o[8];
        if (p.mode == 1) {
          float w[8];
          unpack8(reinterpret_cast<const bf16x8*>(p.weight)[v], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * w[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j];
        }
        const bf16x8 ob = pack8(o);
        const uint4 u = *reinterpret_cast<const uint4*>(&ob);
        const int64_t off = p.out_off + row_byte + (int64_t)v * 16;
        if (p.mc_base != 0) {
          multimem_st_16(p.mc_base + off, u);
        } else {
          for (int k = 0; k < p.world; ++k) {
            const int peer = (p.rank + k) % p.world;
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_bufs[peer]) + off) = u;
          }
        }
      }
    }
  }
  if (!waited) {   // a CTA without rows still may not run ahead of the opening barrier
    wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, e0 + 1, p.budget, p.err, 1);
  }
  // closing barrier: the last CTA to finish tells the peers that this rank's rows have been
  // broadcast and waits for theirs, so that completion of the kernel means `out` is complete here
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(p.epochs + 2, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, e0 + 2);
    }
    wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, e0 + 2, p.budget, p.err, 1);
    __syncthreads();
    if (threadIdx.x == 0) {
      p.epochs[2] = 0u;
      *reinterpret_cast<volatile uint32_t*>(p.epochs) = e0 + 2;
      __threadfence();
    }
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
//   xllm_tp_argmax : greedy sampling over vocabulary-sharded logits without gathering them.
//
// One CTA per row finds the maximum of the local shard and stores (value, global index) into slot
// [parity][rank][row] of EVERY rank's pair area (plain peer stores, 8 bytes per row and peer).  The
// last CTA to finish runs the flag exchange (bounded) and then picks, for every row, the best pair
// over the ranks (ties: lowest index), so all ranks write identical ids.  parity = epoch & 1: a rank
// can be at most one call ahead of a peer that still reads the previous call's pairs.
struct TpArgmaxParams {
  const bf16* logits;         // [B, Vs] local shard
  int64_t row_stride;
  void* const* peer_bufs;
  void* const* signal_pads;
  int64_t pair_off;           // byte offset of the pair area [2][world][max_rows] x 8 bytes
  int64_t sig_off;
  uint32_t* state;            // [0] epoch, [1] CTA arrival counter
  int64_t* out_ids;           // [B]
  int* err;
  int B, Vs, vocab_start, max_rows, rank, world;
  long long budget;
};

__global__ void __launch_bounds__(256) tp_argmax_kernel(TpArgmaxParams p) {
  __shared__ float redv[32];
  __shared__ int redi[32];
  __shared__ int s_last;
  const int row = blockIdx.x;
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;
  const int parity = (int)(epoch & 1u);
  const bf16* x = p.logits + (int64_t)row * p.row_stride;
  float mx = -INFINITY;
  int arg = 0x7fffffff;
  // 8 values per 16-byte load where the row allows it
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  const int nvec = vec_ok ? (p.Vs >> 3) : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (f[j] > mx) { mx = f[j]; arg = v * 8 + j; }
  }
  for (int i = nvec * 8 + threadIdx.x; i < p.Vs; i += blockDim.x) {
    const float f = __bfloat162float(x[i]);
    if (f > mx || (f == mx && i < arg)) { mx = f; arg = i; }
  }
  // block arg-max, ties to the lowest index
  {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
      const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > mx || (ov == mx && oi < arg)) { mx = ov; arg = oi; }
    }
    if (lane == 0) { redv[wid] = mx; redi[wid] = arg; }
    __syncthreads();
    const int nw = blockDim.x >> 5;
    mx = lane < nw ? redv[lane] : -INFINITY;
    arg = lane < nw ? redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
      const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > mx || (ov == mx && oi < arg)) { mx = ov; arg = oi; }
    }
  }
  if (threadIdx.x < p.world) {
    const int64_t slot = ((int64_t)parity * p.world + p.rank) * p.max_rows + row;
    int2 pr;
    pr.x = __float_as_int(mx);
    pr.y = arg == 0x7fffffff ? 0x7fffffff : arg + p.vocab_start;
    *reinterpret_cast<int2*>(reinterpret_cast<uint8_t*>(p.peer_bufs[threadIdx.x]) + p.pair_off + slot * 8) = pr;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(p.state + 1, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  // every CTA of this rank has stored its pairs: tell the peers, wait for theirs
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, epoch);
  }
  wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, epoch, p.budget, p.err, 400);
  __syncthreads();
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(p.peer_bufs[p.rank]) + p.pair_off;
  for (int r = threadIdx.x; r < p.B; r += blockDim.x) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = 0; k < p.world; ++k) {
      const int64_t slot = ((int64_t)parity * p.world + k) * p.max_rows + r;
      const int2 pr = __ldcg(reinterpret_cast<const int2*>(mine + slot * 8));
      const float v = __int_as_float(pr.x);
      if (v > bv || (v == bv && pr.y < bi)) { bv = v; bi = pr.y; }
    }
    p.out_ids[r] = bi == 0x7fffffff ? 0 : bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.state[1] = 0u;
    *reinterpret_cast<volatile uint32_t*>(p.state) = epoch;
    __threadfence();
  }
}

// ------------------------------------------------------------------------------------------------
//   xllm_tp_gather_cols : all-gather of column shards (vocabulary-sharded logits -> full rows).
//
// Every rank copies its [B, Vs] shard into columns [rank * Vs, (rank + 1) * Vs) of the [B, V_pad]
// area of EVERY rank (16-byte peer stores, or one `multimem.st` when a multicast mapping exists).  The
// last CTA to finish runs the flag exchange, so completion of the kernel on a rank means that all
// shards have landed in that rank's area.
struct TpGatherParams {
  const bf16* src;            // [B, Vs] local shard
  int64_t src_stride;
  void* const* peer_bufs;
  void* const* signal_pads;
  uint64_t mc_base;
  int64_t dst_off;            // byte offset of the gathered area in the symmetric buffer
  int64_t dst_stride;         // elements per gathered row (>= world * Vs)
  int64_t sig_off;
  uint32_t* state;
  int* err;
  int B, Vs, rank, world;
  long long budget;
};

__global__ void __launch_bounds__(256) tp_gather_cols_kernel(TpGatherParams p) {
  __shared__ int s_last;
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;
  const int nvec = p.Vs >> 3;
  const int64_t total = (int64_t)p.B * nvec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / nvec;
    const int v = (int)(i - r * nvec);
    const uint4 u = *reinterpret_cast<const uint4*>(p.src + r * p.src_stride + (int64_t)v * 8);
    const int64_t off = p.dst_off + (r * p.dst_stride + (int64_t)p.rank * p.Vs + (int64_t)v * 8) * 2;
    if (p.mc_base != 0) {
      multimem_st_16(p.mc_base + off, u);
    } else {
      for (int k = 0; k < p.world; ++k) {
        const int peer = (p.rank + k) % p.world;
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_bufs[peer]) + off) = u;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(p.state + 1, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, epoch);
  }
  wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, epoch, p.budget, p.err, 500);
  __syncthreads();
  if (threadIdx.x == 0) {
    p.state[1] = 0u;
    *reinterpret_cast<volatile uint32_t*>(p.state) = epoch;
    __threadfence();
  }
}

// ---------------------------------------------------------------------------------- permuting all-to-all
// Ulysses sequence parallelism: x [d0, d1, d2, E] on every rank; dimension `scatter` (1 or 2) is cut
// into `world` parts, part r goes to rank r, and what arrives is laid out along the OTHER of the two
// dimensions in rank order -- the layout change and the exchange in one pass of peer stores:
//   mode 0 (scatter d1, gather d2): out [d0, d1 / n, n * d2, E]  (sequence-sharded -> head-sharded)
//   mode 1 (scatter d2, gather d1): out [d0, n * d1, d2 / n, E]  (head-sharded -> sequence-sharded)
// E elements of 2 bytes, E % 8 == 0.  The receive area is double-buffered by call parity, so a rank may
// run ahead into the next call while a peer still reads the previous result; the caller copies the
// result out before the call after next.
struct A2aParams {
  const bf16* x;
  void* const* peer_bufs;
  void* const* signal_pads;
  int64_t recv_off;           // byte offset of the receive area ([2 halves] of half_bytes)
  int64_t half_bytes;
  int64_t sig_off;
  uint32_t* state;            // [0] epoch, [1] arrival counter
  int* err;
  int d0, d1, d2, E, mode, rank, world;
  long long budget;
};

__global__ void __launch_bounds__(256) a2a_permute_kernel(A2aParams p) {
  __shared__ int s_last;
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;
  const int64_t half = (int64_t)(epoch & 1u) * p.half_bytes;
  const int ev = p.E >> 3;
  const int n = p.world;
  const int64_t total = (int64_t)p.d0 * p.d1 * p.d2 * ev;
  const int d1s = p.d1 / n, d2s = p.d2 / n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % ev);
    int64_t r = i / ev;
    const int i2 = (int)(r % p.d2);
    r /= p.d2;
    const int i1 = (int)(r % p.d1);
    const int i0 = (int)(r / p.d1);
    int dst;
    int64_t idx;
    if (p.mode == 0) {
      dst = i1 / d1s;
      idx = (((int64_t)i0 * d1s + (i1 - dst * d1s)) * ((int64_t)n * p.d2) + (int64_t)p.rank * p.d2 + i2) * p.E;
    } else {
      dst = i2 / d2s;
      idx = (((int64_t)i0 * ((int64_t)n * p.d1) + (int64_t)p.rank * p.d1 + i1) * d2s + (i2 - dst * d2s)) * p.E;
    }
    const uint4 u = *reinterpret_cast<const uint4*>(p.x + (((int64_t)i0 * p.d1 + i1) * p.d2 + i2) * p.E + (int64_t)v * 8);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_bufs[dst]) + p.recv_off + half + (idx + (int64_t)v * 8) * 2) = u;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.state + 1, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, epoch);
  }
  wait_flags(p.signal_pads, p.sig_off, p.rank, p.world, epoch, p.budget, p.err, 600);
  __syncthreads();
  if (threadIdx.x == 0) {
    p.state[1] = 0u;
    *reinterpret_cast<volatile uint32_t*>(p.state) = epoch;
    __threadfence();
  }
}

}  // namespace xllm

// x: local [d0, d1, d2, E] bf16 (16-byte aligned); the result of this call lies at byte offset
// recv_off + (new epoch & 1) * half_bytes of this rank's symmetric buffer, where the new epoch is
// state[0] + 1 at launch (the kernel publishes it in state[0]); shapes as described at the kernel.
XLLM_API int xllm_a2a_permute(const void* x, const void* peer_bufs, const void* signal_pads, int64_t recv_off,
                              int64_t half_bytes, int64_t sig_off, void* state, void* err, int d0, int d1, int d2, int E,
                              int mode, int rank, int world, void* stream) {
  using namespace xllm;
  if ((int64_t)d0 * d1 * d2 * E == 0) return 0;
  if (E % 8 != 0 || world > kMaxRanks || world < 1 || (mode != 0 && mode != 1) || (recv_off & 15) || (half_bytes & 15) ||
      ((uintptr_t)x & 15))
    return (int)cudaErrorInvalidValue;
  if ((mode == 0 ? d1 : d2) % world != 0) return (int)cudaErrorInvalidValue;
  if ((int64_t)d0 * d1 * d2 * E * 2 > half_bytes) return (int)cudaErrorInvalidValue;
  A2aParams p;
  p.x = (const bf16*)x; p.peer_bufs = (void* const*)peer_bufs; p.signal_pads = (void* const*)signal_pads;
  p.recv_off = recv_off; p.half_bytes = half_bytes; p.sig_off = sig_off; p.state = (uint32_t*)state; p.err = (int*)err;
  p.d0 = d0; p.d1 = d1; p.d2 = d2; p.E = E; p.mode = mode; p.rank = rank; p.world = world; p.budget = g_wait_budget_cycles;
  const int64_t total = (int64_t)d0 * d1 * d2 * (E / 8);
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(592, (total + 255) / 256));
  launch_pdl(a2a_permute_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p);
  return XLLM_LAUNCH_CHECK();
}

// Plain copy of `nbytes` (multiple of 16, both pointers 16-byte aligned); either side may be peer-mapped
// memory.  Used to pull expert weights from the rank that holds them (expert re-placement).
namespace xllm {
__global__ void __launch_bounds__(256) peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
}
}  // namespace xllm

XLLM_API int xllm_peer_copy(void* dst, const void* src, int64_t nbytes, void* stream) {
  using namespace xllm;
  if (nbytes == 0) return 0;
  if ((nbytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15)) return (int)cudaErrorInvalidValue;
  const int64_t n = nbytes >> 4;
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(1184, (n + 255) / 256));
  peer_copy_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, n);
  return XLLM_LAUNCH_CHECK();
}

// Number of uint32 flag slots one call site needs in the signal pad.
XLLM_API int64_t xllm_tp_signal_slots(int world) { return (int64_t)world; }

// peer_bufs / signal_pads: device arrays of `world` pointers.  x and out are [T, H] bf16 at byte
// offsets x_off / out_off of the symmetric buffer (16-byte aligned, H % 8 == 0, H <= 16384).
// residual: local [ceil(T/world), H] shard (mode 1).  epochs: 4 zero-initialised device uint32
// (epoch, unused, arrival counter), owned by this communicator; n_ctas: any positive number (CTAs do not
// wait for one another).  err: device int, set non-zero if a flag wait ran out.
XLLM_API int xllm_tp_allreduce_norm(const void* peer_bufs, const void* signal_pads, uint64_t mc_base,
                                    int64_t x_off, int64_t out_off, int64_t sig_off, void* epochs,
                                    void* residual, const void* weight, void* err, int T, int H, int rank,
                                    int world, int mode, float eps, int n_ctas, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 8 != 0 || H > kCommThreads * kCommMaxVec * 8 || world > kMaxRanks || world > kCommThreads)
    return (int)cudaErrorInvalidValue;
  if ((x_off | out_off) & 15) return (int)cudaErrorInvalidValue;
  TpNormParams p;
  p.peer_bufs = (void* const*)peer_bufs; p.signal_pads = (void* const*)signal_pads; p.mc_base = mc_base;
  p.x_off = x_off; p.out_off = out_off; p.sig_off = sig_off; p.epochs = (uint32_t*)epochs;
  p.residual = (bf16*)residual; p.weight = (const bf16*)weight; p.err = (int*)err; p.T = T; p.H = H;
  p.rank = rank; p.world = world; p.mode = mode; p.eps = eps; p.budget = g_wait_budget_cycles;
  const int tpr = row_group_threads(H);
  if (tpr == 0 || n_ctas < 1) return (int)cudaErrorInvalidValue;
  const int rows = kRowThreads / tpr;
  const int S = (T + world - 1) / world;
  const dim3 grid((unsigned)std::max<int64_t>(1, std::min<int64_t>(n_ctas, ((int64_t)S + rows - 1) / rows))), block(kRowThreads);
  cudaStream_t s = (cudaStream_t)stream;
  switch (tpr) {
    case 32: launch_pdl(tp_twoshot_norm_kernel<32>, grid, block, 0, s, p); break;
    case 64: launch_pdl(tp_twoshot_norm_kernel<64>, grid, block, 0, s, p); break;
    case 128: launch_pdl(tp_twoshot_norm_kernel<128>, grid, block, 0, s, p); break;
    default: launch_pdl(tp_twoshot_norm_kernel<256>, grid, block, 0, s, p); break;
  }
  return XLLM_LAUNCH_CHECK();
}

// Owner's half of the fused GEMM -> reduce-scatter (+ residual + RMSNorm + all-gather); see the
// header.  The inbox [world][S][H] starts at byte offset x_off of this rank's symmetric buffer
// (S = ceil(T / world)); `counter_idx` is the uint32 index of the arrival counter in this rank's
// signal pad and `expected` the number of arrivals that completes the inbox.  Other arguments as
// for xllm_tp_allreduce_norm; both kernels may be mixed on one communicator.
XLLM_API int xllm_tp_inbox_norm(const void* peer_bufs, const void* signal_pads, uint64_t mc_base, int64_t x_off,
                                int64_t out_off, int64_t sig_off, int64_t counter_idx, uint32_t expected,
                                void* epochs, void* residual, const void* weight, void* err, int T, int H,
                                int rank, int world, int mode, float eps, int n_ctas, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  if (H % 8 != 0 || H > kCommThreads * kCommMaxVec * 8 || world > kMaxRanks || world > kCommThreads)
    return (int)cudaErrorInvalidValue;
  if ((x_off | out_off) & 15) return (int)cudaErrorInvalidValue;
  TpNormParams p;
  p.peer_bufs = (void* const*)peer_bufs; p.signal_pads = (void* const*)signal_pads; p.mc_base = mc_base;
  p.x_off = x_off; p.out_off = out_off; p.sig_off = sig_off; p.epochs = (uint32_t*)epochs;
  p.residual = (bf16*)residual; p.weight = (const bf16*)weight; p.err = (int*)err; p.T = T; p.H = H;
  p.rank = rank; p.world = world; p.mode = mode; p.eps = eps; p.budget = g_wait_budget_cycles;
  tp_inbox_norm_kernel<<<n_ctas, kCommThreads, 0, (cudaStream_t)stream>>>(p, counter_idx, expected);
  return XLLM_LAUNCH_CHECK();
}

// Cycles a flag wait of the kernels of this file may take before it gives up and sets the error
// word (default 4e9, about two seconds).  Returns the previous value.
XLLM_API long long xllm_comm_set_wait_budget(long long cycles) {
  const long long old = xllm::g_wait_budget_cycles;
  if (cycles > 0) xllm::g_wait_budget_cycles = cycles;
  return old;
}

// One-shot fused all-reduce (see the kernel's header comment).  x is [T, H] bf16 at byte offset x_off
// of the symmetric buffer on every rank; consecutive calls on one communicator must use different
// x_off.  out / residual_in / residual_out are local [T, H] tensors (residual_in and weight may be
// null, residual_out may be null or alias residual_in).  sig_off: uint32 index of `world` flag slots
// reserved for this kernel in the signal pad; state: 2 zero-initialised device uint32 owned by the
// communicator.  n_ctas: any positive number (CTAs do not wait for one another).
XLLM_API int xllm_tp_oneshot_norm(const void* peer_bufs, const void* signal_pads, uint64_t mc_base, int64_t x_off,
                                  int64_t sig_off, void* state, const void* residual_in, void* residual_out,
                                  const void* weight, void* out, void* err, int T, int H, int rank, int world,
                                  float eps, int n_ctas, void* stream) {
  using namespace xllm;
  if (T == 0) return 0;
  const int tpr = row_group_threads(H);
  if (H % 8 != 0 || tpr == 0 || world > kMaxRanks || (x_off & 15) || n_ctas < 1) return (int)cudaErrorInvalidValue;
  TpOneShotParams p;
  p.peer_bufs = (void* const*)peer_bufs; p.signal_pads = (void* const*)signal_pads; p.mc_base = mc_base;
  p.x_off = x_off; p.sig_off = sig_off; p.state = (uint32_t*)state; p.residual_in = (const bf16*)residual_in;
  p.residual_out = (bf16*)residual_out; p.weight = (const bf16*)weight; p.out = (bf16*)out; p.err = (int*)err;
  p.T = T; p.H = H; p.rank = rank; p.world = world; p.eps = eps; p.budget = g_wait_budget_cycles;
  const int rows = kRowThreads / tpr;
  const dim3 grid((unsigned)std::min<int64_t>(n_ctas, ((int64_t)T + rows - 1) / rows)), block(kRowThreads);
  cudaStream_t s = (cudaStream_t)stream;
  switch (tpr) {
    case 32: launch_pdl(tp_oneshot_norm_kernel<32>, grid, block, 0, s, p); break;
    case 64: launch_pdl(tp_oneshot_norm_kernel<64>, grid, block, 0, s, p); break;
    case 128: launch_pdl(tp_oneshot_norm_kernel<128>, grid, block, 0, s, p); break;
    default: launch_pdl(tp_oneshot_norm_kernel<256>, grid, block, 0, s, p); break;
  }
  return XLLM_LAUNCH_CHECK();
}

// Greedy sampling over vocabulary shards: out_ids[r] = argmax over all ranks' shards of row r (ties:
// lowest index), identical on every rank.  logits: local [B, Vs] bf16 (only the first Vs columns of a
// row are looked at: pass the number of real vocabulary rows of the shard); the pair area needs
// 2 * world * max_rows * 8 bytes at byte offset pair_off of the symmetric buffer; B <= max_rows.
XLLM_API int xllm_tp_argmax(const void* logits, int64_t row_stride, const void* peer_bufs, const void* signal_pads,
                            int64_t pair_off, int64_t sig_off, void* state, void* out_ids, void* err, int B, int Vs,
                            int vocab_start, int max_rows, int rank, int world, void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  if (B > max_rows || world > kMaxRanks || (pair_off & 7) || Vs < 0) return (int)cudaErrorInvalidValue;
  TpArgmaxParams p;
  p.logits = (const bf16*)logits; p.row_stride = row_stride; p.peer_bufs = (void* const*)peer_bufs;
  p.signal_pads = (void* const*)signal_pads; p.pair_off = pair_off; p.sig_off = sig_off; p.state = (uint32_t*)state;
  p.out_ids = (int64_t*)out_ids; p.err = (int*)err; p.B = B; p.Vs = Vs; p.vocab_start = vocab_start;
  p.max_rows = max_rows; p.rank = rank; p.world = world; p.budget = g_wait_budget_cycles;
  launch_pdl(tp_argmax_kernel, dim3(B), dim3(256), 0, (cudaStream_t)stream, p);
  return XLLM_LAUNCH_CHECK();
}

// All-gather of column shards into every rank's [B, dst_stride] area at byte offset dst_off of the
// symmetric buffer (see the kernel's header comment).  Vs % 8 == 0, src rows 16-byte aligned,
// dst_off and dst_stride * 2 multiples of 16.
XLLM_API int xllm_tp_gather_cols(const void* src, int64_t src_stride, const void* peer_bufs, const void* signal_pads,
                                 uint64_t mc_base, int64_t dst_off, int64_t dst_stride, int64_t sig_off, void* state,
                                 void* err, int B, int Vs, int rank, int world, void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  if (Vs % 8 != 0 || (dst_off & 15) || (dst_stride % 8) || (src_stride % 8) || world > kMaxRanks)
    return (int)cudaErrorInvalidValue;
  TpGatherParams p;
  p.src = (const bf16*)src; p.src_stride = src_stride; p.peer_bufs = (void* const*)peer_bufs;
  p.signal_pads = (void* const*)signal_pads; p.mc_base = mc_base; p.dst_off = dst_off; p.dst_stride = dst_stride;
  p.sig_off = sig_off; p.state = (uint32_t*)state; p.err = (int*)err; p.B = B; p.Vs = Vs; p.rank = rank;
  p.world = world; p.budget = g_wait_budget_cycles;
  const int64_t total = (int64_t)B * (Vs / 8);
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(296, (total + 255) / 256));
  launch_pdl(tp_gather_cols_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p);
  return XLLM_LAUNCH_CHECK();
}
