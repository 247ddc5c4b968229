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
// A barrier is a flag exchange through the symmetric signal pad done by one CTA per rank (a growing
// epoch stored into slot [my rank] of every peer, then a wait on the own slots); the other CTAs of
// the grid synchronise with that CTA through device-local flags.  Every wait is bounded;
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
#include "common.cuh"

namespace xllm {

constexpr int kCommThreads = 256;
constexpr int kCommMaxVec = 8;
constexpr int kMaxRanks = 16;
constexpr long long kFlagBudgetCycles = 4000000000LL;

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
      if (clock64() - t0 > kFlagBudgetCycles) {
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

__global__ void __launch_bounds__(kCommThreads) tp_allreduce_norm_kernel(TpNormParams p) {
  __shared__ float red[32];
  __shared__ int s_last;
  volatile uint32_t* state = p.epochs;
  const uint32_t e0 = state[0];
  const int S = (p.T + p.world - 1) / p.world;
  const int row_begin = p.rank * S;
  const int row_end = min(row_begin + S, p.T);
  const int nvec = p.H >> 3;
  pdl_wait();
  // ---- barrier 1: CTA 0 talks to the peers, the other CTAs wait for its local "go"
  if (blockIdx.x == 0) {
    exchange_flags(p, e0 + 1);
    if (threadIdx.x == 0) {
      __threadfence();
      state[1] = e0 + 1;
    }
  } else {
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      while (state[1] != e0 + 1) {
        if (clock64() - t0 > kFlagBudgetCycles) {
          atomicExch(p.err, 100);
          break;
        }
      }
      __threadfence();
    }
    __syncthreads();
  }

  for (int row = row_begin + blockIdx.x; row < row_end; row += gridDim.x) {
    float vals[kCommMaxVec][8];
    float ss = 0.f;
    const int64_t row_byte = (int64_t)row * p.H * 2;
#pragma unroll
    for (int i = 0; i < kCommMaxVec; ++i) {
      const int v = threadIdx.x + i * kCommThreads;
      if (v < nvec) {
        const int64_t off = p.x_off + row_byte + (int64_t)v * 16;
        if (p.mc_base != 0) {
          const uint4 u = multimem_ld_reduce_bf16x8(p.mc_base + off);
          unpack8(*reinterpret_cast<const bf16x8*>(&u), vals[i]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
          for (int k = 0; k < p.world; ++k) {
            const int peer = (p.rank + k) % p.world;  // start at home, spread the link load
            const bf16x8 u = *reinterpret_cast<const bf16x8*>(reinterpret_cast<const uint8_t*>(p.peer_bufs[peer]) + off);
            float f[8];
            unpack8(u, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] += f[j];
          }
        }
        if (p.mode == 1) {
          bf16x8* rr = reinterpret_cast<bf16x8*>(p.residual + (int64_t)(row - row_begin) * p.H) + v;
          float r[8];
          unpack8(*rr, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
          const bf16x8 nr = pack8(vals[i]);  // the residual stream is bf16: round once
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
  // ---- barrier 2: the last CTA to finish tells the peers and waits for theirs, so that the
  // completion of this kernel means `out` is complete on this rank
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(const_cast<uint32_t*>(&state[2]), 1u);
    s_last = prev == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (s_last) {
    exchange_flags(p, e0 + 2);
    if (threadIdx.x == 0) {
      state[2] = 0;
      state[0] = e0 + 2;
      __threadfence();
    }
  }
  pdl_launch_dependents();
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
      if (clock64() - t0 > kFlagBudgetCycles) {
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

}  // namespace xllm

// Number of uint32 flag slots one call site needs in the signal pad.
XLLM_API int64_t xllm_tp_signal_slots(int world) { return (int64_t)world; }

// peer_bufs / signal_pads: device arrays of `world` pointers.  x and out are [T, H] bf16 at byte
// offsets x_off / out_off of the symmetric buffer (16-byte aligned, H % 8 == 0, H <= 16384).
// residual: local [ceil(T/world), H] shard (mode 1).  epochs: 4 zero-initialised device uint32
// (epoch, go flag, arrival counter), owned by this communicator; n_ctas <= 296 (all CTAs must be co-resident).  err: device int, set non-zero if a flag wait ran out.
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
  p.rank = rank; p.world = world; p.mode = mode; p.eps = eps;
  tp_allreduce_norm_kernel<<<n_ctas, kCommThreads, 0, (cudaStream_t)stream>>>(p);
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
  p.rank = rank; p.world = world; p.mode = mode; p.eps = eps;
  tp_inbox_norm_kernel<<<n_ctas, kCommThreads, 0, (cudaStream_t)stream>>>(p, counter_idx, expected);
  return XLLM_LAUNCH_CHECK();
}
