// Expert-parallel all-to-all over NVLink peer memory: token dispatch to the ranks that own the
// routed experts, and the return path fused with the top-k weighted sum.
//
// The reference's CUDA build has no all-to-all: every rank runs the fused MoE over all tokens with an
// expert filter and the partial outputs are all-reduced (xllm/core/layers/cuda/fused_moe.cpp:96-118);
// its DeepEP wrapper (layers/common/deep_ep.h) is not wired on CUDA.  Here tokens travel once:
//
//   xllm_ep_publish_counts  every rank tells every peer how many of its tokens go to each expert
//                           (W x E int32 matrix replicated on all ranks) + flag exchange
//   xllm_ep_layout          from that matrix each rank derives, without further communication,
//                           (a) where its own tokens of expert e land in the owner's receive buffer
//                           (experts in order, each padded to 128 rows, sources in rank order),
//                           (b) the tile -> expert table of its own receive buffer for the grouped GEMM
//   xllm_ep_dispatch        one CTA per (token, k): 16-byte peer stores of the token row into the
//                           owner's receive buffer; remembers (owner, row) for the way back
//   xllm_ep_barrier         flag exchange (bounded wait) between the phases
//   [grouped tcgen05 GEMMs run on the receive buffer: gate|up, SiLU*mul, down -> recv_y]
//   xllm_ep_combine         one CTA per local token: pulls its K expert outputs from the owners'
//                           recv_y with peer loads and forms sum_k w[t,k] * y  (+ shared expert)
//
// All buffers live at the same offsets of one symmetric allocation per rank.  Every wait is
// bounded: on expiry the kernel records an error code and returns; the GPU stays usable.
#include "common.cuh"

namespace xllm {

constexpr int kEpMaxRanks = 16;
constexpr int kEpMaxExperts = 512;
constexpr int kEpTile = 128;
// Budget of a flag wait in SM cycles (about two seconds by default); a launch parameter copied from
// this host value, which xllm_ep_set_wait_budget() changes.
static long long g_ep_wait_budget = 4000000000LL;

struct EpParams {
  void* const* peer_bufs;    // [world] symmetric buffer bases
  void* const* signal_pads;  // [world]
  int64_t cnt_off;           // int32 [world][E]
  int64_t recvx_off;         // bf16 [cap_rows][H]
  int64_t recvy_off;         // bf16 [cap_rows][H]
  int64_t sig_off;           // uint32 index of this communicator's flag slots
  uint32_t* epochs;          // [0] epoch of the last completed exchange
  int* err;
  int rank, world, E, E_local, H, cap_rows;
  long long budget;
};

__device__ __forceinline__ void ep_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ep_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA: publish epoch+1 to every peer, wait for theirs.  Threads 0..world-1 take one peer each.
__device__ __forceinline__ void ep_exchange(const EpParams& p) {
  volatile uint32_t* state = p.epochs;
  const uint32_t e = state[0] + 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    ep_st_release(reinterpret_cast<uint32_t*>(p.signal_pads[peer]) + p.sig_off + p.rank, e);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.signal_pads[p.rank]) + p.sig_off + peer;
    const long long t0 = clock64();
    while ((int32_t)(ep_ld_acquire(mine) - e) < 0) {
      if (clock64() - t0 > p.budget) {
        atomicExch(p.err, 1 + peer);
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    state[0] = e;
    __threadfence();
  }
}

__global__ void ep_barrier_kernel(EpParams p) { ep_exchange(p); }

__global__ void ep_publish_counts_kernel(EpParams p, int32_t* __restrict__ counts) {
  for (int i = threadIdx.x; i < p.E * p.world; i += blockDim.x) {
    const int peer = i / p.E, e = i - peer * p.E;
    int32_t* dst = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(p.peer_bufs[peer]) + p.cnt_off);
    dst[p.rank * p.E + e] = counts[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) counts[e] = 0;  // ready for the next routing pass
  ep_exchange(p);
}

// send_off[e]   : first row, in the owner's receive buffer, of this rank's tokens of expert e
// tile_expert[i]: local expert of row tile i of this rank's receive buffer (-1 = unused)
// meta[0] = rows used in the local receive buffer (multiple of 128)
__device__ __forceinline__ void ep_layout_dev(const EpParams& p, int32_t* __restrict__ send_off,
                                              int32_t* __restrict__ tile_expert, int32_t* __restrict__ meta,
                                              int max_tiles) {
  __shared__ int s_tot[kEpMaxExperts], s_before[kEpMaxExperts], s_base[kEpMaxExperts + kEpMaxRanks];
  const int32_t* C = reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(p.peer_bufs[p.rank]) + p.cnt_off);
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < p.world; ++s) {
      const int c = C[s * p.E + e];
      if (s < p.rank) before += c;
      tot += c;
    }
    s_tot[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  if (threadIdx.x < p.world) {  // one thread per owner rank: padded prefix over its experts
    const int d = threadIdx.x;
    int acc = 0;
    for (int le = 0; le < p.E_local; ++le) {
      const int e = d * p.E_local + le;
      s_base[e] = acc;
      acc += (s_tot[e] + kEpTile - 1) / kEpTile * kEpTile;
    }
    if (d == p.rank) {
      meta[0] = acc;
      if (acc > p.cap_rows) atomicExch(p.err, 300);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) send_off[e] = s_base[e] + s_before[e];
  const int e0 = p.rank * p.E_local;
  for (int le = threadIdx.x; le < p.E_local; le += blockDim.x) {
    const int t0 = s_base[e0 + le] / kEpTile;
    const int t1 = t0 + (s_tot[e0 + le] + kEpTile - 1) / kEpTile;
    for (int i = t0; i < t1 && i < max_tiles; ++i) tile_expert[i] = le;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int used = 0;
    for (int le = 0; le < p.E_local; ++le) used += (s_tot[e0 + le] + kEpTile - 1) / kEpTile;
    meta[1] = used;
  }
  __syncthreads();
  for (int i = meta[1] + threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
}

__global__ void ep_layout_kernel(EpParams p, int32_t* __restrict__ send_off, int32_t* __restrict__ tile_expert,
                                 int32_t* __restrict__ meta, int max_tiles) {
  ep_layout_dev(p, send_off, tile_expert, meta, max_tiles);
}

// publish_counts + layout in one launch (one CTA): the counts go to every peer, the flag exchange
// makes every peer's counts visible here, the layout follows from them.
__global__ void ep_counts_layout_kernel(EpParams p, int32_t* __restrict__ counts, int32_t* __restrict__ send_off,
                                        int32_t* __restrict__ tile_expert, int32_t* __restrict__ meta, int max_tiles) {
  for (int i = threadIdx.x; i < p.E * p.world; i += blockDim.x) {
    const int peer = i / p.E, e = i - peer * p.E;
    int32_t* dst = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(p.peer_bufs[peer]) + p.cnt_off);
    dst[p.rank * p.E + e] = counts[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) counts[e] = 0;  // ready for the next routing pass
  ep_exchange(p);
  ep_layout_dev(p, send_off, tile_expert, meta, max_tiles);
}

__global__ void __launch_bounds__(128)
ep_dispatch_kernel(EpParams p, const bf16* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   const int32_t* __restrict__ slot, const int32_t* __restrict__ send_off,
                   int32_t* __restrict__ where, int T, int K, int close) {
  __shared__ int s_last;
  const int pair = blockIdx.x;
  const int t = pair / K;
  const int e = topk_ids[pair];
  const int d = e / p.E_local;
  const int row = send_off[e] + slot[pair];
  if (row >= p.cap_rows || d >= p.world) {
    if (threadIdx.x == 0) {
      where[pair] = -1;
      atomicExch(p.err, 301);
    }
  } else {
    if (threadIdx.x == 0) where[pair] = d * p.cap_rows + row;
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * p.H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_bufs[d]) + p.recvx_off + (int64_t)row * p.H * 2);
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) dst[v] = src[v];
  }
  if (!close) return;
  // closing exchange by the last CTA to finish: when this kernel has completed on a rank, the rows of
  // every rank have landed in its receive buffer
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.epochs + 1, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) p.epochs[1] = 0u;
    ep_exchange(p);
  }
}

__global__ void __launch_bounds__(128)
ep_combine_kernel(EpParams p, bf16* __restrict__ out, const int32_t* __restrict__ where, const float* __restrict__ w,
                  const bf16* __restrict__ shared_out, int T, int K, int open) {
  const int t = blockIdx.x;
  uint32_t e_open = 0;
  if (open) {
    // opening exchange: every rank's expert outputs are complete before anybody reads them.  CTA 0
    // signals, every CTA polls its own (local) flag slots; the last CTA to finish publishes the epoch.
    e_open = *reinterpret_cast<volatile uint32_t*>(p.epochs) + 1u;
    if (blockIdx.x == 0 && threadIdx.x < p.world)
      ep_st_release(reinterpret_cast<uint32_t*>(p.signal_pads[threadIdx.x]) + p.sig_off + p.rank, e_open);
    if (threadIdx.x < p.world) {
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.signal_pads[p.rank]) + p.sig_off + threadIdx.x;
      const long long t0 = clock64();
      while ((int32_t)(ep_ld_acquire(mine) - e_open) < 0) {
        if (clock64() - t0 > p.budget) {
          atomicExch(p.err, 1 + (int)threadIdx.x);
          break;
        }
      }
    }
    __syncthreads();
  }
  for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (shared_out != nullptr) unpack8(reinterpret_cast<const bf16x8*>(shared_out + (int64_t)t * p.H)[v], acc);
    for (int k = 0; k < K; ++k) {
      const int loc = where[t * K + k];
      if (loc < 0) continue;
      const int d = loc / p.cap_rows, row = loc - d * p.cap_rows;
      const uint4 raw = *(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.peer_bufs[d]) + p.recvy_off +
                                                        (int64_t)row * p.H * 2) + v);
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(&raw), f);
      const float wk = w[t * K + k];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * f[j];
    }
    reinterpret_cast<bf16x8*>(out + (int64_t)t * p.H)[v] = pack8(acc);
  }
  if (open) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.epochs + 1, 1u) == gridDim.x - 1) {
        p.epochs[1] = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.epochs) = e_open;
        __threadfence();
      }
    }
  }
}

static EpParams make_ep(const void* peer_bufs, const void* signal_pads, int64_t cnt_off, int64_t recvx_off,
                        int64_t recvy_off, int64_t sig_off, void* epochs, void* err, int rank, int world, int E,
                        int H, int cap_rows) {
  EpParams p;
  p.peer_bufs = (void* const*)peer_bufs; p.signal_pads = (void* const*)signal_pads; p.cnt_off = cnt_off;
  p.recvx_off = recvx_off; p.recvy_off = recvy_off; p.sig_off = sig_off; p.epochs = (uint32_t*)epochs;
  p.err = (int*)err; p.rank = rank; p.world = world; p.E = E; p.E_local = E / world; p.H = H; p.cap_rows = cap_rows;
  p.budget = g_ep_wait_budget;
  return p;
}

}  // namespace xllm

#define EP_COMMON_ARGS                                                                                         \
  const void *peer_bufs, const void *signal_pads, int64_t cnt_off, int64_t recvx_off, int64_t recvy_off,      \
      int64_t sig_off, void *epochs, void *err, int rank, int world, int E, int H, int cap_rows
#define EP_MAKE make_ep(peer_bufs, signal_pads, cnt_off, recvx_off, recvy_off, sig_off, epochs, err, rank, world, E, H, cap_rows)

static int ep_check(int world, int E, int H) {
  using namespace xllm;
  if (world < 1 || world > kEpMaxRanks || E > kEpMaxExperts || E % world || H % 8) return (int)cudaErrorInvalidValue;
  return 0;
}

XLLM_API int xllm_ep_barrier(EP_COMMON_ARGS, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(EP_MAKE);
  return XLLM_LAUNCH_CHECK();
}

// counts: int32 [E], this rank's tokens per (global) expert; cleared afterwards.
XLLM_API int xllm_ep_publish_counts(EP_COMMON_ARGS, void* counts, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  ep_publish_counts_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(EP_MAKE, (int32_t*)counts);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_ep_layout(EP_COMMON_ARGS, void* send_off, void* tile_expert, void* meta, int max_tiles, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  ep_layout_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(EP_MAKE, (int32_t*)send_off, (int32_t*)tile_expert,
                                                       (int32_t*)meta, max_tiles);
  return XLLM_LAUNCH_CHECK();
}

// x [T, H] bf16 local tokens; topk_ids / slot int32 [T*K] (slot = index of the pair among this rank's
// tokens of that expert); where int32 [T*K] receives owner * cap_rows + row.
XLLM_API int xllm_ep_dispatch(EP_COMMON_ARGS, const void* x, const void* topk_ids, const void* slot,
                              const void* send_off, void* where, int T, int K, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  if (T * K == 0) return 0;
  ep_dispatch_kernel<<<T * K, 128, 0, (cudaStream_t)stream>>>(EP_MAKE, (const bf16*)x, (const int32_t*)topk_ids,
                                                             (const int32_t*)slot, (const int32_t*)send_off,
                                                             (int32_t*)where, T, K, 0);
  return XLLM_LAUNCH_CHECK();
}

// Fused forms (fewer launches and flag exchanges per MoE layer):
//   xllm_ep_counts_layout  = publish_counts + layout                       (one exchange)
//   xllm_ep_dispatch_sync  = dispatch, then the exchange that says "all rows have landed"
//   xllm_ep_combine_sync   = the exchange that says "all expert outputs are complete", then combine
// With these a layer needs three exchanges and no closing barrier: a rank can only pass the dispatch
// exchange of the next layer after every rank has finished this layer's combine, so the receive and
// output buffers are free again by the time anybody writes them.
XLLM_API int xllm_ep_counts_layout(EP_COMMON_ARGS, void* counts, void* send_off, void* tile_expert, void* meta,
                                   int max_tiles, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  ep_counts_layout_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(EP_MAKE, (int32_t*)counts, (int32_t*)send_off,
                                                              (int32_t*)tile_expert, (int32_t*)meta, max_tiles);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_ep_dispatch_sync(EP_COMMON_ARGS, const void* x, const void* topk_ids, const void* slot,
                                   const void* send_off, void* where, int T, int K, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  if (T * K == 0) {   // nothing to send: only the exchange
    ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(EP_MAKE);
    return XLLM_LAUNCH_CHECK();
  }
  ep_dispatch_kernel<<<T * K, 128, 0, (cudaStream_t)stream>>>(EP_MAKE, (const bf16*)x, (const int32_t*)topk_ids,
                                                             (const int32_t*)slot, (const int32_t*)send_off,
                                                             (int32_t*)where, T, K, 1);
  return XLLM_LAUNCH_CHECK();
}

XLLM_API int xllm_ep_combine_sync(EP_COMMON_ARGS, void* out, const void* where, const void* w, const void* shared_out,
                                  int T, int K, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  if (T == 0) {
    ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(EP_MAKE);
    return XLLM_LAUNCH_CHECK();
  }
  ep_combine_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(EP_MAKE, (bf16*)out, (const int32_t*)where, (const float*)w,
                                                        (const bf16*)shared_out, T, K, 1);
  return XLLM_LAUNCH_CHECK();
}

// out[t] = (shared_out[t]) + sum_k w[t,k] * recv_y(owner(t,k))[row(t,k)]
XLLM_API int xllm_ep_combine(EP_COMMON_ARGS, void* out, const void* where, const void* w, const void* shared_out,
                             int T, int K, void* stream) {
  using namespace xllm;
  if (int rc = ep_check(world, E, H)) return rc;
  if (T == 0) return 0;
  ep_combine_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(EP_MAKE, (bf16*)out, (const int32_t*)where, (const float*)w,
                                                        (const bf16*)shared_out, T, K, 0);
  return XLLM_LAUNCH_CHECK();
}

// Cycles a flag wait of the expert-parallel kernels may take before it gives up and sets the error
// word (default 4e9, about two seconds).  Returns the previous value.
XLLM_API long long xllm_ep_set_wait_budget(long long cycles) {
  const long long old = xllm::g_ep_wait_budget;
  if (cycles > 0) xllm::g_ep_wait_budget = cycles;
  return old;
}
