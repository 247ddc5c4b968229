// Gated delta rule, one decode token per sequence (linear-attention layers of Qwen3-Next / Qwen3.5):
//
//   S <- S * exp(g);  delta = (v - S^T k) * beta;  S <- S + k (x) delta;  o = S^T q
//
// S is the per-request, per-head recurrent state [d_k, d_v] in fp32, addressed through a slot index.
// One CTA per (head, sequence), one thread per state column: a thread reads its column once from
// HBM for S^T k and once more (from L1/L2) while it rewrites it and accumulates o, so the state
// crosses HBM once in each direction -- the step is bound by that traffic.
//
// Parity: the reference runs this update through Triton FLA kernels on its Python executor
// (xllm/python/.../kernels_cuda, fused_recurrent_gated_delta_rule); there is no CUDA C++ version.
#include "common.cuh"

namespace xllm {

__global__ void gdn_decode_kernel(float* __restrict__ state, const int64_t* __restrict__ slots,
                                  const float* __restrict__ q, const float* __restrict__ k,
                                  const float* __restrict__ v, const float* __restrict__ g,
                                  const float* __restrict__ beta, float* __restrict__ out, int nv, int dk, int dv) {
  extern __shared__ float sm[];
  float* ks = sm;
  float* qs = sm + dk;
  const int h = blockIdx.x, b = blockIdx.y;
  const int64_t row = (int64_t)b * nv + h;
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    ks[i] = k[row * dk + i];
    qs[i] = q[row * dk + i];
  }
  __syncthreads();
  const float decay = __expf(g[row]);
  const float bt = beta[row];
  float* S = state + ((slots[b] * nv + h) * (int64_t)dk) * dv;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float kv = 0.f;
    for (int i = 0; i < dk; ++i) kv += S[(int64_t)i * dv + j] * ks[i];
    const float delta = (v[row * dv + j] - kv * decay) * bt;
    float o = 0.f;
    for (int i = 0; i < dk; ++i) {
      const float s = S[(int64_t)i * dv + j] * decay + ks[i] * delta;
      S[(int64_t)i * dv + j] = s;
      o += s * qs[i];
    }
    out[row * dv + j] = o;
  }
}

// The same update with the state column held in registers: four row groups per CTA (threadIdx.y), each
// thread keeps R = dk / 4 rows of its column, so that the state is read from HBM exactly once, all of a
// thread's loads are in flight together, and the two column sums (S^T k and S^T q) are completed
// through shared memory.
constexpr int gdn_reg_max_threads(int R) { return R >= 64 ? 256 : (R >= 32 ? 512 : (R >= 16 ? 768 : 1024)); }

template <int R>
__global__ void __launch_bounds__(gdn_reg_max_threads(R)) gdn_decode_reg_kernel(float* __restrict__ state, const int64_t* __restrict__ slots,
                                      const float* __restrict__ q, const float* __restrict__ k,
                                      const float* __restrict__ v, const float* __restrict__ g,
                                      const float* __restrict__ beta, float* __restrict__ out, int nv, int dv) {
  constexpr int dk = 4 * R;
  extern __shared__ float sm[];
  float* ks = sm;
  float* qs = sm + dk;
  float* red = sm + 2 * dk;                         // [4][blockDim.x]
  const int h = blockIdx.x, b = blockIdx.y;
  // a CTA owns blockDim.x columns of the state (the columns are independent of one another)
  const int tx = threadIdx.x, gy = threadIdx.y, dvp = blockDim.x;
  const int j = blockIdx.z * dvp + tx;
  const int64_t row = (int64_t)b * nv + h;
  pdl_wait();
  pdl_launch_dependents();
  for (int i = gy * dvp + tx; i < dk; i += 4 * dvp) {
    ks[i] = k[row * dk + i];
    qs[i] = q[row * dk + i];
  }
  const float decay = __expf(g[row]);
  const float bt = beta[row];
  const bool live = j < dv;
  float* S = state + ((slots[b] * nv + h) * (int64_t)dk + gy * R) * dv + j;
  float s[R];
#pragma unroll
  for (int r = 0; r < R; ++r) s[r] = live ? S[(int64_t)r * dv] : 0.f;
  __syncthreads();
  float part = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) part += s[r] * ks[gy * R + r];
  red[gy * dvp + tx] = part;
  __syncthreads();
  const float kv = (red[tx] + red[dvp + tx] + red[2 * dvp + tx] + red[3 * dvp + tx]) * decay;
  const float delta = ((live ? v[row * dv + j] : 0.f) - kv) * bt;
  float o = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    s[r] = s[r] * decay + ks[gy * R + r] * delta;
    if (live) S[(int64_t)r * dv] = s[r];
    o += s[r] * qs[gy * R + r];
  }
  __syncthreads();
  red[gy * dvp + tx] = o;
  __syncthreads();
  if (gy == 0 && live) out[row * dv + j] = red[tx] + red[dvp + tx] + red[2 * dvp + tx] + red[3 * dvp + tx];
}

// Prompt chunks: the same recurrence over the n tokens of ONE sequence without leaving the kernel.
// A CTA owns blockDim.x state columns of one head (four row groups, R rows of the column per thread,
// as above) and walks the tokens in order; k_t and q_t of the next token are staged in shared memory
// while the current one is reduced.  The state is read from HBM once (or starts at zero for a new
// sequence) and written once; per token the CTA moves 2 dk + 1 inputs and one output per column.
// The reference reaches this through FLA's chunked Triton kernels
// (xllm/python/kernels_cuda/triton/gdn_prefill.py); this is the fused-recurrent form of the same rule.
template <int R>
__global__ void __launch_bounds__(256) gdn_prefill_reg_kernel(   // the launcher uses at most 64 x 4 threads

    float* __restrict__ state, int64_t slot, int fresh, const float* __restrict__ q, const float* __restrict__ k,
    const float* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ out,
    int n, int nv, int dv) {
  constexpr int dk = 4 * R;
  extern __shared__ float sm[];
  float* kq = sm;                                   // [2 buffers][k: dk | q: dk]
  float* red_a = sm + 4 * dk;                       // [4][blockDim.x]
  float* red_b = red_a + 4 * blockDim.x;            // [4][blockDim.x]
  const int h = blockIdx.x;
  const int tx = threadIdx.x, gy = threadIdx.y, dvp = blockDim.x;
  const int j = blockIdx.y * dvp + tx;
  const bool live = j < dv;
  const int tid = gy * dvp + tx, nthreads = 4 * dvp;
  float* S = state + ((slot * nv + h) * (int64_t)dk + gy * R) * dv + j;
  float s[R];
#pragma unroll
  for (int r = 0; r < R; ++r) s[r] = (live && !fresh) ? S[(int64_t)r * dv] : 0.f;
  // Software pipeline over tokens, so that no global load is waited for inside a step: the inputs of token
  // t + D are requested while token t is computed and sit in a ring of D register slots (slot = t mod D, the
  // token loop is unrolled D times so that the slots are plain registers).  k_t / q_t go from their slot to
  // shared memory one step before they are used (after that step's first barrier), v_t, g_t, beta_t are
  // read from their slot directly.
  constexpr int KQ = dk >= 64 ? dk / 64 : 1;        // k|q values per thread (blockDim.x >= 32: 2 dk / 128 at most)
  constexpr int D = R >= 64 ? 2 : 8;                // ring depth (the largest state leaves few registers)
  float kq_r[D][KQ], v_r[D], g_r[D], b_r[D];
  auto fetch = [&](int t, float* dst) {             // this thread's share of token t's k | q
    const int64_t row = (int64_t)t * nv + h;
#pragma unroll
    for (int e = 0; e < KQ; ++e) {
      const int i = tid + e * nthreads;
      dst[e] = (t < n && i < 2 * dk) ? (i < dk ? k[row * dk + i] : q[row * dk + (i - dk)]) : 0.f;
    }
  };
  auto fetch_vgb = [&](int t, float& vv, float& gg, float& bb) {
    const int64_t row = (int64_t)t * nv + h;
    vv = (t < n && live) ? v[row * dv + j] : 0.f;
    gg = t < n ? g[row] : 0.f;
    bb = t < n ? beta[row] : 0.f;
  };
  auto put = [&](const float* src, int buf) {
    float* dst = kq + buf * 2 * dk;
#pragma unroll
    for (int e = 0; e < KQ; ++e) {
      const int i = tid + e * nthreads;
      if (i < 2 * dk) dst[i] = src[e];
    }
  };
#pragma unroll
  for (int d = 0; d < D; ++d) {
    fetch(d, kq_r[d]);
    fetch_vgb(d, v_r[d], g_r[d], b_r[d]);
  }
  put(kq_r[0], 0);
  fetch(D, kq_r[0]);                                // slot 0 is free again: token D
  __syncthreads();
  for (int t0 = 0; t0 < n; t0 += D) {
#pragma unroll
    for (int u = 0; u < D; ++u) {
      const int t = t0 + u;
      if (t >= n) break;                            // uniform over the CTA
      const int buf = t & 1;
      const float* ks = kq + buf * 2 * dk;
      const float* qs = ks + dk;
      const int64_t row = (int64_t)t * nv + h;
      const float v_t = v_r[u], decay = __expf(g_r[u]), bt = b_r[u];
      fetch_vgb(t + D, v_r[u], g_r[u], b_r[u]);
      // this thread's R values of k_t and q_t: 16-byte shared loads (the whole warp reads the same address),
      // four independent partial sums so that the multiply-adds pipeline
      float kr[R], qr[R];
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 a = *reinterpret_cast<const float4*>(ks + gy * R + r);
        const float4 b = *reinterpret_cast<const float4*>(qs + gy * R + r);
        kr[r] = a.x; kr[r + 1] = a.y; kr[r + 2] = a.z; kr[r + 3] = a.w;
        qr[r] = b.x; qr[r + 1] = b.y; qr[r + 2] = b.z; qr[r + 3] = b.w;
      }
      float p4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < R; ++r) p4[r & 3] += s[r] * kr[r];
      red_a[gy * dvp + tx] = (p4[0] + p4[1]) + (p4[2] + p4[3]);
      __syncthreads();
      if (t + 1 < n) {
        const int nu = (u + 1) % D;                 // static after unrolling
        put(kq_r[nu], buf ^ 1);                     // that buffer was last read in step t-1: all threads are past it
        fetch(t + 1 + D, kq_r[nu]);
      }
      const float kv = (red_a[tx] + red_a[dvp + tx] + red_a[2 * dvp + tx] + red_a[3 * dvp + tx]) * decay;
      const float delta = (v_t - kv) * bt;
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < R; ++r) {
        s[r] = s[r] * decay + kr[r] * delta;
        o4[r & 3] += s[r] * qr[r];
      }
      red_b[gy * dvp + tx] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
      __syncthreads();
      if (gy == 0 && live) out[row * dv + j] = red_b[tx] + red_b[dvp + tx] + red_b[2 * dvp + tx] + red_b[3 * dvp + tx];
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) S[(int64_t)r * dv] = s[r];
  }
}

}  // namespace xllm

// Prompt chunk of one sequence: q, k [n, nv, dk]; v, out [n, nv, dv]; g, beta [n, nv] (fp32); the
// state of slot `slot` is advanced over the n tokens (from zero when `fresh`).  dk in {32, 64, 128, 256}.
XLLM_API int xllm_gdn_prefill(void* state, int64_t slot, int fresh, const void* q, const void* k, const void* v,
                              const void* g, const void* beta, void* out, int n, int nv, int dk, int dv, void* stream) {
  using namespace xllm;
  if (n == 0) return 0;
  if (!(dk == 32 || dk == 64 || dk == 128 || dk == 256) || dv <= 0) return (int)cudaErrorInvalidValue;
  const int dvp = ((dv + 31) / 32) * 32;
  const int cols = dk == 256 ? 32 : (dvp < 64 ? dvp : 64);
  const dim3 grid(nv, (dv + cols - 1) / cols), block(cols, 4);
  const size_t smem = (size_t)(4 * dk + 8 * cols) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define XLLM_GDN_PF_CASE(RR)                                                                                      \
  case RR:                                                                                                        \
    gdn_prefill_reg_kernel<RR><<<grid, block, smem, st>>>((float*)state, slot, fresh, (const float*)q,            \
                                                          (const float*)k, (const float*)v, (const float*)g,      \
                                                          (const float*)beta, (float*)out, n, nv, dv);            \
    return XLLM_LAUNCH_CHECK();
  switch (dk / 4) {
    XLLM_GDN_PF_CASE(8)
    XLLM_GDN_PF_CASE(16)
    XLLM_GDN_PF_CASE(32)
    XLLM_GDN_PF_CASE(64)
    default: break;
  }
#undef XLLM_GDN_PF_CASE
  return (int)cudaErrorInvalidValue;
}

// state [n_slots, nv, dk, dv] fp32; slots [B] int64; q, k [B, nv, dk]; v, out [B, nv, dv]; g, beta [B, nv] (all fp32).
XLLM_API int xllm_gdn_decode_step(void* state, const void* slots, const void* q, const void* k, const void* v,
                                  const void* g, const void* beta, void* out, int B, int nv, int dk, int dv,
                                  void* stream) {
  using namespace xllm;
  if (B == 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 4096) return (int)cudaErrorInvalidValue;
  const int dvp = ((dv + 31) / 32) * 32;
  if (dk == 32 || dk == 64 || dk == 128 || dk == 256) {   // register-resident state columns
    // 64 columns per CTA (32 for the largest state rows): 256 threads, so that two or more CTAs share an SM
    const int cols = dk == 256 ? 32 : (dvp < 64 ? dvp : 64);
    const dim3 grid(nv, B, (dv + cols - 1) / cols), block(cols, 4);
    const size_t smem = (size_t)(2 * dk + 4 * cols) * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
#define XLLM_GDN_CASE(RR)                                                                                       \
  case RR:                                                                                                      \
    launch_pdl(gdn_decode_reg_kernel<RR>, grid, block, smem, st, (float*)state, (const int64_t*)slots,          \
               (const float*)q, (const float*)k, (const float*)v, (const float*)g, (const float*)beta,          \
               (float*)out, nv, dv);                                                                            \
    return XLLM_LAUNCH_CHECK();
    switch (dk / 4) {
      XLLM_GDN_CASE(8)
      XLLM_GDN_CASE(16)
      XLLM_GDN_CASE(32)
      XLLM_GDN_CASE(64)
      default: break;
    }
#undef XLLM_GDN_CASE
  }
  int threads = dvp;
  if (threads > 256) threads = 256;
  launch_pdl(gdn_decode_kernel, dim3(nv, B), dim3(threads), (size_t)(2 * dk * sizeof(float)), (cudaStream_t)stream,
             (float*)state, (const int64_t*)slots, (const float*)q, (const float*)k, (const float*)v, (const float*)g,
             (const float*)beta, (float*)out, nv, dk, dv);
  return XLLM_LAUNCH_CHECK();
}
