// One pass over packed QKV: per-head RMSNorm (optional) + RoPE + paged KV-cache write.
//
// Replaces three reference launches: fused_qknorm_rope (or rms_norm x2 + rotary_embedding)
// followed by reshape_paged_cache (xllm/core/kernels/cuda/fused_qknorm_rope.cu:84-382,
// rope.cu:27-256, reshape_paged_cache.cu:23-99).  Here Q is written to a dense buffer and K/V
// go straight from registers into the paged cache, so QKV is read from HBM exactly once.
//
// KV cache layout (this engine's choice): [n_blocks, n_kv_heads, block_size, head_dim]; a
// (block, head) pair is one contiguous block_size*head_dim tile, which is what the attention
// kernels stream.
#include "common.cuh"

namespace xllm {

struct RopeKvParams {
  const bf16* qkv;      // [T, (nq + 2*nkv) * d]
  int64_t qkv_stride;   // elements between token rows
  bf16* q_out;          // [T, nq, d]
  bf16* k_cache;        // paged, may be null
  bf16* v_cache;
  bf16* k_out;          // optional dense [T, nkv, d]
  bf16* v_out;
  const bf16* q_norm_w; // [d] or null
  const bf16* k_norm_w;
  const float* cos_sin; // [max_pos, rot] : cos | sin halves, fp32; null => no rope
  const int64_t* positions;  // [T]
  const int32_t* slots;      // [T] (block*block_size + offset; <0 skips the cache write), may be null
  int tokens, nq, nkv, d, rot, block_size, interleaved;
  float eps;
};

// One CTA per token.  A thread owns the same 8-element slot of up to kRopeHeadsPerThread heads (the
// heads of one token share the position, hence the cos / sin values, which are read once per thread);
// all of a thread's 16-byte loads are issued before anything is computed, so that a CTA has its whole
// token row (12 KB for 48 heads of 128) in flight at once.
constexpr int kRopeHeadsPerThread = 4;

__global__ void __launch_bounds__(256) rope_kv_kernel(RopeKvParams p) {
  const int tph = p.d >> 3;  // threads per head (each owns 8 contiguous elements)
  const int heads_per_pass = blockDim.x / tph;
  const int total_heads = p.nq + 2 * p.nkv;
  const int local = threadIdx.x / tph;
  const int g = threadIdx.x - local * tph;
  const int64_t t = blockIdx.x;
  const int e0 = g * 8;
  pdl_wait();
  pdl_launch_dependents();  // dependents may be scheduled now; they block in their own pdl_wait()

  // cos / sin of this thread's slot (shared by all its heads)
  const int half = p.rot >> 1;
  const bool rotates = p.cos_sin != nullptr && e0 < p.rot;
  float c[8], sn[8];
  if (rotates) {
    const float* cs = p.cos_sin + p.positions[t] * p.rot;
    if (p.interleaved) {
      const int pi = e0 >> 1;
      const float4 c4 = *reinterpret_cast<const float4*>(cs + pi);
      const float4 s4 = *reinterpret_cast<const float4*>(cs + half + pi);
      c[0] = c4.x; c[1] = c4.y; c[2] = c4.z; c[3] = c4.w;
      sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
    } else {
      const int ci = e0 < half ? e0 : e0 - half;
      const float4 ca = *reinterpret_cast<const float4*>(cs + ci), cb = *reinterpret_cast<const float4*>(cs + ci + 4);
      const float4 sa = *reinterpret_cast<const float4*>(cs + half + ci), sb = *reinterpret_cast<const float4*>(cs + half + ci + 4);
      c[0] = ca.x; c[1] = ca.y; c[2] = ca.z; c[3] = ca.w; c[4] = cb.x; c[5] = cb.y; c[6] = cb.z; c[7] = cb.w;
      sn[0] = sa.x; sn[1] = sa.y; sn[2] = sa.z; sn[3] = sa.w; sn[4] = sb.x; sn[5] = sb.y; sn[6] = sb.z; sn[7] = sb.w;
    }
  }
  const int slot = (p.slots != nullptr) ? p.slots[t] : -1;
  const bf16* row = p.qkv + t * p.qkv_stride;

  for (int h0 = 0; h0 < total_heads; h0 += heads_per_pass * kRopeHeadsPerThread) {
    bf16x8 raw[kRopeHeadsPerThread];
#pragma unroll
    for (int u = 0; u < kRopeHeadsPerThread; ++u) {
      const int h = h0 + u * heads_per_pass + local;
      if (h < total_heads) raw[u] = reinterpret_cast<const bf16x8*>(row + (int64_t)h * p.d)[g];
    }
#pragma unroll
    for (int u = 0; u < kRopeHeadsPerThread; ++u) {
      const int h = h0 + u * heads_per_pass + local;
      // whole heads are active or not together, so the shuffles below always see their partners
      const bool active = h < total_heads;
      float x[8];
      if (active) {
        unpack8(raw[u], x);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = 0.f;
      }
      const bool is_q = h < p.nq;
      const bool is_k = !is_q && h < p.nq + p.nkv;
      const bf16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
      // per-head RMSNorm (segmented reduce across the tph lanes of this head)
      if (p.q_norm_w != nullptr || p.k_norm_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
        for (int o = tph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (active && nw != nullptr) {
          const float inv = rsqrtf(ss / (float)p.d + p.eps);
          float w[8];
          unpack8(reinterpret_cast<const bf16x8*>(nw)[g], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            // match the usual bf16 module: normalise, round to bf16, scale by the bf16 weight
            x[j] = __bfloat162float(__float2bfloat16(x[j] * inv)) * w[j];
          }
        }
      }
      // RoPE on q and k
      if (p.cos_sin != nullptr) {
        if (p.interleaved) {
          if (active && (is_q || is_k) && rotates) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float a = x[j], b = x[j + 1];
              x[j] = a * c[j >> 1] - b * sn[j >> 1];
              x[j + 1] = b * c[j >> 1] + a * sn[j >> 1];
            }
          }
        } else {
          const int half_lanes = half >> 3;
          float other[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) other[j] = __shfl_xor_sync(0xffffffffu, x[j], half_lanes);
          if (active && (is_q || is_k) && rotates) {
            const bool first = e0 < half;
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = first ? (x[j] * c[j] - other[j] * sn[j]) : (x[j] * c[j] + other[j] * sn[j]);
          }
        }
      }
      if (!active) continue;
      const bf16x8 o = pack8(x);
      if (is_q) {
        reinterpret_cast<bf16x8*>(p.q_out + (t * p.nq + h) * (int64_t)p.d)[g] = o;
        continue;
      }
      const int kvh = is_k ? h - p.nq : h - p.nq - p.nkv;
      bf16* dense = is_k ? p.k_out : p.v_out;
      if (dense) reinterpret_cast<bf16x8*>(dense + (t * p.nkv + kvh) * (int64_t)p.d)[g] = o;
      bf16* cache = is_k ? p.k_cache : p.v_cache;
      if (cache && slot >= 0) {
        const int64_t blk = slot / p.block_size;
        const int off = slot - (int)blk * p.block_size;
        bf16* dst = cache + (((blk * p.nkv + kvh) * p.block_size) + off) * (int64_t)p.d;
        reinterpret_cast<bf16x8*>(dst)[g] = o;
      }
    }
  }
}

}  // namespace xllm

XLLM_API int xllm_rope_kv(const void* qkv, int64_t qkv_stride, void* q_out, void* k_cache,
                          void* v_cache, void* k_out, void* v_out, const void* q_norm_w,
                          const void* k_norm_w, const void* cos_sin, const void* positions,
                          const void* slots, int tokens, int nq, int nkv, int d, int rot,
                          int block_size, int interleaved, float eps, void* stream) {
  using namespace xllm;
  if (tokens == 0) return 0;
  const int tph = d >> 3;
  if (d % 8 != 0 || tph > 32 || (tph & (tph - 1)) != 0) return (int)cudaErrorInvalidValue;
  if (cos_sin && !interleaved) {
    const int hl = (rot >> 1) >> 3;
    if (hl == 0 || (hl & (hl - 1)) != 0 || rot > d) return (int)cudaErrorInvalidValue;
  }
  RopeKvParams p;
  p.qkv = (const bf16*)qkv; p.qkv_stride = qkv_stride; p.q_out = (bf16*)q_out;
  p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.k_out = (bf16*)k_out; p.v_out = (bf16*)v_out;
  p.q_norm_w = (const bf16*)q_norm_w; p.k_norm_w = (const bf16*)k_norm_w;
  p.cos_sin = (const float*)cos_sin; p.positions = (const int64_t*)positions;
  p.slots = (const int32_t*)slots; p.tokens = tokens; p.nq = nq; p.nkv = nkv; p.d = d; p.rot = rot;
  p.block_size = block_size; p.interleaved = interleaved; p.eps = eps;
  // float4 loads of the cos / sin rows: `rot` floats per position, 8-element slots
  if (cos_sin && (rot % 8 != 0 || ((uintptr_t)cos_sin & 15))) return (int)cudaErrorInvalidValue;
  launch_pdl(rope_kv_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, p);
  return XLLM_LAUNCH_CHECK();
}
