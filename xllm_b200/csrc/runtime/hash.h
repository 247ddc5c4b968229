// 128-bit chained block hash for the prefix cache.
//
// The reference chains XXH3-128 over (previous block hash, token ids of the block)
// (xllm/core/framework/prefix_cache/block_hasher.cpp).  xxHash is not available here, so the
// chain uses MurmurHash3 x64-128 (public-domain algorithm by Austin Appleby), written out below.
// Only the chaining contract matters: hash_i = H(hash_{i-1} || tokens of block i [|| extra keys]).
#pragma once
#include <cstdint>
#include <cstring>
#include <functional>

namespace xllm {

struct Hash128 {
  uint64_t lo = 0, hi = 0;
  bool operator==(const Hash128& o) const { return lo == o.lo && hi == o.hi; }
  bool operator!=(const Hash128& o) const { return !(*this == o); }
  bool is_zero() const { return lo == 0 && hi == 0; }
};

struct Hash128Hasher {
  size_t operator()(const Hash128& h) const { return (size_t)(h.lo ^ (h.hi * 0x9E3779B97F4A7C15ull)); }
};

namespace detail {
inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t fmix64(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}
}  // namespace detail

inline Hash128 murmur3_128(const void* key, size_t len, uint64_t seed_lo, uint64_t seed_hi) {
  using namespace detail;
  const uint8_t* data = (const uint8_t*)key;
  const size_t nblocks = len / 16;
  uint64_t h1 = seed_lo, h2 = seed_hi;
  const uint64_t c1 = 0x87c37b91114253d5ull, c2 = 0x4cf5ad432745937full;
  for (size_t i = 0; i < nblocks; i++) {
    uint64_t k1, k2;
    memcpy(&k1, data + i * 16, 8);
    memcpy(&k2, data + i * 16 + 8, 8);
    k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
    h1 = rotl64(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
    k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;
    h2 = rotl64(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
  }
  const uint8_t* tail = data + nblocks * 16;
  uint64_t k1 = 0, k2 = 0;
  switch (len & 15) {
    case 15: k2 ^= ((uint64_t)tail[14]) << 48; [[fallthrough]];
    case 14: k2 ^= ((uint64_t)tail[13]) << 40; [[fallthrough]];
    case 13: k2 ^= ((uint64_t)tail[12]) << 32; [[fallthrough]];
    case 12: k2 ^= ((uint64_t)tail[11]) << 24; [[fallthrough]];
    case 11: k2 ^= ((uint64_t)tail[10]) << 16; [[fallthrough]];
    case 10: k2 ^= ((uint64_t)tail[9]) << 8; [[fallthrough]];
    case 9:  k2 ^= ((uint64_t)tail[8]) << 0;
             k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2; [[fallthrough]];
    case 8:  k1 ^= ((uint64_t)tail[7]) << 56; [[fallthrough]];
    case 7:  k1 ^= ((uint64_t)tail[6]) << 48; [[fallthrough]];
    case 6:  k1 ^= ((uint64_t)tail[5]) << 40; [[fallthrough]];
    case 5:  k1 ^= ((uint64_t)tail[4]) << 32; [[fallthrough]];
    case 4:  k1 ^= ((uint64_t)tail[3]) << 24; [[fallthrough]];
    case 3:  k1 ^= ((uint64_t)tail[2]) << 16; [[fallthrough]];
    case 2:  k1 ^= ((uint64_t)tail[1]) << 8; [[fallthrough]];
    case 1:  k1 ^= ((uint64_t)tail[0]) << 0;
             k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
  }
  h1 ^= (uint64_t)len; h2 ^= (uint64_t)len;
  h1 += h2; h2 += h1;
  h1 = fmix64(h1); h2 = fmix64(h2);
  h1 += h2; h2 += h1;
  return Hash128{h1, h2};
}

// hash of one full block chained on the previous block's hash; `extra` distinguishes e.g.
// multimodal content or LoRA ids that make equal token ids non-shareable.
inline Hash128 chain_block_hash(const Hash128& prev, const int32_t* tokens, size_t n, uint64_t extra = 0) {
  return murmur3_128(tokens, n * sizeof(int32_t), prev.lo ^ extra, prev.hi + 0x6a09e667f3bcc908ull);
}

}  // namespace xllm
