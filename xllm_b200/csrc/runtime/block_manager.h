// Paged KV block manager with an LRU prefix cache.
//
// Capability parity with the reference's BlockManagerImpl + PrefixCache + BlockManagerPool
// (xllm/core/framework/block/block_manager_impl.cpp:50-267, block_manager_pool.cpp,
// xllm/core/framework/prefix_cache/prefix_cache.cpp): ref-counted blocks, block 0 reserved as the
// padding block, chained 128-bit block hashes, match / insert / LRU evict, one manager per DP rank.
//
// Design: a block is in exactly one of three states — free (uncached, on the free list), cached
// and unreferenced (on the LRU list, evictable), or referenced (ref > 0, possibly also cached and
// shared).  `allocate` takes free blocks first and evicts from the cold end of the LRU list only
// when it must, so a cache hit costs nothing until memory is actually short.
#pragma once
#include <tuple>
#include <algorithm>
#include <cstdint>
#include <list>
#include <mutex>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#include "hash.h"

namespace xllm {

struct BlockStats {
  int64_t num_blocks = 0, num_free = 0, num_evictable = 0, num_used = 0;
  int64_t match_queries = 0, match_hits_blocks = 0, match_query_blocks = 0;
  int64_t evictions = 0, cached_blocks = 0;
};

class BlockManager {
 public:
  BlockManager(int32_t num_blocks, int32_t block_size, bool enable_prefix_cache)
      : num_blocks_(num_blocks), block_size_(block_size), prefix_(enable_prefix_cache),
        meta_(num_blocks) {
    if (num_blocks < 2) throw std::invalid_argument("BlockManager needs at least 2 blocks");
    free_.reserve(num_blocks);
    // block 0 is the padding block: never handed out, padded batch rows point at it
    for (int32_t i = num_blocks - 1; i >= 1; --i) free_.push_back(i);
  }

  int32_t block_size() const { return block_size_; }
  int32_t num_blocks() const { return num_blocks_; }
  bool prefix_cache_enabled() const { return prefix_; }
  int64_t num_free_blocks() const { return (int64_t)free_.size() + (int64_t)lru_.size(); }
  int64_t num_used_blocks() const { return num_blocks_ - 1 - num_free_blocks(); }
  double utilization() const { return (double)num_used_blocks() / (double)(num_blocks_ - 1); }

  // n fresh (uncached) blocks with ref = 1; empty vector when fewer than n can be had.
  std::vector<int32_t> allocate(int32_t n) {
    std::vector<int32_t> out;
    if (n <= 0) return out;
    if (num_free_blocks() < n) return out;
    out.reserve(n);
    for (int32_t i = 0; i < n; ++i) {
      if (free_.empty()) evict_one();
      int32_t b = free_.back();
      free_.pop_back();
      meta_[b].ref = 1;
      out.push_back(b);
    }
    return out;
  }

  // Longest cached prefix of `tokens` in whole blocks; the returned blocks are referenced
  // (ref += 1).  At most (n_tokens - 1) / block_size blocks are matched so that at least one
  // token is left to run through the model.
  std::vector<int32_t> match_prefix(const int32_t* tokens, int64_t n_tokens, uint64_t extra = 0) {
    std::vector<int32_t> out;
    if (!prefix_ || n_tokens <= 1) return out;
    const int64_t max_blocks = (n_tokens - 1) / block_size_;
    stats_queries_++;
    stats_query_blocks_ += max_blocks;
    Hash128 h;
    for (int64_t i = 0; i < max_blocks; ++i) {
      h = chain_block_hash(h, tokens + i * block_size_, block_size_, extra);
      auto it = table_.find(h);
      if (it == table_.end()) break;
      const int32_t b = it->second;
      ref_block(b);
      out.push_back(b);
    }
    stats_hit_blocks_ += (int64_t)out.size();
    return out;
  }

  // Register the first `n_tokens / block_size` blocks of a sequence in the prefix cache.
  // `start_block` skips blocks already known to be cached.  When a block with the same hash is
  // already cached the sequence keeps its own (duplicate) block, which simply stays uncached.
  void cache_blocks(const int32_t* tokens, int64_t n_tokens, const std::vector<int32_t>& blocks,
                    int64_t start_block = 0, uint64_t extra = 0) {
    if (!prefix_) return;
    const int64_t full = std::min<int64_t>(n_tokens / block_size_, (int64_t)blocks.size());
    Hash128 h;
    for (int64_t i = 0; i < full; ++i) {
      h = chain_block_hash(h, tokens + i * block_size_, block_size_, extra);
      if (i < start_block) continue;
      const int32_t b = blocks[i];
      if (meta_[b].cached) continue;
      if (table_.find(h) != table_.end()) continue;
      table_.emplace(h, b);
      meta_[b].cached = true;
      meta_[b].hash = h;
    }
  }

  void ref_block(int32_t b) {
    Meta& m = meta_[b];
    if (m.ref == 0 && m.cached) lru_.erase(m.lru_it);  // leaves the evictable list
    m.ref++;
  }

  void free_blocks(const std::vector<int32_t>& blocks) {
    // release in reverse so that the tail of a sequence is evicted before its head
    for (auto it = blocks.rbegin(); it != blocks.rend(); ++it) {
      const int32_t b = *it;
      if (b <= 0 || b >= num_blocks_) continue;
      Meta& m = meta_[b];
      if (m.ref <= 0) throw std::runtime_error("double free of KV block");
      if (--m.ref == 0) {
        if (m.cached) {
          lru_.push_front(b);
          m.lru_it = lru_.begin();
        } else {
          free_.push_back(b);
        }
      }
    }
  }

  // Drop every cached-but-unreferenced block (e.g. after weights change).
  void reset_prefix_cache() {
    while (!lru_.empty()) evict_one();
    // referenced cached blocks lose their hash so that nothing new can match them
    for (int32_t b = 1; b < num_blocks_; ++b) {
      if (meta_[b].cached) {
        table_.erase(meta_[b].hash);
        meta_[b].cached = false;
      }
    }
  }

  // ---- hooks for a second (host-memory) tier of the prefix cache
  // With tracking on, every eviction is logged as (block, hash) so that the owner of the cache
  // tensors can save the block's contents before the block is written again.
  void set_track_evictions(bool on) { track_evictions_ = on; }
  std::vector<std::tuple<int32_t, uint64_t, uint64_t>> take_evictions() {
    std::vector<std::tuple<int32_t, uint64_t, uint64_t>> out;
    out.swap(evicted_);
    return out;
  }
  // Device block that caches `h`, or -1.
  int32_t lookup(uint64_t lo, uint64_t hi) const {
    Hash128 h;
    h.lo = lo;
    h.hi = hi;
    auto it = table_.find(h);
    return it == table_.end() ? -1 : it->second;
  }
  // Take a block, register it under `h` and leave it cached and unreferenced (most recently
  // used): the caller then fills it from the host tier.  -1 when no block can be had or the hash is
  // already cached.
  int32_t insert_cached(uint64_t lo, uint64_t hi) {
    Hash128 h;
    h.lo = lo;
    h.hi = hi;
    if (!prefix_ || table_.find(h) != table_.end() || num_free_blocks() < 1) return -1;
    if (free_.empty()) evict_one();
    const int32_t b = free_.back();
    free_.pop_back();
    Meta& m = meta_[b];
    m.ref = 0;
    m.cached = true;
    m.hash = h;
    table_.emplace(h, b);
    lru_.push_front(b);
    m.lru_it = lru_.begin();
    return b;
  }

  int32_t ref_count(int32_t b) const { return meta_[b].ref; }
  bool is_cached(int32_t b) const { return meta_[b].cached; }

  BlockStats stats() const {
    BlockStats s;
    s.num_blocks = num_blocks_;
    s.num_free = (int64_t)free_.size();
    s.num_evictable = (int64_t)lru_.size();
    s.num_used = num_used_blocks();
    s.match_queries = stats_queries_;
    s.match_hits_blocks = stats_hit_blocks_;
    s.match_query_blocks = stats_query_blocks_;
    s.evictions = stats_evictions_;
    s.cached_blocks = (int64_t)table_.size();
    return s;
  }

 private:
  struct Meta {
    int32_t ref = 0;
    bool cached = false;
    Hash128 hash;
    std::list<int32_t>::iterator lru_it;
  };

  void evict_one() {
    if (lru_.empty()) throw std::runtime_error("no evictable KV block");
    const int32_t b = lru_.back();  // coldest
    lru_.pop_back();
    Meta& m = meta_[b];
    table_.erase(m.hash);
    m.cached = false;
    free_.push_back(b);
    stats_evictions_++;
    if (track_evictions_) evicted_.emplace_back(b, m.hash.lo, m.hash.hi);
  }

  int32_t num_blocks_, block_size_;
  bool prefix_;
  std::vector<Meta> meta_;
  std::vector<int32_t> free_;
  std::list<int32_t> lru_;  // front = most recently released
  std::unordered_map<Hash128, int32_t, Hash128Hasher> table_;
  int64_t stats_queries_ = 0, stats_hit_blocks_ = 0, stats_query_blocks_ = 0, stats_evictions_ = 0;
  bool track_evictions_ = false;
  std::vector<std::tuple<int32_t, uint64_t, uint64_t>> evicted_;
};

}  // namespace xllm
