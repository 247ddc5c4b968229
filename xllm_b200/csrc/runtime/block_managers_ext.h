// Block managers beyond the basic pool: sliding-window, composite (several pools allocated together),
// embedding slots, and a thread-safe wrapper.
//
// Parity: xllm/core/framework/block/sliding_window_block_manager.cpp, composite_block_manager.cpp,
// embedding_block_manager.cpp, concurrent_block_manager_impl.cpp.  The pools themselves are
// `BlockManager`s (block_manager.h); these classes add the policies on top.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "block_manager.h"

namespace xllm {

// A pool for layers that attend to the last `window` tokens only: a sequence never holds more than
// ceil(window / block_size) + 1 blocks; grow() appends a block for new tokens and gives back the blocks
// that fell out of the window (their table entries become 0, the padding block).
class SlidingWindowBlockManager {
 public:
  SlidingWindowBlockManager(int32_t num_blocks, int32_t block_size, int32_t window)
      : bm_(num_blocks, block_size, /*enable_prefix_cache=*/false), bs_(block_size), window_(window) {
    if (window <= 0) throw std::invalid_argument("window must be positive");
  }
  int32_t max_blocks_per_sequence() const { return (window_ + bs_ - 1) / bs_ + 1; }

  // Extends `table` so that positions [0, n_tokens) are addressable, releases what lies entirely
  // before position n_tokens - window.  Returns false (table untouched) when the pool is short.
  bool grow(std::vector<int32_t>& table, int32_t n_tokens) {
    const int32_t need_len = (n_tokens + bs_ - 1) / bs_;
    const int32_t dead = std::max(0, (n_tokens - window_ + 1) / bs_);
    int32_t to_alloc = 0;
    for (int32_t i = (int32_t)table.size(); i < need_len; ++i) to_alloc += i >= dead ? 1 : 0;
    std::vector<int32_t> fresh = bm_.allocate(to_alloc);
    if ((int32_t)fresh.size() < to_alloc) {
      bm_.free_blocks(fresh);
      return false;
    }
    size_t k = 0;
    for (int32_t i = (int32_t)table.size(); i < need_len; ++i) table.push_back(i >= dead ? fresh[k++] : 0);
    std::vector<int32_t> give;
    for (int32_t i = 0; i < dead && i < (int32_t)table.size(); ++i) {
      if (table[i] > 0) give.push_back(table[i]);
      table[i] = 0;
    }
    bm_.free_blocks(give);
    return true;
  }
  void release(std::vector<int32_t>& table) {
    bm_.free_blocks(table);
    table.clear();
  }
  int64_t num_free_blocks() const { return bm_.num_free_blocks(); }
  int64_t num_used_blocks() const { return bm_.num_used_blocks(); }
  int32_t window() const { return window_; }

 private:
  BlockManager bm_;
  int32_t bs_, window_;
};

// Several pools that a sequence needs together (full-attention layers, sliding-window layers, recurrent
// state slots, ...): an allocation succeeds in all of them or in none.
class CompositeBlockManager {
 public:
  void add_pool(const std::string& name, int32_t num_blocks, int32_t block_size, bool prefix_cache) {
    if (pools_.count(name)) throw std::invalid_argument("pool exists: " + name);
    pools_[name] = std::make_unique<BlockManager>(num_blocks, block_size, prefix_cache);
  }
  BlockManager& pool(const std::string& name) {
    auto it = pools_.find(name);
    if (it == pools_.end()) throw std::out_of_range("no such pool: " + name);
    return *it->second;
  }
  std::vector<std::string> names() const {
    std::vector<std::string> n;
    for (auto& kv : pools_) n.push_back(kv.first);
    return n;
  }
  // counts: pool name -> number of blocks.  Empty result = not enough room somewhere (nothing taken).
  std::map<std::string, std::vector<int32_t>> allocate(const std::map<std::string, int32_t>& counts) {
    std::map<std::string, std::vector<int32_t>> got;
    for (auto& kv : counts) {
      std::vector<int32_t> b = pool(kv.first).allocate(kv.second);
      if ((int32_t)b.size() < kv.second) {
        pool(kv.first).free_blocks(b);
        for (auto& g : got) pool(g.first).free_blocks(g.second);
        return {};
      }
      got[kv.first] = std::move(b);
    }
    return got;
  }
  void free(const std::map<std::string, std::vector<int32_t>>& blocks) {
    for (auto& kv : blocks) pool(kv.first).free_blocks(kv.second);
  }
  // the scarcest pool decides how full the cache is
  double utilization() {
    double u = 0;
    for (auto& kv : pools_) u = std::max(u, kv.second->utilization());
    return u;
  }

 private:
  std::map<std::string, std::unique_ptr<BlockManager>> pools_;
};

// Requests that only produce an embedding hold no KV after their single forward pass; what limits them
// is the number of activations in flight.  A counting manager with the allocate / free shape.
class EmbeddingBlockManager {
 public:
  explicit EmbeddingBlockManager(int32_t max_in_flight) : cap_(max_in_flight) {}
  bool allocate(const std::string& request_id) {
    if ((int32_t)held_.size() >= cap_ || held_.count(request_id)) return false;
    held_[request_id] = 1;
    return true;
  }
  bool free(const std::string& request_id) { return held_.erase(request_id) > 0; }
  int32_t num_in_flight() const { return (int32_t)held_.size(); }
  int32_t capacity() const { return cap_; }

 private:
  int32_t cap_;
  std::unordered_map<std::string, int> held_;
};

// A BlockManager behind a mutex, for callers on several threads (request threads probing the prefix
// cache while the scheduler thread allocates).
class ConcurrentBlockManager {
 public:
  ConcurrentBlockManager(int32_t num_blocks, int32_t block_size, bool prefix_cache)
      : bm_(num_blocks, block_size, prefix_cache) {}
  std::vector<int32_t> allocate(int32_t n) {
    std::lock_guard<std::mutex> lk(mu_);
    return bm_.allocate(n);
  }
  void free_blocks(const std::vector<int32_t>& b) {
    std::lock_guard<std::mutex> lk(mu_);
    bm_.free_blocks(b);
  }
  std::vector<int32_t> match_prefix(const std::vector<int32_t>& tokens, uint64_t extra) {
    std::lock_guard<std::mutex> lk(mu_);
    return bm_.match_prefix(tokens.data(), (int64_t)tokens.size(), extra);
  }
  void cache_blocks(const std::vector<int32_t>& tokens, const std::vector<int32_t>& blocks, int64_t start, uint64_t extra) {
    std::lock_guard<std::mutex> lk(mu_);
    bm_.cache_blocks(tokens.data(), (int64_t)tokens.size(), blocks, start, extra);
  }
  int64_t num_free_blocks() {
    std::lock_guard<std::mutex> lk(mu_);
    return bm_.num_free_blocks();
  }
  int64_t num_used_blocks() {
    std::lock_guard<std::mutex> lk(mu_);
    return bm_.num_used_blocks();
  }

 private:
  std::mutex mu_;
  BlockManager bm_;
};

}  // namespace xllm
