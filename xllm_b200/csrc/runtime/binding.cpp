// pybind11 module `xllm_b200._rt`: the C++ runtime exposed to the Python front end.
//
// Counterpart of the reference's `xllm_export` module (xllm/pybind/bind.cpp:38-418), which
// exposes Options / LLMMaster / RequestParams / RequestOutput; here the exposed surface is the
// runtime building blocks (scheduler, block manager, tokenizer, loaders, server) that the Python
// `LLM` / `serve` front ends compose.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "block_manager.h"
#include "block_managers_ext.h"
#include "scheduler.h"
#include "sequence.h"

namespace py = pybind11;
using namespace xllm;

void bind_frontend(py::module_& m);  // csrc/frontend
void bind_server(py::module_& m);    // csrc/server
void bind_runtime_extra(py::module_& m);

template <typename T>
static py::array_t<T> to_np(const std::vector<T>& v) {
  py::array_t<T> a((py::ssize_t)v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

PYBIND11_MODULE(_rt, m) {
  m.doc() = "xllm_b200 native runtime";

  py::class_<BlockStats>(m, "BlockStats")
      .def_readonly("num_blocks", &BlockStats::num_blocks)
      .def_readonly("num_free", &BlockStats::num_free)
      .def_readonly("num_evictable", &BlockStats::num_evictable)
      .def_readonly("num_used", &BlockStats::num_used)
      .def_readonly("match_queries", &BlockStats::match_queries)
      .def_readonly("match_hits_blocks", &BlockStats::match_hits_blocks)
      .def_readonly("match_query_blocks", &BlockStats::match_query_blocks)
      .def_readonly("evictions", &BlockStats::evictions)
      .def_readonly("cached_blocks", &BlockStats::cached_blocks);

  py::class_<BlockManager>(m, "BlockManager")
      .def(py::init<int32_t, int32_t, bool>(), py::arg("num_blocks"), py::arg("block_size"),
           py::arg("enable_prefix_cache") = true)
      .def("allocate", &BlockManager::allocate)
      .def("free", &BlockManager::free_blocks)
      .def("match_prefix",
           [](BlockManager& bm, const std::vector<int32_t>& toks, uint64_t extra) {
             return bm.match_prefix(toks.data(), (int64_t)toks.size(), extra);
           },
           py::arg("tokens"), py::arg("extra") = 0)
      .def("cache_blocks",
           [](BlockManager& bm, const std::vector<int32_t>& toks, const std::vector<int32_t>& blocks,
              int64_t start_block, uint64_t extra) {
             bm.cache_blocks(toks.data(), (int64_t)toks.size(), blocks, start_block, extra);
           },
           py::arg("tokens"), py::arg("blocks"), py::arg("start_block") = 0, py::arg("extra") = 0)
      .def("reset_prefix_cache", &BlockManager::reset_prefix_cache)
      .def("set_track_evictions", &BlockManager::set_track_evictions)
      .def("take_evictions", &BlockManager::take_evictions)
      .def("lookup", &BlockManager::lookup)
      .def("insert_cached", &BlockManager::insert_cached)
      .def("ref_count", &BlockManager::ref_count)
      .def("is_cached", &BlockManager::is_cached)
      .def_property_readonly("num_free_blocks", &BlockManager::num_free_blocks)
      .def_property_readonly("num_used_blocks", &BlockManager::num_used_blocks)
      .def_property_readonly("utilization", &BlockManager::utilization)
      .def_property_readonly("block_size", &BlockManager::block_size)
      .def_property_readonly("num_blocks", &BlockManager::num_blocks)
      .def("stats", &BlockManager::stats);

  py::class_<SlidingWindowBlockManager>(m, "SlidingWindowBlockManager")
      .def(py::init<int32_t, int32_t, int32_t>(), py::arg("num_blocks"), py::arg("block_size"), py::arg("window"))
      .def("grow",
           [](SlidingWindowBlockManager& bm, std::vector<int32_t> table, int32_t n_tokens) {
             const bool ok = bm.grow(table, n_tokens);
             return py::make_tuple(ok, table);
           })
      .def("release", [](SlidingWindowBlockManager& bm, std::vector<int32_t> table) { bm.release(table); })
      .def_property_readonly("max_blocks_per_sequence", &SlidingWindowBlockManager::max_blocks_per_sequence)
      .def_property_readonly("num_free_blocks", &SlidingWindowBlockManager::num_free_blocks)
      .def_property_readonly("num_used_blocks", &SlidingWindowBlockManager::num_used_blocks)
      .def_property_readonly("window", &SlidingWindowBlockManager::window);

  py::class_<CompositeBlockManager>(m, "CompositeBlockManager")
      .def(py::init<>())
      .def("add_pool", &CompositeBlockManager::add_pool, py::arg("name"), py::arg("num_blocks"), py::arg("block_size"),
           py::arg("prefix_cache") = false)
      .def("pool", &CompositeBlockManager::pool, py::return_value_policy::reference_internal)
      .def("names", &CompositeBlockManager::names)
      .def("allocate", &CompositeBlockManager::allocate)
      .def("free", &CompositeBlockManager::free)
      .def_property_readonly("utilization", &CompositeBlockManager::utilization);

  py::class_<EmbeddingBlockManager>(m, "EmbeddingBlockManager")
      .def(py::init<int32_t>(), py::arg("max_in_flight"))
      .def("allocate", &EmbeddingBlockManager::allocate)
      .def("free", &EmbeddingBlockManager::free)
      .def_property_readonly("num_in_flight", &EmbeddingBlockManager::num_in_flight)
      .def_property_readonly("capacity", &EmbeddingBlockManager::capacity);

  py::class_<ConcurrentBlockManager>(m, "ConcurrentBlockManager")
      .def(py::init<int32_t, int32_t, bool>(), py::arg("num_blocks"), py::arg("block_size"), py::arg("prefix_cache") = true)
      .def("allocate", &ConcurrentBlockManager::allocate, py::call_guard<py::gil_scoped_release>())
      .def("free", &ConcurrentBlockManager::free_blocks, py::call_guard<py::gil_scoped_release>())
      .def("match_prefix", &ConcurrentBlockManager::match_prefix, py::arg("tokens"), py::arg("extra") = 0,
           py::call_guard<py::gil_scoped_release>())
      .def("cache_blocks", &ConcurrentBlockManager::cache_blocks, py::arg("tokens"), py::arg("blocks"),
           py::arg("start_block") = 0, py::arg("extra") = 0, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("num_free_blocks", &ConcurrentBlockManager::num_free_blocks)
      .def_property_readonly("num_used_blocks", &ConcurrentBlockManager::num_used_blocks);

  m.def("block_hash_chain", [](const std::vector<int32_t>& toks, int32_t block_size, uint64_t extra) {
    std::vector<std::pair<uint64_t, uint64_t>> out;
    Hash128 h;
    for (size_t i = 0; i + block_size <= toks.size(); i += block_size) {
      h = chain_block_hash(h, toks.data() + i, block_size, extra);
      out.emplace_back(h.lo, h.hi);
    }
    return out;
  }, py::arg("tokens"), py::arg("block_size"), py::arg("extra") = 0);

  // Byte offsets of the packed per-step input buffer for T token rows, S sequences and NS sample
  // rows (the layout Batch.fill_packed writes; same return convention).
  m.def("packed_layout", [](int64_t T, int64_t S, int64_t NS, int64_t bt_stride) {
    auto al = [](int64_t x) { return (x + 15) & ~(int64_t)15; };
    std::vector<int64_t> off(17);
    int64_t o = 0;
    off[0] = o; o = al(o + T * 8);
    off[1] = o; o = al(o + T * 8);
    off[2] = o; o = al(o + NS * 8);
    off[3] = o; o = al(o + T * 4);
    off[4] = o; o = al(o + S * 4);
    off[5] = o; o = al(o + (S + 1) * 4);
    off[6] = o; o = al(o + S * 4);
    off[7] = o; o = al(o + NS * 4);
    off[8] = o; o = al(o + NS * 4);
    off[9] = o; o = al(o + NS * 4);
    off[10] = o; o = al(o + S * bt_stride * 4);
    off[15] = o; o = al(o + NS * 8);
    off[16] = o; o = al(o + NS * 4);
    off[11] = o; off[12] = T; off[13] = S; off[14] = NS;
    return off;
  });

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("frequency_penalty", &SamplingParams::frequency_penalty)
      .def_readwrite("presence_penalty", &SamplingParams::presence_penalty)
      .def_readwrite("repetition_penalty", &SamplingParams::repetition_penalty)
      .def_readwrite("logprobs", &SamplingParams::logprobs)
      .def_readwrite("top_logprobs", &SamplingParams::top_logprobs)
      .def_readwrite("seed", &SamplingParams::seed);

  py::class_<StoppingParams>(m, "StoppingParams")
      .def(py::init<>())
      .def_readwrite("max_tokens", &StoppingParams::max_tokens)
      .def_readwrite("max_context_len", &StoppingParams::max_context_len)
      .def_readwrite("eos_token_id", &StoppingParams::eos_token_id)
      .def_readwrite("ignore_eos", &StoppingParams::ignore_eos)
      .def_readwrite("stop_token_ids", &StoppingParams::stop_token_ids)
      .def_readwrite("stop_sequences", &StoppingParams::stop_sequences);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_tokens_per_batch", &SchedulerConfig::max_tokens_per_batch)
      .def_readwrite("max_seqs_per_batch", &SchedulerConfig::max_seqs_per_batch)
      .def_readwrite("enable_chunked_prefill", &SchedulerConfig::enable_chunked_prefill)
      .def_readwrite("max_tokens_per_chunk_for_prefill", &SchedulerConfig::max_tokens_per_chunk_for_prefill)
      .def_readwrite("enable_prefix_cache", &SchedulerConfig::enable_prefix_cache)
      .def_readwrite("block_size", &SchedulerConfig::block_size)
      .def_readwrite("num_blocks", &SchedulerConfig::num_blocks)
      .def_readwrite("policy", &SchedulerConfig::policy)
      .def_readwrite("priority_strategy", &SchedulerConfig::priority_strategy)
      .def_readwrite("prefill_scheduling_memory_usage_threshold",
                     &SchedulerConfig::prefill_scheduling_memory_usage_threshold)
      .def_readwrite("enable_schedule_overlap", &SchedulerConfig::enable_schedule_overlap)
      .def_readwrite("enable_online_preempt_offline", &SchedulerConfig::enable_online_preempt_offline)
      .def_readwrite("dp_size", &SchedulerConfig::dp_size)
      .def_readwrite("num_speculative_tokens", &SchedulerConfig::num_speculative_tokens)
      .def_readwrite("max_decode_batch", &SchedulerConfig::max_decode_batch)
      .def_readwrite("max_running_seqs", &SchedulerConfig::max_running_seqs)
      .def_readwrite("min_prefill_tokens", &SchedulerConfig::min_prefill_tokens)
      .def_readwrite("max_prefill_wait_steps", &SchedulerConfig::max_prefill_wait_steps)
      .def_readwrite("hold_finished_blocks", &SchedulerConfig::hold_finished_blocks)
      .def_readwrite("admission", &SchedulerConfig::admission)
      .def_readwrite("sliding_window", &SchedulerConfig::sliding_window);

  py::enum_<PauseMode>(m, "PauseMode")
      .value("KEEP", PauseMode::KEEP)
      .value("ABORT", PauseMode::ABORT)
      .value("WAIT", PauseMode::WAIT);

  py::class_<Batch>(m, "Batch")
      .def_readonly("batch_id", &Batch::batch_id)
      .def_readonly("dp_rank", &Batch::dp_rank)
      .def_readonly("n_decode", &Batch::n_decode)
      .def_readonly("n_prefill", &Batch::n_prefill)
      .def_readonly("n_tokens", &Batch::n_tokens)
      .def_readonly("max_q_len", &Batch::max_q_len)
      .def_readonly("max_kv_len", &Batch::max_kv_len)
      .def_readonly("max_blocks", &Batch::max_blocks)
      .def_readonly("any_penalty", &Batch::any_penalty)
      .def_readonly("any_logprobs", &Batch::any_logprobs)
      .def_readonly("all_greedy", &Batch::all_greedy)
      .def_readonly("max_top_logprobs", &Batch::max_top_logprobs)
      .def_property_readonly("n_seqs", &Batch::n_seqs)
      .def_property_readonly("n_samples", [](const Batch& b) { return (int64_t)b.sample_rows.size(); })
      .def_property_readonly("tokens", [](const Batch& b) { return to_np(b.tokens); })
      .def_property_readonly("positions", [](const Batch& b) { return to_np(b.positions); })
      .def_property_readonly("slots", [](const Batch& b) { return to_np(b.slots); })
      .def_property_readonly("q_lens", [](const Batch& b) { return to_np(b.q_lens); })
      .def_property_readonly("kv_lens", [](const Batch& b) { return to_np(b.kv_lens); })
      .def_property_readonly("cu_q", [](const Batch& b) { return to_np(b.cu_q); })
      .def_property_readonly("block_tables",
                             [](const Batch& b) {
                               py::array_t<int32_t> a({(py::ssize_t)b.n_seqs(), (py::ssize_t)b.max_blocks});
                               if (!b.block_tables.empty())
                                 std::memcpy(a.mutable_data(), b.block_tables.data(),
                                             b.block_tables.size() * sizeof(int32_t));
                               return a;
                             })
      .def_property_readonly("sample_rows", [](const Batch& b) { return to_np(b.sample_rows); })
      .def_property_readonly("sample_seq", [](const Batch& b) { return to_np(b.sample_seq); })
      .def_property_readonly("temperature", [](const Batch& b) { return to_np(b.temperature); })
      .def_property_readonly("top_p", [](const Batch& b) { return to_np(b.top_p); })
      .def_property_readonly("top_k", [](const Batch& b) { return to_np(b.top_k); })
      .def_property_readonly("frequency_penalty", [](const Batch& b) { return to_np(b.freq_pen); })
      .def_property_readonly("presence_penalty", [](const Batch& b) { return to_np(b.pres_pen); })
      .def_property_readonly("repetition_penalty", [](const Batch& b) { return to_np(b.rep_pen); })
      .def_property_readonly("seeds", [](const Batch& b) { return to_np(b.seeds); })
      .def_property_readonly("sample_offsets", [](const Batch& b) { return to_np(b.sample_offsets); })
      .def_property_readonly("seq_ids", [](const Batch& b) { return to_np(b.seq_ids); })
      // the last `max_n` tokens (prompt + generated) of sequence `i` of the batch (all when max_n <= 0)
      .def("history",
           [](const Batch& b, int64_t i, int64_t max_n) {
             const std::vector<int32_t>& t = b.seqs.at((size_t)i)->tokens;
             const size_t n = max_n > 0 && (size_t)max_n < t.size() ? (size_t)max_n : t.size();
             py::array_t<int32_t> a((py::ssize_t)n);
             std::memcpy(a.mutable_data(), t.data() + (t.size() - n), n * sizeof(int32_t));
             return a;
           },
           py::arg("i"), py::arg("max_n") = 0)
      .def("request_id", [](const Batch& b, int64_t i) { return b.seqs.at((size_t)i)->request->request_id; })
      // Pack every per-step device input into ONE caller-owned (pinned) byte buffer so that a step
      // costs a single H2D copy.  Segments are 16-byte aligned, in this order:
      //   tokens i64[T] | positions i64[T] | sample_rows i64[NS] | slots i32[T] | kv_lens i32[S] |
      //   cu_q i32[S+1] | q_lens i32[S] | top_k i32[NS] | temperature f32[NS] | top_p f32[NS] |
      //   block_table i32[S, bt_stride]
      // With pad_seqs > n_seqs (decode-only batches replayed from a CUDA graph) T = S = NS =
      // pad_seqs and the padding rows are inert: token 0, slot -1, kv_len 0, greedy.
      // followed by seeds u64[NS] | sample_offsets i32[NS].
      // With pad_prefill_tokens / pad_prefill_seqs > 0 (steps with prompt chunks replayed from a CUDA
      // graph) the layout is fixed: pad_seqs decode rows, then pad_prefill_tokens prompt-chunk rows;
      // pad_seqs + pad_prefill_seqs sequences; padding sequences have q_len 0 and kv_len 0.
      // Returns [off_tokens, off_positions, off_sample_rows, off_slots, off_kv_lens, off_cu_q,
      //          off_q_lens, off_top_k, off_temperature, off_top_p, off_bt, total_bytes, T, S, NS,
      //          off_seeds, off_sample_offsets].
      // Unique token ids and their counts over each sampled sequence (prompt + generated), padded
      // with -1 / 0 to the widest row; None when the batch has no penalties.
      .def("penalty_tokens",
           [](const Batch& b) -> py::object {
             if (!b.any_penalty) return py::none();
             const int64_t ns = (int64_t)b.sample_seq.size();
             std::vector<std::unordered_map<int32_t, int32_t>> maps(ns);
             size_t width = 1;
             for (int64_t r = 0; r < ns; ++r) {
               const Sequence* s = b.seqs[b.sample_seq[r]];
               if (!s->request->sampling.has_penalty()) continue;
               for (int32_t t : s->tokens) maps[r][t]++;
               width = std::max(width, maps[r].size());
             }
             py::array_t<int32_t> ids({(py::ssize_t)ns, (py::ssize_t)width});
             py::array_t<int32_t> cnt({(py::ssize_t)ns, (py::ssize_t)width});
             int32_t* pi = ids.mutable_data();
             int32_t* pc = cnt.mutable_data();
             std::fill(pi, pi + ns * width, -1);
             std::fill(pc, pc + ns * width, 0);
             for (int64_t r = 0; r < ns; ++r) {
               size_t j = 0;
               for (auto& kv : maps[r]) { pi[r * width + j] = kv.first; pc[r * width + j] = kv.second; ++j; }
             }
             return py::make_tuple(ids, cnt);
           })
      .def("fill_packed",
           [](const Batch& b, uintptr_t ptr, int64_t capacity, int32_t bt_stride, int32_t pad_seqs,
              int32_t pad_prefill_tokens, int32_t pad_prefill_seqs) {
             // real sizes
             const int64_t nd = b.n_decode, npf = b.n_prefill;
             const int64_t rT = b.n_tokens, rS = b.n_seqs(), rNS = (int64_t)b.sample_rows.size();
             const int64_t ptok = rT - nd;  // prompt-chunk token rows
             // padded layout: decode rows [0, D), prompt-chunk rows [D, D + Q), sequences D + P
             const bool mixed = pad_prefill_tokens > 0 || pad_prefill_seqs > 0;
             int64_t D = nd, Q = ptok, P = npf;
             if (mixed) {
               D = std::max<int64_t>(pad_seqs, 0);
               Q = pad_prefill_tokens;
               P = pad_prefill_seqs;
               if (nd > D || ptok > Q || npf > P) throw std::runtime_error("batch does not fit the padded layout");
             } else if (pad_seqs > rS) {
               if (npf != 0) throw std::runtime_error("decode padding needs a decode-only batch");
               D = pad_seqs;
             }
             const int64_t T = D + Q, S = D + P, NS = (mixed || D > nd) ? S : rNS;
             if (bt_stride < b.max_blocks) throw std::runtime_error("block table stride too small");
             auto al = [](int64_t x) { return (x + 15) & ~(int64_t)15; };
             std::vector<int64_t> off(17);
             int64_t o = 0;
             off[0] = o; o = al(o + T * 8);
             off[1] = o; o = al(o + T * 8);
             off[2] = o; o = al(o + NS * 8);
             off[3] = o; o = al(o + T * 4);
             off[4] = o; o = al(o + S * 4);
             off[5] = o; o = al(o + (S + 1) * 4);
             off[6] = o; o = al(o + S * 4);
             off[7] = o; o = al(o + NS * 4);
             off[8] = o; o = al(o + NS * 4);
             off[9] = o; o = al(o + NS * 4);
             off[10] = o; o = al(o + S * (int64_t)bt_stride * 4);
             off[15] = o; o = al(o + NS * 8);
             off[16] = o; o = al(o + NS * 4);
             off[11] = o; off[12] = T; off[13] = S; off[14] = NS;
             if (o > capacity) throw std::runtime_error("staging buffer too small");
             uint8_t* base = reinterpret_cast<uint8_t*>(ptr);
             int64_t* tok = (int64_t*)(base + off[0]);
             int64_t* pos = (int64_t*)(base + off[1]);
             int64_t* srow = (int64_t*)(base + off[2]);
             int32_t* slots = (int32_t*)(base + off[3]);
             int32_t* kvl = (int32_t*)(base + off[4]);
             int32_t* cuq = (int32_t*)(base + off[5]);
             int32_t* ql = (int32_t*)(base + off[6]);
             int32_t* topk = (int32_t*)(base + off[7]);
             float* temp = (float*)(base + off[8]);
             float* topp = (float*)(base + off[9]);
             int32_t* bt = (int32_t*)(base + off[10]);
             uint64_t* seeds = (uint64_t*)(base + off[15]);
             int32_t* soff = (int32_t*)(base + off[16]);
             // token rows
             std::memcpy(tok, b.tokens.data(), nd * 8);
             std::memcpy(pos, b.positions.data(), nd * 8);
             std::memcpy(slots, b.slots.data(), nd * 4);
             for (int64_t i = nd; i < D; ++i) { tok[i] = 0; pos[i] = 0; slots[i] = -1; }
             std::memcpy(tok + D, b.tokens.data() + nd, ptok * 8);
             std::memcpy(pos + D, b.positions.data() + nd, ptok * 8);
             std::memcpy(slots + D, b.slots.data() + nd, ptok * 4);
             for (int64_t i = D + ptok; i < T; ++i) { tok[i] = 0; pos[i] = 0; slots[i] = -1; }
             // sequences
             std::memcpy(kvl, b.kv_lens.data(), nd * 4);
             std::memcpy(ql, b.q_lens.data(), nd * 4);
             for (int64_t i = 0; i <= nd; ++i) cuq[i] = b.cu_q[i];
             for (int64_t i = nd; i < D; ++i) { kvl[i] = 0; ql[i] = 1; cuq[i + 1] = cuq[i] + 1; }
             const int32_t shift = (int32_t)(D - nd);   // how far the prompt-chunk rows moved
             for (int64_t j = 0; j < npf; ++j) {
               kvl[D + j] = b.kv_lens[nd + j];
               ql[D + j] = b.q_lens[nd + j];
               cuq[D + j + 1] = b.cu_q[nd + j + 1] + shift;
             }
             for (int64_t j = npf; j < P; ++j) { kvl[D + j] = 0; ql[D + j] = 0; cuq[D + j + 1] = cuq[D + j]; }
             // sample rows keep their order (decode rows, then the prompt chunks that end a prompt);
             // padding entries sample row 0 greedily and are ignored by the caller
             for (int64_t r = 0; r < rNS; ++r) {
               const int64_t row = b.sample_rows[r];
               srow[r] = row >= nd ? row + shift : row;
               topk[r] = b.top_k[r]; temp[r] = b.temperature[r]; topp[r] = b.top_p[r];
               seeds[r] = b.seeds[r]; soff[r] = b.sample_offsets[r];
             }
             for (int64_t r = rNS; r < NS; ++r) {
               srow[r] = mixed ? 0 : r; topk[r] = 0; temp[r] = 0.f; topp[r] = 1.f; seeds[r] = 0; soff[r] = 0;
             }
             // block tables
             for (int64_t i = 0; i < rS; ++i) {
               int32_t* dst = bt + (i < nd ? i : i + shift) * (int64_t)bt_stride;
               std::memcpy(dst, b.block_tables.data() + i * b.max_blocks, b.max_blocks * 4);
               if (bt_stride > b.max_blocks) std::memset(dst + b.max_blocks, 0, (size_t)(bt_stride - b.max_blocks) * 4);
             }
             for (int64_t i = nd; i < D; ++i) std::memset(bt + i * (int64_t)bt_stride, 0, (size_t)bt_stride * 4);
             for (int64_t j = npf; j < P; ++j) std::memset(bt + (D + j) * (int64_t)bt_stride, 0, (size_t)bt_stride * 4);
             return off;
           },
           py::arg("ptr"), py::arg("capacity"), py::arg("bt_stride"), py::arg("pad_seqs") = 0,
           py::arg("pad_prefill_tokens") = 0, py::arg("pad_prefill_seqs") = 0);

  py::class_<OutputEvent>(m, "OutputEvent")
      .def_readonly("request_id", &OutputEvent::request_id)
      .def_readonly("seq_index", &OutputEvent::seq_index)
      .def_readonly("token", &OutputEvent::token)
      .def_readonly("logprob", &OutputEvent::logprob)
      .def_readonly("has_logprob", &OutputEvent::has_logprob)
      .def_readonly("finished", &OutputEvent::finished)
      .def_readonly("finish_reason", &OutputEvent::finish_reason)
      .def_readonly("num_prompt_tokens", &OutputEvent::num_prompt_tokens)
      .def_readonly("num_generated", &OutputEvent::num_generated)
      .def_readonly("prefix_hit_tokens", &OutputEvent::prefix_hit_tokens)
      .def_readonly("request_finished", &OutputEvent::request_finished)
      .def_readonly("seq_id", &OutputEvent::seq_id)
      .def_readonly("top_ids", &OutputEvent::top_ids)
      .def_readonly("top_logprobs", &OutputEvent::top_logprobs);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerConfig&>())
      .def("add_request", &Scheduler::add_request, py::arg("request_id"), py::arg("prompt_tokens"),
           py::arg("sampling"), py::arg("stopping"), py::arg("n") = 1, py::arg("priority") = 0,
           py::arg("deadline") = 0.0, py::arg("offline") = false, py::arg("stream") = false,
           py::arg("extra_hash_key") = 0)
      .def("abort_request", &Scheduler::abort_request)
      .def("adopt_prefilled", &Scheduler::adopt_prefilled, py::arg("request_id"), py::arg("tokens"),
           py::arg("num_prompt_tokens"), py::arg("sampling"), py::arg("stopping"), py::arg("priority") = 0,
           py::arg("offline") = false, py::arg("stream") = false)
      .def("reserve_blocks", &Scheduler::reserve_blocks, py::arg("request_id"), py::arg("n_tokens"))
      .def("cancel_reserved", &Scheduler::cancel_reserved)
      .def("num_reserved", &Scheduler::num_reserved)
      .def("reserved_ids", &Scheduler::reserved_ids)
      .def("adopt_reserved", &Scheduler::adopt_reserved, py::arg("request_id"), py::arg("tokens"),
           py::arg("num_prompt_tokens"), py::arg("sampling"), py::arg("stopping"), py::arg("priority") = 0,
           py::arg("offline") = false, py::arg("stream") = false)
      .def("set_hold_finished_blocks", &Scheduler::set_hold_finished_blocks)
      .def("held_blocks", &Scheduler::held_blocks)
      .def("release_held", &Scheduler::release_held)
      .def("schedule", &Scheduler::schedule, py::call_guard<py::gil_scoped_release>())
      .def("process_output",
           [](Scheduler& s, int64_t batch_id, py::array_t<int64_t, py::array::c_style | py::array::forcecast> toks,
              py::object logprobs) {
             const float* lp = nullptr;
             py::array_t<float, py::array::c_style | py::array::forcecast> lpa;
             if (!logprobs.is_none()) {
               lpa = logprobs.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
               lp = lpa.data();
             }
             return s.process_output(batch_id, toks.data(), (int64_t)toks.size(), lp);
           },
           py::arg("batch_id"), py::arg("next_tokens"), py::arg("logprobs") = py::none())
      .def("process_output_multi",
           [](Scheduler& s, int64_t batch_id, py::array_t<int64_t, py::array::c_style | py::array::forcecast> toks,
              py::array_t<int32_t, py::array::c_style | py::array::forcecast> counts, py::object logprobs) {
             const float* lp = nullptr;
             py::array_t<float, py::array::c_style | py::array::forcecast> lpa;
             if (!logprobs.is_none()) {
               lpa = logprobs.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
               lp = lpa.data();
             }
             int64_t total = 0;
             for (py::ssize_t i = 0; i < counts.size(); ++i) total += std::max<int32_t>(counts.data()[i], 1);
             if (total > (int64_t)toks.size()) throw std::invalid_argument("process_output_multi: too few tokens");
             return s.process_output_multi(batch_id, toks.data(), counts.data(), (int64_t)counts.size(), lp);
           },
           py::arg("batch_id"), py::arg("tokens"), py::arg("counts"), py::arg("logprobs") = py::none())
      .def("set_top_logprobs",
           [](Scheduler& s, int64_t batch_id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> ids,
              py::array_t<float, py::array::c_style | py::array::forcecast> lps) {
             if (ids.ndim() != 2 || lps.ndim() != 2 || ids.shape(0) != lps.shape(0) || ids.shape(1) != lps.shape(1))
               throw std::invalid_argument("set_top_logprobs: ids and logprobs must both be [rows, n]");
             s.set_top_logprobs(batch_id, ids.data(), lps.data(), (int64_t)ids.shape(0), (int32_t)ids.shape(1));
           })
      .def("take_pending_events", &Scheduler::take_pending_events)
      .def("take_preempted", &Scheduler::take_preempted)
      .def("set_prefill_batching", &Scheduler::set_prefill_batching, py::arg("min_prefill_tokens"),
           py::arg("max_prefill_wait_steps") = 0)
      .def("reconfigure", &Scheduler::reconfigure, py::arg("policy") = "", py::arg("max_tokens_per_batch") = 0,
           py::arg("max_seqs_per_batch") = 0, py::arg("max_tokens_per_chunk_for_prefill") = 0)
      .def("pause", &Scheduler::pause)
      .def("resume", &Scheduler::resume)
      .def("is_drained", &Scheduler::is_drained)
      .def("paused", &Scheduler::paused)
      .def("reset_prefix_cache", &Scheduler::reset_prefix_cache)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def_property_readonly("num_prefilling", &Scheduler::num_prefilling)
      .def_property_readonly("num_requests", &Scheduler::num_requests)
      .def_property_readonly("num_preemptions", &Scheduler::num_preemptions)
      .def_property_readonly("num_window_released_blocks", &Scheduler::num_window_released_blocks)
      .def_property_readonly("num_admission_refusals", &Scheduler::num_admission_refusals)
      .def("block_manager", [](Scheduler& s, int dp) -> BlockManager& { return s.block_manager(dp); },
           py::arg("dp") = 0, py::return_value_policy::reference_internal)
      .def("block_stats", [](Scheduler& s, int dp) { return s.block_manager(dp).stats(); }, py::arg("dp") = 0)
      .def("kv_utilization", [](Scheduler& s, int dp) { return s.block_manager(dp).utilization(); },
           py::arg("dp") = 0);

  bind_runtime_extra(m);
  bind_frontend(m);
  bind_server(m);
}
