// Continuous-batching scheduler + batch input builder.
//
// Capability parity with the reference's ContinuousScheduler and its policies
// (xllm/core/scheduler/continuous_scheduler.cpp:300-517, 739-1018; scheduler_policy.cpp;
// prefill_first_policy.cpp:31-124; decode_first_policy.cpp; unified_policy.cpp) and with
// Batch / BatchInputBuilder / BatchFactory (xllm/core/framework/batch/batch.cpp:183-206,
// batch_input_builder.cpp:417-1400, batch_factory.cpp):
//   * waiting / running queues, token + sequence budgets per step, one batch per DP rank
//   * policies: prefill_first (prefill-only batches while prompt work exists, else decode),
//     decode_first (Sarathi: decodes first, prompt chunks fill the left-over token budget),
//     unified (same mix, but prompt chunks are ordered by deadline slack)
//   * chunked prefill, prefix-cache admission, recompute preemption when KV runs out,
//     online-preempts-offline, priority strategies fcfs / priority / deadline
//   * schedule overlap: a step can be scheduled before the previous step's tokens reached the
//     host; unknown input tokens are written as placeholders -(row+1) that the device resolves
//     from the previous step's sampled ids
//   * pause(KEEP | ABORT | WAIT) / resume for RL-style weight updates
//
// The scheduler produces flat arrays ready for one H2D copy (tokens, positions, slot mapping,
// q/kv lengths, block tables, sample rows, sampling parameters); decode rows come first, then
// prompt-chunk rows, so the attention layer can run its decode and prefill kernels on two
// contiguous halves.
#pragma once
#include <algorithm>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "block_manager.h"
#include "sequence.h"

namespace xllm {

struct SchedulerConfig {
  int32_t max_tokens_per_batch = 10240;
  int32_t max_seqs_per_batch = 1024;
  bool enable_chunked_prefill = true;
  int32_t max_tokens_per_chunk_for_prefill = -1;  // -1: the whole token budget
  bool enable_prefix_cache = true;
  int32_t block_size = 128;
  int32_t num_blocks = 0;  // per DP rank
  std::string policy = "prefill_first";
  // Admission rule on top of the batching policy:
  //   ""              admit while blocks last; a running sequence that cannot grow preempts others
  //   "zero_eviction" admit a request only when a simulation of every running sequence up to its
  //                   max_tokens shows that the pool never runs short, so nothing is ever preempted
  //                   (xllm/core/scheduler/zero_eviction_scheduler.cpp:200-237)
  //   "fixed_steps"   waves: requests are admitted only when nothing is running, then the whole wave
  //                   runs its (short, fixed) number of steps to the end; generative recommendation
  //                   (xllm/core/scheduler/fixed_steps_scheduler.h:49)
  std::string admission = "";
  // Sliding-window attention in every layer: KV blocks that lie entirely before the window of the
  // next query are given back while the sequence runs (0 = full attention)
  int32_t sliding_window = 0;
  std::string priority_strategy = "fcfs";
  double prefill_scheduling_memory_usage_threshold = 0.95;
  bool enable_schedule_overlap = false;
  bool enable_online_preempt_offline = true;
  int32_t dp_size = 1;
  int32_t num_speculative_tokens = 0;  // extra KV slots reserved per decode step
  int32_t max_decode_batch = 0;        // 0: max_seqs_per_batch
  // Cap on sequences that hold KV / state at the same time (running queue), 0 = no cap.  The
  // per-step sequence budget does not bound it: with prefill_first the running set grows over
  // successive steps.  Models with per-sequence state slots size their pool by this number.
  int32_t max_running_seqs = 0;
  // Prompt batching for the mixing policies (decode_first / unified): while sequences are decoding,
  // prompt chunks are only scheduled once at least `min_prefill_tokens` prompt tokens are pending,
  // or after `max_prefill_wait_steps` steps of holding them back.  Large prompt batches run the
  // GEMMs at their compute-bound rate; a trickle of small chunks makes every step pay for a
  // mid-size GEMM.  0 = schedule prompt work as soon as it exists.
  int32_t min_prefill_tokens = 0;
  int32_t max_prefill_wait_steps = 8;
  // PD disaggregation, prefill side: a sequence that finishes keeps its KV blocks until
  // release_held() so that they can be pushed to the decode instance first.
  bool hold_finished_blocks = false;
};

enum class PauseMode : int { KEEP = 0, ABORT = 1, WAIT = 2 };

struct Batch {
  int64_t batch_id = -1;
  int32_t dp_rank = 0;
  int32_t n_decode = 0;   // leading rows with q_len == 1 in decode stage
  int32_t n_prefill = 0;  // following sequences with q_len >= 1 (prompt chunks)
  int32_t n_tokens = 0;
  int32_t max_q_len = 0, max_kv_len = 0, max_blocks = 0;
  std::vector<int64_t> tokens, positions;
  std::vector<int32_t> slots;                 // [n_tokens]
  std::vector<int32_t> q_lens, kv_lens, cu_q; // per sequence; cu_q has n_seq + 1 entries
  std::vector<int32_t> block_tables;          // [n_seq, max_blocks], padded with 0
  std::vector<int64_t> sample_rows;           // token rows whose hidden state is sampled
  std::vector<int32_t> sample_seq;            // index into seqs for each sample row
  std::vector<float> temperature, top_p, freq_pen, pres_pen, rep_pen;
  std::vector<int32_t> top_k;
  std::vector<uint64_t> seeds;                // per sample row: the sequence's own random stream
  std::vector<int32_t> sample_offsets;        // per sample row: tokens the sequence has generated so far
  std::vector<int64_t> seq_ids;
  bool any_penalty = false, any_logprobs = false, all_greedy = true;
  int32_t max_top_logprobs = 0;               // widest `top_logprobs` request among the sample rows
  std::vector<Sequence*> seqs;  // not exposed
  int32_t n_seqs() const { return n_decode + n_prefill; }
  bool empty() const { return n_tokens == 0; }
};

struct OutputEvent {
  std::string request_id;
  int32_t seq_index = 0;
  int32_t token = -1;
  float logprob = 0.f;
  bool has_logprob = false;
  bool finished = false;
  std::string finish_reason;
  int32_t num_prompt_tokens = 0, num_generated = 0, prefix_hit_tokens = 0;
  bool request_finished = false;
  int64_t seq_id = -1;
  // the most likely alternatives at this position (requests with top_logprobs > 0), best first
  std::vector<int32_t> top_ids;
  std::vector<float> top_logprobs;
};

class Scheduler {
 public:
  explicit Scheduler(const SchedulerConfig& cfg) : cfg_(cfg) {
    if (cfg_.dp_size < 1) cfg_.dp_size = 1;
    for (int i = 0; i < cfg_.dp_size; ++i)
      bm_.emplace_back(new BlockManager(cfg_.num_blocks, cfg_.block_size, cfg_.enable_prefix_cache));
  }

  const SchedulerConfig& config() const { return cfg_; }

  // Change the batching policy and the per-step budgets of a live scheduler (takes effect at the
  // next schedule()); values <= 0 and an empty policy keep the current setting.
  void reconfigure(const std::string& policy, int32_t max_tokens_per_batch, int32_t max_seqs_per_batch,
                   int32_t max_tokens_per_chunk_for_prefill) {
    if (!policy.empty()) cfg_.policy = policy;
    if (max_tokens_per_batch > 0) cfg_.max_tokens_per_batch = max_tokens_per_batch;
    if (max_seqs_per_batch > 0) cfg_.max_seqs_per_batch = max_seqs_per_batch;
    if (max_tokens_per_chunk_for_prefill != 0) cfg_.max_tokens_per_chunk_for_prefill = max_tokens_per_chunk_for_prefill;
  }
  void set_prefill_batching(int32_t min_prefill_tokens, int32_t max_prefill_wait_steps) {
    cfg_.min_prefill_tokens = min_prefill_tokens;
    if (max_prefill_wait_steps > 0) cfg_.max_prefill_wait_steps = max_prefill_wait_steps;
  }
  BlockManager& block_manager(int dp = 0) { return *bm_[dp]; }

  // ---------------------------------------------------------------- intake
  bool add_request(const std::string& id, const std::vector<int32_t>& prompt, const SamplingParams& sp,
                   const StoppingParams& st, int32_t n, int32_t priority, double deadline, bool offline,
                   bool stream, uint64_t extra_hash_key = 0) {
    if (requests_.count(id) || prompt.empty() || n < 1) return false;
    auto req = std::make_unique<Request>();
    req->request_id = id;
    req->sampling = sp;
    req->stopping = st;
    req->priority = priority;
    req->deadline = deadline;
    req->offline = offline;
    req->stream = stream;
    req->arrival_time = now_seconds();
    for (int32_t i = 0; i < n; ++i) {
      auto s = std::make_unique<Sequence>();
      s->seq_id = next_seq_id_++;
      s->index = i;
      s->request = req.get();
      s->tokens = prompt;
      s->num_prompt_tokens = (int32_t)prompt.size();
      s->extra_hash_key = extra_hash_key;  // e.g. content hash of the images of a multimodal prompt
      req->seqs.push_back(std::move(s));
    }
    Request* r = req.get();
    requests_.emplace(id, std::move(req));
    if (pause_mode_active_ && pause_mode_ == PauseMode::ABORT) {
      // accepted but immediately aborted while paused in ABORT mode
      abort_request(id);
      return true;
    }
    // sibling samples wait until the first one has put the prompt in the prefix cache
    enqueue_waiting(r->seqs[0].get());
    if (!(cfg_.enable_prefix_cache && n > 1))
      for (int32_t i = 1; i < n; ++i) enqueue_waiting(r->seqs[i].get());
    return true;
  }

  // PD disaggregation, decode side: take over a request whose prompt was prefilled elsewhere.
  // `tokens` = prompt + the first generated token; KV of all but the last token is (about to be)
  // in the blocks returned here, which the caller fills through the KV transfer.  The sequence
  // enters the running queue in decode stage.  Returns an empty vector when blocks are short.
  std::vector<int32_t> adopt_prefilled(const std::string& id, const std::vector<int32_t>& tokens,
                                       int32_t num_prompt_tokens, const SamplingParams& sp, const StoppingParams& st,
                                       int32_t priority, bool offline, bool stream) {
    std::vector<int32_t> none;
    if (requests_.count(id) || (int32_t)tokens.size() < 2 || num_prompt_tokens < 1 ||
        num_prompt_tokens >= (int32_t)tokens.size())
      return none;
    BlockManager& bm = *bm_[0];
    const int32_t need = ((int32_t)tokens.size() + 1 + cfg_.num_speculative_tokens + cfg_.block_size - 1) / cfg_.block_size;
    std::vector<int32_t> blocks = bm.allocate(need);
    if ((int32_t)blocks.size() < need) return none;
    auto req = std::make_unique<Request>();
    req->request_id = id;
    req->sampling = sp;
    req->stopping = st;
    req->priority = priority;
    req->offline = offline;
    req->stream = stream;
    req->arrival_time = now_seconds();
    auto s = std::make_unique<Sequence>();
    s->seq_id = next_seq_id_++;
    s->request = req.get();
    s->tokens = tokens;
    s->num_prompt_tokens = num_prompt_tokens;
    s->kv_computed = (int32_t)tokens.size() - 1;
    s->blocks = blocks;
    s->stage = SeqStage::DECODE;
    s->first_token_time = req->arrival_time;
    Sequence* sp_ = s.get();
    req->seqs.push_back(std::move(s));
    requests_.emplace(id, std::move(req));
    running_.push_back(sp_);
    return blocks;
  }

  // PD disaggregation, decode side, in two phases (the prompt's KV is pushed into the reserved
  // blocks WHILE the prefill instance computes it, so the blocks must exist before the tokens do):
  // reserve_blocks() sets blocks aside for `n_tokens` (+ one decode step), adopt_reserved() turns
  // the reservation into a running sequence once the first token has arrived, cancel_reserved()
  // gives the blocks back (prefill side gone, request aborted).
  std::vector<int32_t> reserve_blocks(const std::string& id, int32_t n_tokens) {
    std::vector<int32_t> none;
    if (n_tokens < 1 || reserved_.count(id) || requests_.count(id)) return none;
    BlockManager& bm = *bm_[0];
    const int32_t need = (n_tokens + 2 + cfg_.num_speculative_tokens + cfg_.block_size - 1) / cfg_.block_size;
    std::vector<int32_t> blocks = bm.allocate(need);
    if ((int32_t)blocks.size() < need) return none;
    reserved_.emplace(id, blocks);
    return blocks;
  }
  bool cancel_reserved(const std::string& id) {
    auto it = reserved_.find(id);
    if (it == reserved_.end()) return false;
    bm_[0]->free_blocks(it->second);
    reserved_.erase(it);
    return true;
  }
  int32_t num_reserved() const { return (int32_t)reserved_.size(); }
  std::vector<std::string> reserved_ids() const {
    std::vector<std::string> out;
    for (auto& kv : reserved_) out.push_back(kv.first);
    return out;
  }
  bool adopt_reserved(const std::string& id, const std::vector<int32_t>& tokens, int32_t num_prompt_tokens,
                      const SamplingParams& sp, const StoppingParams& st, int32_t priority, bool offline,
                      bool stream) {
    auto it = reserved_.find(id);
    if (it == reserved_.end() || requests_.count(id) || (int32_t)tokens.size() < 2 || num_prompt_tokens < 1 ||
        num_prompt_tokens >= (int32_t)tokens.size())
      return false;
    const int32_t need = ((int32_t)tokens.size() + 1 + cfg_.num_speculative_tokens + cfg_.block_size - 1) / cfg_.block_size;
    if ((int32_t)it->second.size() < need) return false;
    auto req = std::make_unique<Request>();
    req->request_id = id;
    req->sampling = sp;
    req->stopping = st;
    req->priority = priority;
    req->offline = offline;
    req->stream = stream;
    req->arrival_time = now_seconds();
    auto s = std::make_unique<Sequence>();
    s->seq_id = next_seq_id_++;
    s->request = req.get();
    s->tokens = tokens;
    s->num_prompt_tokens = num_prompt_tokens;
    s->kv_computed = (int32_t)tokens.size() - 1;
    s->blocks = it->second;
    s->stage = SeqStage::DECODE;
    s->first_token_time = req->arrival_time;
    Sequence* sp_ = s.get();
    req->seqs.push_back(std::move(s));
    requests_.emplace(id, std::move(req));
    running_.push_back(sp_);
    reserved_.erase(it);
    return true;
  }

  // Prefill side of a disaggregated pair: finished prompts keep their blocks until released.
  void set_hold_finished_blocks(bool on) { cfg_.hold_finished_blocks = on; }
  // Blocks of a finished sequence that hold_finished_blocks kept alive (empty if none).
  std::vector<int32_t> held_blocks(const std::string& id) const {
    auto it = held_.find(id);
    return it == held_.end() ? std::vector<int32_t>() : it->second;
  }
  void release_held(const std::string& id) {
    auto it = held_.find(id);
    if (it == held_.end()) return;
    bm_[0]->free_blocks(it->second);
    held_.erase(it);
  }

  bool abort_request(const std::string& id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return false;
    Request* r = it->second.get();
    r->aborted = true;
    for (auto& s : r->seqs) {
      if (s->finished()) continue;
      remove_from_queues(s.get());
      finish_seq(s.get(), FinishReason::ABORT);
    }
    pending_events_.push_back(make_event(r->seqs[0].get(), -1, 0.f, false));
    pending_events_.back().request_finished = true;
    maybe_erase_request(r);
    return true;
  }

  // ---------------------------------------------------------------- scheduling
  std::vector<Batch> schedule() {
    std::vector<Batch> out;
    if (paused_) return out;
    for (int dp = 0; dp < cfg_.dp_size; ++dp) {
      Batch b = schedule_dp(dp);
      if (!b.empty()) {
        b.batch_id = next_batch_id_++;
        InFlight f;  // what process_output needs once the device is done
        f.seqs = b.seqs;
        f.q_lens = b.q_lens;
        f.sample_seq = b.sample_seq;
        f.n_decode = b.n_decode;
        in_flight_batches_.emplace(b.batch_id, std::move(f));
        out.push_back(std::move(b));
      }
    }
    return out;
  }

  // next_tokens: one id per sample row of the batch (in order).  logprobs may be null.
  std::vector<OutputEvent> process_output(int64_t batch_id, const int64_t* next_tokens, int64_t n,
                                          const float* logprobs) {
    return process_output_multi(batch_id, next_tokens, nullptr, n, logprobs);
  }

  // Speculative decoding: sample row r appends counts[r] >= 1 tokens (the accepted draft tokens
  // followed by the bonus / corrected token), read consecutively from `tokens` (and `logprobs`).
  // counts == null means one token per row.  The KV of every appended token but the last is in the
  // cache already (the verification pass wrote it), which keeps the invariant
  // kv_computed == num_tokens - 1 for sequences in decode.  A stop condition met in the middle of
  // a row drops the rest of that row.
  std::vector<OutputEvent> process_output_multi(int64_t batch_id, const int64_t* tokens, const int32_t* counts,
                                                int64_t n_rows, const float* logprobs) {
    std::vector<OutputEvent> ev;
    ev.swap(pending_events_);
    auto it = in_flight_batches_.find(batch_id);
    if (it == in_flight_batches_.end()) return ev;
    InFlight& b = it->second;
    const double t = now_seconds();
    // prompt chunks: advance kv_computed and publish full blocks to the prefix cache
    for (int32_t i = 0; i < (int32_t)b.seqs.size(); ++i) {
      Sequence* s = b.seqs[i];
      if (s->in_flight > 0) s->in_flight--;
      if (s->finished()) continue;
      if (i >= b.n_decode) {
        s->kv_computed += b.q_lens[i];
        publish_blocks(s);
        if (s->kv_computed >= s->num_tokens()) {
          s->stage = SeqStage::DECODE;
          release_siblings(s);
        }
      } else if (counts == nullptr) {
        s->kv_computed += 1;
      }
    }
    const int64_t ns = std::min<int64_t>(n_rows, (int64_t)b.sample_seq.size());
    int64_t cursor = 0;
    for (int64_t r = 0; r < ns; ++r) {
      const int32_t cnt = counts ? std::max<int32_t>(counts[r], 1) : 1;
      const int64_t base = cursor;
      cursor += cnt;
      const int32_t si = b.sample_seq[r];
      Sequence* s = b.seqs[si];
      if (s->pending_samples > 0) s->pending_samples--;
      if (s->finished()) continue;  // finished (or aborted) while this step was in flight
      for (int32_t j = 0; j < cnt; ++j) {
        const int32_t tok = (int32_t)tokens[base + j];
        s->tokens.push_back(tok);
        if (counts != nullptr && si < b.n_decode) s->kv_computed += 1;
        if (s->first_token_time == 0) s->first_token_time = t;
        s->last_token_time = t;
        const bool want_lp = s->request->sampling.logprobs && logprobs != nullptr;
        if (want_lp) s->logprobs.push_back(logprobs[base + j]);
        const FinishReason fr = check_stop(*s, s->request->stopping);
        if (fr != FinishReason::NONE) {
          remove_from_queues(s);
          finish_seq(s, fr);
        }
        ev.push_back(make_event(s, tok, want_lp ? logprobs[base + j] : 0.f, want_lp));
        if (want_lp && b.top_n > 0 && counts == nullptr && (r + 1) * b.top_n <= (int64_t)b.top_ids.size()) {
          const int32_t k = std::min<int32_t>(b.top_n, s->request->sampling.top_logprobs);
          ev.back().top_ids.assign(b.top_ids.begin() + r * b.top_n, b.top_ids.begin() + r * b.top_n + k);
          ev.back().top_logprobs.assign(b.top_lps.begin() + r * b.top_n, b.top_lps.begin() + r * b.top_n + k);
        }
        if (s->request->all_finished()) ev.back().request_finished = true;
        if (s->finished()) break;
      }
    }
    // free blocks of sequences that finished earlier but still had this step in flight
    for (Sequence* s : b.seqs)
      if (s->finished() && s->in_flight == 0 && !s->blocks.empty()) release_blocks(s);
    std::vector<Request*> done;
    for (Sequence* s : b.seqs)
      if (s->request->all_finished()) done.push_back(s->request);
    in_flight_batches_.erase(it);
    std::sort(done.begin(), done.end());
    done.erase(std::unique(done.begin(), done.end()), done.end());
    for (Request* r : done) maybe_erase_request(r);
    return ev;
  }

  // Alternatives for the sample rows of a batch still in flight: ids / logprobs are [n_rows, n]
  // (best first); the next process_output of that batch attaches the first `top_logprobs` of each
  // row to its event.  One token per row only (no speculative rows).
  void set_top_logprobs(int64_t batch_id, const int32_t* ids, const float* lps, int64_t n_rows, int32_t n) {
    auto it = in_flight_batches_.find(batch_id);
    if (it == in_flight_batches_.end() || n <= 0) return;
    it->second.top_n = n;
    it->second.top_ids.assign(ids, ids + n_rows * n);
    it->second.top_lps.assign(lps, lps + n_rows * n);
  }

  // Sequence ids preempted since the last call (their KV - and any per-sequence state - is gone and
  // will be rebuilt from position 0).
  std::vector<int64_t> take_preempted() {
    std::vector<int64_t> out;
    out.swap(preempted_ids_);
    return out;
  }

  std::vector<OutputEvent> take_pending_events() {
    std::vector<OutputEvent> ev;
    ev.swap(pending_events_);
    return ev;
  }

  // ---------------------------------------------------------------- control
  void pause(PauseMode mode) {
    pause_mode_ = mode;
    pause_mode_active_ = true;
    if (mode == PauseMode::ABORT) {
      std::vector<std::string> ids;
      for (auto& kv : requests_) ids.push_back(kv.first);
      for (auto& id : ids) abort_request(id);
      paused_ = true;
    } else if (mode == PauseMode::KEEP) {
      // running sequences keep their tokens, give their KV back and re-prefill after resume
      std::vector<Sequence*> run = running_;
      for (Sequence* s : run) preempt(s);
      paused_ = true;
    } else {
      // WAIT: stop admitting, let running sequences drain; the caller polls is_drained()
      admit_blocked_ = true;
    }
  }
  bool is_drained() const { return running_.empty() && in_flight_batches_.empty(); }
  void resume() {
    paused_ = false;
    admit_blocked_ = false;
    pause_mode_active_ = false;
  }
  bool paused() const { return paused_ || admit_blocked_; }
  void reset_prefix_cache() {
    for (auto& b : bm_) b->reset_prefix_cache();
  }

  bool has_unfinished() const { return !waiting_.empty() || !running_.empty() || !in_flight_batches_.empty(); }
  int64_t num_waiting() const { return (int64_t)waiting_.size(); }
  int64_t num_running() const { return (int64_t)running_.size(); }
  // running sequences whose prompt is not in the cache yet (a chunk may be in flight)
  int64_t num_prefilling() const {
    int64_t n = 0;
    for (const Sequence* s : running_) n += s->stage == SeqStage::PREFILL ? 1 : 0;
    return n;
  }
  int64_t num_requests() const { return (int64_t)requests_.size(); }
  int64_t num_preemptions() const { return preemptions_; }
  int64_t num_window_released_blocks() const { return window_released_blocks_; }
  int64_t num_admission_refusals() const { return admission_refusals_; }

 private:
  std::unordered_map<std::string, std::vector<int32_t>> held_;
  std::unordered_map<std::string, std::vector<int32_t>> reserved_;
  int64_t window_released_blocks_ = 0;
  int64_t admission_refusals_ = 0;  // decode side of PD: blocks awaiting a prefill
  struct InFlight {
    std::vector<Sequence*> seqs;
    std::vector<int32_t> q_lens, sample_seq;
    int32_t n_decode = 0;
    int32_t top_n = 0;
    std::vector<int32_t> top_ids;
    std::vector<float> top_lps;
  };
  // ---------------------------------------------------------------- queues
  bool before(const Sequence* a, const Sequence* b) const {
    const Request *ra = a->request, *rb = b->request;
    if (cfg_.enable_online_preempt_offline && ra->offline != rb->offline) return !ra->offline;
    if (cfg_.priority_strategy == "priority" && ra->priority != rb->priority) return ra->priority > rb->priority;
    if (cfg_.priority_strategy == "deadline" && ra->deadline != rb->deadline) {
      if (ra->deadline == 0) return false;
      if (rb->deadline == 0) return true;
      return ra->deadline < rb->deadline;
    }
    if (ra->arrival_time != rb->arrival_time) return ra->arrival_time < rb->arrival_time;
    return a->seq_id < b->seq_id;
  }

  void enqueue_waiting(Sequence* s, bool front = false) {
    s->stage = SeqStage::WAITING;
    if (front) {
      // a preempted sequence goes back ahead of everything of equal or lower urgency
      auto it = waiting_.begin();
      while (it != waiting_.end() && before(*it, s)) ++it;
      waiting_.insert(it, s);
      return;
    }
    auto it = waiting_.end();
    while (it != waiting_.begin() && before(s, *(it - 1))) --it;
    waiting_.insert(it, s);
  }

  void remove_from_queues(Sequence* s) {
    auto it = std::find(running_.begin(), running_.end(), s);
    if (it != running_.end()) running_.erase(it);
    auto wt = std::find(waiting_.begin(), waiting_.end(), s);
    if (wt != waiting_.end()) waiting_.erase(wt);
  }

  void release_siblings(Sequence* s) {
    Request* r = s->request;
    if (s->index != 0 || r->seqs.size() <= 1 || !cfg_.enable_prefix_cache) return;
    for (size_t i = 1; i < r->seqs.size(); ++i) {
      Sequence* sib = r->seqs[i].get();
      if (sib->stage == SeqStage::WAITING && !sib->finished() &&
          std::find(waiting_.begin(), waiting_.end(), sib) == waiting_.end() && sib->blocks.empty())
        enqueue_waiting(sib, /*front=*/true);
    }
  }

  void publish_blocks(Sequence* s) {
    BlockManager& bm = *bm_[s->dp_rank];
    if (bm.prefix_cache_enabled()) {
      const int32_t full = std::min<int32_t>(s->kv_computed, s->num_tokens()) / cfg_.block_size;
      if (full > s->cached_blocks) {
        bm.cache_blocks(s->tokens.data(), (int64_t)full * cfg_.block_size, s->blocks, s->cached_blocks,
                        s->extra_hash_key);
        s->cached_blocks = full;
      }
    }
    release_out_of_window(s);
  }

  // Sliding window: the next query (position >= kv_computed) attends to positions > its own minus
  // the window, so blocks that end at or before kv_computed - window are dead.  Their table entries
  // become the padding block (0), which the windowed attention kernels never read.
  void release_out_of_window(Sequence* s) {
    if (cfg_.sliding_window <= 0 || s->in_flight > 0) return;
    const int32_t dead = (s->kv_computed - cfg_.sliding_window + 1) / cfg_.block_size;
    if (dead <= s->window_released) return;
    std::vector<int32_t> give;
    for (int32_t i = s->window_released; i < dead && i < (int32_t)s->blocks.size(); ++i) {
      if (s->blocks[i] > 0) give.push_back(s->blocks[i]);
      s->blocks[i] = 0;
    }
    s->window_released = dead;
    window_released_blocks_ += (int64_t)give.size();
    bm_[s->dp_rank]->free_blocks(give);
  }

  // zero_eviction / fixed_steps: would the pool of rank `dp` hold every running sequence plus
  // `cand` all the way to their stopping lengths?  Sequences are sorted by remaining steps; the
  // demand peaks right before one of them finishes, so only those moments are checked.
  bool fits_without_eviction(const Sequence* cand, int dp) const {
    struct Item { int64_t len, remaining; };
    std::vector<Item> items;
    int64_t held = 0;
    auto add = [&](const Sequence* q) {
      const int64_t len = q->num_tokens();
      int64_t rem = (int64_t)q->request->stopping.max_tokens - q->num_generated();
      if (q->request->stopping.max_context_len > 0)
        rem = std::min<int64_t>(rem, (int64_t)q->request->stopping.max_context_len - len);
      items.push_back({len, std::max<int64_t>(rem, 0)});
    };
    for (const Sequence* q : running_) {
      if (q->dp_rank != dp || q->finished()) continue;
      add(q);
      for (int32_t b : q->blocks) held += b > 0;
    }
    add(cand);
    std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.remaining < b.remaining; });
    const int64_t bs = cfg_.block_size, extra = 1 + cfg_.num_speculative_tokens;
    const int64_t capacity = bm_[dp]->num_free_blocks() + held;
    for (size_t k = 0; k < items.size(); ++k) {
      const int64_t t = items[k].remaining;
      int64_t demand = 0;
      for (size_t i = k; i < items.size(); ++i) demand += (items[i].len + t + extra + bs - 1) / bs;
      if (demand > capacity) return false;
    }
    return true;
  }

  void release_blocks(Sequence* s) {
    if (s->blocks.empty()) return;
    if (cfg_.hold_finished_blocks && s->finished() && s->finish_reason != FinishReason::ABORT && s->index == 0 &&
        !held_.count(s->request->request_id)) {
      held_[s->request->request_id] = s->blocks;  // ownership moves to the hold table
      s->blocks.clear();
      s->cached_blocks = 0;
      return;
    }
    bm_[s->dp_rank]->free_blocks(s->blocks);
    s->blocks.clear();
    s->cached_blocks = 0;
    s->window_released = 0;
  }

  void finish_seq(Sequence* s, FinishReason fr) {
    s->finish_reason = fr;
    s->stage = SeqStage::FINISHED;
    s->finish_time = now_seconds();
    if (fr != FinishReason::ABORT) publish_blocks(s);
    if (s->in_flight == 0) release_blocks(s);  // else freed when the in-flight step returns
  }

  void maybe_erase_request(Request* r) {
    if (!r->all_finished()) return;
    for (auto& s : r->seqs)
      if (s->in_flight > 0 || !s->blocks.empty()) return;
    for (auto& kv : in_flight_batches_)
      for (Sequence* s : kv.second.seqs)
        if (s->request == r) return;
    requests_.erase(r->request_id);
  }

  void preempt(Sequence* s) {
    auto it = std::find(running_.begin(), running_.end(), s);
    if (it != running_.end()) running_.erase(it);
    release_blocks(s);
    s->kv_computed = 0;
    s->preempt_count++;
    preemptions_++;
    preempted_ids_.push_back(s->seq_id);
    enqueue_waiting(s, /*front=*/true);
  }

  OutputEvent make_event(Sequence* s, int32_t tok, float lp, bool has_lp) {
    OutputEvent e;
    e.request_id = s->request->request_id;
    e.seq_index = s->index;
    e.seq_id = s->seq_id;
    e.token = tok;
    e.logprob = lp;
    e.has_logprob = has_lp;
    e.finished = s->finished();
    e.finish_reason = finish_reason_str(s->finish_reason);
    e.num_prompt_tokens = s->num_prompt_tokens;
    e.num_generated = s->num_generated();
    e.prefix_hit_tokens = s->prefix_hit_tokens;
    return e;
  }

  // Make sure `s` owns blocks for `upto` tokens. Returns false when memory is short.
  bool ensure_blocks(Sequence* s, int32_t upto) {
    const int32_t need = (upto + cfg_.block_size - 1) / cfg_.block_size - (int32_t)s->blocks.size();
    if (need <= 0) return true;
    auto nb = bm_[s->dp_rank]->allocate(need);
    if ((int32_t)nb.size() < need) return false;
    s->blocks.insert(s->blocks.end(), nb.begin(), nb.end());
    return true;
  }

  int pick_dp_rank() const {
    int best = 0;
    int64_t best_free = -1;
    for (int i = 0; i < cfg_.dp_size; ++i) {
      const int64_t f = bm_[i]->num_free_blocks();
      if (f > best_free) { best_free = f; best = i; }
    }
    return best;
  }

  struct Pick {
    Sequence* s;
    int32_t n_new;
    bool decode;
  };

  static bool picked_in(const std::vector<Pick>& v, const Sequence* s) {
    for (auto& p : v)
      if (p.s == s) return true;
    return false;
  }

  Batch schedule_dp(int dp) {
    const bool overlap = cfg_.enable_schedule_overlap;
    int32_t tok_budget = cfg_.max_tokens_per_batch;
    int32_t seq_budget = cfg_.max_seqs_per_batch;
    const int32_t chunk_cap = !cfg_.enable_chunked_prefill ? INT32_MAX
                              : (cfg_.max_tokens_per_chunk_for_prefill > 0 ? cfg_.max_tokens_per_chunk_for_prefill
                                                                           : cfg_.max_tokens_per_batch);
    std::vector<Pick> decodes, prefills;
    BlockManager& bm = *bm_[dp];

    // running sequences of this rank, most urgent first
    std::vector<Sequence*> run;
    for (Sequence* s : running_)
      if (s->dp_rank == dp) run.push_back(s);
    std::stable_sort(run.begin(), run.end(), [&](Sequence* a, Sequence* b) { return before(a, b); });
    auto still_running = [&](Sequence* s) {
      return (s->stage == SeqStage::DECODE || s->stage == SeqStage::PREFILL) && !s->finished();
    };
    // least urgent running sequence that can give its KV back (not `keep`, not already picked,
    // nothing in flight)
    auto find_victim = [&](Sequence* keep, bool offline_only) -> Sequence* {
      for (size_t j = run.size(); j-- > 0;) {
        Sequence* c = run[j];
        if (c == keep) { if (!offline_only) break; else continue; }  // only less urgent ones
        if (!still_running(c) || c->in_flight > 0 || c->blocks.empty()) continue;
        if (offline_only && !c->request->offline) continue;
        if (picked_in(decodes, c) || picked_in(prefills, c)) continue;
        return c;
      }
      return nullptr;
    };

    bool prompt_work = !admit_blocked_ && !waiting_.empty();
    for (Sequence* s : run)
      if (s->stage == SeqStage::PREFILL && s->in_flight == 0 && s->kv_computed < s->num_tokens())
        prompt_work = true;

    auto try_decode = [&]() {
      for (Sequence* s : run) {
        if (tok_budget <= 0 || seq_budget <= 0) break;
        if (s->stage != SeqStage::DECODE || s->finished()) continue;
        if (s->in_flight > (overlap ? 1 : 0)) continue;  // at most one step ahead of the device
        if (s->num_generated() + s->pending_samples >= s->request->stopping.max_tokens) continue;
        const int32_t upto = s->num_tokens() + s->pending_samples + cfg_.num_speculative_tokens;
        bool ok = ensure_blocks(s, upto);
        while (!ok) {
          Sequence* victim = find_victim(s, false);
          if (!victim) break;
          preempt(victim);
          ok = ensure_blocks(s, upto);
        }
        if (!ok) {
          // nobody less urgent to evict: if this is the only sequence left, it can never grow
          int alive = 0;
          for (Sequence* c : run) alive += still_running(c) ? 1 : 0;
          if (alive == 1 && s->in_flight == 0) {
            remove_from_queues(s);
            finish_seq(s, FinishReason::LENGTH);
            pending_events_.push_back(make_event(s, -1, 0.f, false));
            pending_events_.back().request_finished = s->request->all_finished();
          } else if (decodes.empty() && s->in_flight == 0) {
            preempt(s);  // free its KV so that more urgent sequences can move
          }
          continue;
        }
        decodes.push_back({s, 1, true});
        tok_budget -= 1;
        seq_budget -= 1;
      }
    };

    auto try_prefill = [&]() {
      // continue partially prefilled running sequences, then admit waiting ones
      for (Sequence* s : run) {
        if (tok_budget <= 0 || seq_budget <= 0) return;
        if (s->stage != SeqStage::PREFILL || s->finished() || s->in_flight > 0) continue;
        const int32_t remaining = s->num_tokens() - s->kv_computed;
        if (remaining <= 0) continue;
        const int32_t n_new = std::min({remaining, tok_budget, chunk_cap});
        if (!ensure_blocks(s, s->kv_computed + n_new)) continue;
        prefills.push_back({s, n_new, false});
        tok_budget -= n_new;
        seq_budget -= 1;
      }
      if (admit_blocked_) return;
      while (!waiting_.empty() && tok_budget > 0 && seq_budget > 0) {
        if (cfg_.max_running_seqs > 0 && (int32_t)running_.size() >= cfg_.max_running_seqs) break;
        Sequence* s = waiting_.front();
        if (cfg_.admission == "fixed_steps" && !run.empty()) break;   // a wave is running: the next one waits
        if (!cfg_.admission.empty() && !fits_without_eviction(s, dp)) {
          if (running_.empty() && in_flight_batches_.empty()) {
            // alone it still does not fit up to its stopping length: it never will
            waiting_.pop_front();
            finish_seq(s, FinishReason::LENGTH);
            pending_events_.push_back(make_event(s, -1, 0.f, false));
            pending_events_.back().request_finished = s->request->all_finished();
            continue;
          }
          ++admission_refusals_;
          break;
        }
        const int target_dp = cfg_.dp_size == 1 ? 0 : pick_dp_rank();
        if (target_dp != dp) break;  // this request goes to another rank's batch
        if (!cfg_.enable_chunked_prefill && s->num_tokens() > tok_budget &&
            (!prefills.empty() || !decodes.empty() || s->num_tokens() <= cfg_.max_tokens_per_batch))
          break;  // whole prompts only: wait for a step with room
        s->dp_rank = dp;
        // prefix cache: share the longest cached run of whole blocks
        std::vector<int32_t> shared = bm.match_prefix(s->tokens.data(), s->num_tokens(), s->extra_hash_key);
        const int32_t hit = (int32_t)shared.size() * cfg_.block_size;
        const int32_t remaining = s->num_tokens() - hit;
        const int32_t n_new = cfg_.enable_chunked_prefill ? std::min({remaining, tok_budget, chunk_cap}) : remaining;
        const int32_t need = (hit + n_new + cfg_.block_size - 1) / cfg_.block_size - (int32_t)shared.size();
        int alive = 0;
        for (Sequence* c : run) alive += still_running(c) ? 1 : 0;
        const int64_t reserve = (alive == 0 && prefills.empty()) ? 0
            : (int64_t)((1.0 - cfg_.prefill_scheduling_memory_usage_threshold) * (bm.num_blocks() - 1));
        if (bm.num_free_blocks() - need < reserve) {
          bm.free_blocks(shared);
          // an online request may push out offline work
          if (cfg_.enable_online_preempt_offline && !s->request->offline) {
            Sequence* victim = find_victim(nullptr, true);
            if (victim) {
              preempt(victim);
              continue;
            }
          }
          if (alive == 0 && prefills.empty() && decodes.empty() && in_flight_batches_.empty() &&
              bm.num_free_blocks() < need) {
            // the cache is empty and the first chunk still does not fit: it never will
            waiting_.pop_front();
            finish_seq(s, FinishReason::LENGTH);
            pending_events_.push_back(make_event(s, -1, 0.f, false));
            pending_events_.back().request_finished = s->request->all_finished();
            continue;
          }
          break;
        }
        s->blocks = std::move(shared);
        s->cached_blocks = (int32_t)s->blocks.size();
        s->kv_computed = hit;
        s->prefix_hit_tokens = hit;
        if (!ensure_blocks(s, hit + n_new)) {
          release_blocks(s);
          s->kv_computed = 0;
          break;
        }
        waiting_.pop_front();
        s->stage = SeqStage::PREFILL;
        if (s->request->schedule_time == 0) s->request->schedule_time = now_seconds();
        running_.push_back(s);
        prefills.push_back({s, n_new, false});
        tok_budget -= n_new;
        seq_budget -= 1;
      }
    };

    if (cfg_.policy == "prefill_first") {
      if (prompt_work) try_prefill();
      if (prefills.empty()) try_decode();
    } else {
      try_decode();
      if (cfg_.min_prefill_tokens > 0 && prompt_work && !decodes.empty()) {
        // hold small amounts of prompt work back while the step has decode rows anyway
        int64_t pending = 0;
        for (Sequence* s : run)
          if (s->stage == SeqStage::PREFILL && s->in_flight == 0) pending += s->num_tokens() - s->kv_computed;
        if (!admit_blocked_)
          for (Sequence* s : waiting_) {
            pending += s->num_tokens();
            if (pending >= cfg_.min_prefill_tokens) break;
          }
        if (pending < cfg_.min_prefill_tokens && prefill_held_steps_ < cfg_.max_prefill_wait_steps) {
          ++prefill_held_steps_;
          return build_batch(dp, decodes, prefills);
        }
      }
      prefill_held_steps_ = 0;
      if (cfg_.policy == "unified") {
        // prompt work ordered by deadline (earliest first), the configured order otherwise
        std::stable_sort(waiting_.begin(), waiting_.end(), [&](Sequence* a, Sequence* b) {
          const double da = a->request->deadline, db = b->request->deadline;
          if (da != db && da != 0 && db != 0) return da < db;
          return false;
        });
      }
      try_prefill();
    }
    return build_batch(dp, decodes, prefills);
  }

  Batch build_batch(int dp, const std::vector<Pick>& decodes, const std::vector<Pick>& prefills) {
    Batch b;
    b.dp_rank = dp;
    b.n_decode = (int32_t)decodes.size();
    b.n_prefill = (int32_t)prefills.size();
    const int32_t n_seq = b.n_seqs();
    if (n_seq == 0) return b;
    const int32_t bs = cfg_.block_size;
    for (auto& p : decodes) b.n_tokens += p.n_new;
    for (auto& p : prefills) b.n_tokens += p.n_new;
    b.tokens.reserve(b.n_tokens);
    b.positions.reserve(b.n_tokens);
    b.slots.reserve(b.n_tokens);
    b.cu_q.push_back(0);
    // placeholder rows refer to the sample order of the previous batch of this rank
    const std::unordered_map<Sequence*, int32_t>& prev_rows = last_sample_row_[dp];
    std::unordered_map<Sequence*, int32_t> new_rows;
    auto add = [&](const Pick& p) {
      Sequence* s = p.s;
      const int32_t idx = (int32_t)b.seqs.size();
      const int32_t start = p.decode ? s->num_tokens() - 1 + s->pending_samples : s->kv_computed;
      for (int32_t i = 0; i < p.n_new; ++i) {
        const int32_t pos = start + i;
        int64_t tok;
        if (pos < s->num_tokens()) {
          tok = s->tokens[pos];
        } else {
          auto it = prev_rows.find(s);
          tok = it != prev_rows.end() ? -(int64_t)(it->second + 1) : 0;
        }
        b.tokens.push_back(tok);
        b.positions.push_back(pos);
        b.slots.push_back(s->blocks[pos / bs] * bs + pos % bs);
      }
      const int32_t kv_len = start + p.n_new;
      b.q_lens.push_back(p.n_new);
      b.kv_lens.push_back(kv_len);
      b.cu_q.push_back(b.cu_q.back() + p.n_new);
      b.max_q_len = std::max(b.max_q_len, p.n_new);
      b.max_kv_len = std::max(b.max_kv_len, kv_len);
      // with speculative decoding the table also covers the slots reserved for the draft tokens
      b.max_blocks = std::max(b.max_blocks, (kv_len + cfg_.num_speculative_tokens + bs - 1) / bs);
      b.seqs.push_back(s);
      b.seq_ids.push_back(s->seq_id);
      const bool samples = p.decode || (start + p.n_new >= s->num_tokens());
      if (samples) {
        new_rows[s] = (int32_t)b.sample_rows.size();
        b.sample_rows.push_back(b.cu_q.back() - 1);
        b.sample_seq.push_back(idx);
        const SamplingParams& sp = s->request->sampling;
        b.temperature.push_back(sp.temperature);
        b.top_p.push_back(sp.top_p);
        b.top_k.push_back(sp.top_k);
        b.freq_pen.push_back(sp.frequency_penalty);
        b.pres_pen.push_back(sp.presence_penalty);
        b.rep_pen.push_back(sp.repetition_penalty);
        // one random stream per sequence (parallel samples of a request must not draw the same
        // numbers), advanced by the number of tokens generated so far: a sample depends neither on
        // the row a sequence happens to occupy nor on who shares the batch
        b.seeds.push_back(sp.seed + 0x9E3779B97F4A7C15ull * (uint64_t)s->index);
        b.sample_offsets.push_back(s->num_generated() + s->pending_samples);
        b.any_penalty |= sp.has_penalty();
        b.any_logprobs |= sp.logprobs;
        if (sp.logprobs) b.max_top_logprobs = std::max(b.max_top_logprobs, sp.top_logprobs);
        b.all_greedy &= !(sp.temperature > 0.f);
        s->pending_samples++;
      }
      s->in_flight++;
    };
    for (auto& p : decodes) add(p);
    for (auto& p : prefills) add(p);
    b.block_tables.assign((size_t)n_seq * b.max_blocks, 0);
    for (int32_t i = 0; i < n_seq; ++i) {
      Sequence* s = b.seqs[i];
      const int32_t nb = std::min<int32_t>((int32_t)s->blocks.size(), b.max_blocks);
      std::copy(s->blocks.begin(), s->blocks.begin() + nb, b.block_tables.begin() + (size_t)i * b.max_blocks);
    }
    last_sample_row_[dp] = std::move(new_rows);
    return b;
  }

  SchedulerConfig cfg_;
  std::vector<std::unique_ptr<BlockManager>> bm_;
  std::unordered_map<std::string, std::unique_ptr<Request>> requests_;
  std::deque<Sequence*> waiting_;
  std::vector<Sequence*> running_;
  std::map<int64_t, InFlight> in_flight_batches_;
  std::map<int, std::unordered_map<Sequence*, int32_t>> last_sample_row_;
  std::vector<OutputEvent> pending_events_;
  std::vector<int64_t> preempted_ids_;
  int64_t next_seq_id_ = 0, next_batch_id_ = 0, preemptions_ = 0;
  int32_t prefill_held_steps_ = 0;
  bool paused_ = false, admit_blocked_ = false, pause_mode_active_ = false;
  PauseMode pause_mode_ = PauseMode::KEEP;
};

}  // namespace xllm
