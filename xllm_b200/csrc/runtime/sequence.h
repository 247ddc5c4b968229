// Request / Sequence model and stop checking.
//
// Capability parity with the reference's framework/request (Request, RequestState, Sequence,
// SequencesGroup, StoppingChecker, RequestParams: xllm/core/framework/request/sequence.cpp,
// stopping_checker.cpp, request_params.cpp).  A Request owns `n` Sequences (parallel samples /
// best_of / beams share the prompt through the prefix cache); the scheduler works on Sequences.
#pragma once
#include <chrono>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace xllm {

inline double now_seconds() {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

struct SamplingParams {
  float temperature = 0.0f;  // <= 0 => greedy
  float top_p = 1.0f;
  int32_t top_k = -1;
  float frequency_penalty = 0.0f;
  float presence_penalty = 0.0f;
  float repetition_penalty = 1.0f;
  bool logprobs = false;
  int32_t top_logprobs = 0;
  uint64_t seed = 0;
  bool has_penalty() const {
    return frequency_penalty != 0.f || presence_penalty != 0.f || repetition_penalty != 1.f;
  }
};

struct StoppingParams {
  int32_t max_tokens = 16;
  int32_t max_context_len = 0;  // 0 = unlimited
  int32_t eos_token_id = -1;
  bool ignore_eos = false;
  std::vector<int32_t> stop_token_ids;
  std::vector<std::vector<int32_t>> stop_sequences;  // token-id sequences
};

enum class FinishReason : int { NONE = 0, STOP = 1, LENGTH = 2, ABORT = 3, FUNCTION_CALL = 4 };

inline const char* finish_reason_str(FinishReason r) {
  switch (r) {
    case FinishReason::STOP: return "stop";
    case FinishReason::LENGTH: return "length";
    case FinishReason::ABORT: return "abort";
    case FinishReason::FUNCTION_CALL: return "function_call";
    default: return "";
  }
}

enum class SeqStage : int { WAITING = 0, PREFILL = 1, DECODE = 2, FINISHED = 3 };

struct Request;

struct Sequence {
  int64_t seq_id = 0;
  int32_t index = 0;  // index inside the request (n > 1)
  Request* request = nullptr;
  std::vector<int32_t> tokens;  // prompt + generated
  int32_t num_prompt_tokens = 0;
  int32_t kv_computed = 0;       // tokens whose KV is in the cache
  int32_t cached_blocks = 0;     // leading blocks already registered in the prefix cache
  int32_t prefix_hit_tokens = 0; // tokens served from the prefix cache at admission
  std::vector<int32_t> blocks;
  int32_t dp_rank = 0;
  SeqStage stage = SeqStage::WAITING;
  FinishReason finish_reason = FinishReason::NONE;
  std::vector<float> logprobs;   // per generated token (when requested)
  double first_token_time = 0, last_token_time = 0, finish_time = 0;
  int32_t preempt_count = 0;
  int32_t window_released = 0;   // leading blocks given back because they fell out of the sliding window
  int32_t in_flight = 0;         // batches containing this sequence that the device has not returned yet
  int32_t pending_samples = 0;   // of those, how many will append a token
  uint64_t extra_hash_key = 0;   // e.g. multimodal / LoRA discriminator for the prefix cache

  int32_t num_tokens() const { return (int32_t)tokens.size(); }
  int32_t num_generated() const { return num_tokens() - num_prompt_tokens; }
  bool finished() const { return stage == SeqStage::FINISHED; }
};

struct Request {
  std::string request_id;
  SamplingParams sampling;
  StoppingParams stopping;
  int32_t priority = 0;       // larger = more urgent (priority strategy)
  double deadline = 0;        // absolute seconds (deadline strategy)
  bool offline = false;       // offline requests can be preempted by online ones
  bool stream = false;
  double arrival_time = 0;
  double schedule_time = 0;
  std::vector<std::unique_ptr<Sequence>> seqs;
  bool aborted = false;
  bool all_finished() const {
    for (auto& s : seqs)
      if (!s->finished()) return false;
    return true;
  }
};

// Returns the finish reason after `seq` received its newest token (already appended).
inline FinishReason check_stop(const Sequence& seq, const StoppingParams& sp) {
  const int32_t n_gen = seq.num_generated();
  if (n_gen <= 0) return FinishReason::NONE;
  const int32_t last = seq.tokens.back();
  if (!sp.ignore_eos && sp.eos_token_id >= 0 && last == sp.eos_token_id) return FinishReason::STOP;
  if (!sp.ignore_eos) {
    for (int32_t t : sp.stop_token_ids)
      if (t == last) return FinishReason::STOP;
  }
  for (const auto& ss : sp.stop_sequences) {
    const int32_t k = (int32_t)ss.size();
    if (k == 0 || k > n_gen) continue;
    bool eq = true;
    for (int32_t i = 0; i < k && eq; ++i) eq = seq.tokens[seq.tokens.size() - k + i] == ss[i];
    if (eq) return FinishReason::STOP;
  }
  if (n_gen >= sp.max_tokens) return FinishReason::LENGTH;
  if (sp.max_context_len > 0 && seq.num_tokens() >= sp.max_context_len) return FinishReason::LENGTH;
  return FinishReason::NONE;
}

}  // namespace xllm
