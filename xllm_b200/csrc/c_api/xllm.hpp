// C++ interface of the engine: a thin, header-only class over the C API (xllm.h).
//
// Counterpart of the reference's C++ wrapper (xllm/cc_api/llm.h: `LLM::Initialize`,
// `Completions`, `ChatCompletions`): the host program owns an `xllm_b200::LLM`, results come back
// as JSON text (the same documents the HTTP routes produce).  Errors are exceptions carrying the
// engine's message.
//
//   xllm_b200::LLM llm;
//   llm.Initialize("/models/qwen3-8b", R"({"devices": "cuda:0", "max_seqs_per_batch": 64})");
//   std::string out = llm.Completions("[\"Hello\"]", R"({"max_tokens": 32})");
#pragma once

#include <stdexcept>
#include <string>

#include "xllm.h"

namespace xllm_b200 {

class LLM {
 public:
  LLM() = default;
  ~LLM() { Shutdown(); }
  LLM(const LLM&) = delete;
  LLM& operator=(const LLM&) = delete;

  // Loads the model and builds the engine; options_json = keyword arguments of the Python `LLM`.
  bool Initialize(const std::string& model_path, const std::string& options_json = "{}") {
    Shutdown();
    handle_ = xllm_llm_create(model_path.c_str(), options_json.c_str());
    return handle_ != nullptr;
  }
  bool initialized() const { return handle_ != nullptr; }
  static std::string LastError() { return xllm_last_error(); }

  // prompts_json: a JSON array of strings or token-id arrays; returns a JSON array of results.
  std::string Completions(const std::string& prompts_json, const std::string& sampling_json = "{}") {
    return take(xllm_llm_generate(need(), prompts_json.c_str(), sampling_json.c_str()));
  }
  // messages_json: [{"role": "user", "content": "..."}, ...]
  std::string ChatCompletions(const std::string& messages_json, const std::string& sampling_json = "{}") {
    return Call("chat", "{\"messages\": " + messages_json + ", \"sampling\": " + sampling_json + "}");
  }
  std::string Embeddings(const std::string& prompts_json) { return Call("embed", "{\"prompts\": " + prompts_json + "}"); }
  // Generative recommendation: histories (JSON list of token-id lists) -> per history the best items with scores.
  std::string Recommend(const std::string& histories_json, int beam_width = 32, int num_steps = 3) {
    return Call("recommend", "{\"prompts\": " + histories_json + ", \"beam_width\": " + std::to_string(beam_width) +
                                 ", \"num_steps\": " + std::to_string(num_steps) + "}");
  }
  std::string Stats() { return take(xllm_llm_stats(need())); }
  void Sleep(int level = 1) { Call("sleep", "{\"level\": " + std::to_string(level) + "}"); }
  void WakeUp() { Call("wake_up", "{}"); }
  std::string Call(const std::string& method, const std::string& args_json) {
    return take(xllm_llm_call(need(), method.c_str(), args_json.c_str()));
  }
  void Shutdown() {
    if (handle_ != nullptr) xllm_llm_destroy(handle_);
    handle_ = nullptr;
  }

 private:
  xllm_llm* need() {
    if (handle_ == nullptr) throw std::runtime_error("xllm_b200::LLM is not initialized");
    return handle_;
  }
  static std::string take(char* s) {
    if (s == nullptr) throw std::runtime_error(xllm_last_error());
    std::string out(s);
    xllm_free_string(s);
    return out;
  }
  xllm_llm* handle_ = nullptr;
};

}  // namespace xllm_b200
