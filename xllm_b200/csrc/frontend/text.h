// Text-side request processing: incremental detokenisation with stop-string hold-back, chat
// templates, reasoning ("thinking") splitting and tool-call extraction, all usable on streams.
//
// Parity: IncrementalDecoder + StoppingChecker string stops (xllm/core/framework/request/
// incremental_decoder.cpp, stopping_checker.cpp), native chat templates + the Jinja path
// (xllm/core/framework/chat_template/*), reasoning detectors (xllm/parser/reasoning_parser.h) and
// the tool-call detectors qwen25 / qwen3_coder / deepseek v3 / kimi_k2 / glm45
// (xllm/function_call/*_detector.cpp, function_call_parser.h) with their partial-JSON handling.
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "json.h"
#include "tokenizer.h"

namespace xllm {

// ------------------------------------------------------------------------------------------------
// Emits text as tokens arrive.  Bytes of an unfinished UTF-8 sequence and text that could still
// turn into a stop string are held back.
class IncrementalDecoder {
 public:
  IncrementalDecoder(const Tokenizer* tok, std::vector<std::string> stops, bool skip_special)
      : tok_(tok), stops_(std::move(stops)), skip_special_(skip_special) {
    for (auto& s : stops_) max_stop_ = std::max(max_stop_, s.size());
  }

  // Returns newly releasable text; sets `stopped` when a stop string completed (the stop string
  // itself and everything after it is dropped).
  std::string push(int32_t token, bool* stopped) {
    *stopped = false;
    if (stopped_) { *stopped = true; return std::string(); }
    ids_.push_back(token);
    // decode a short tail so that multi-token characters come out right
    const size_t from = ids_.size() > 6 ? ids_.size() - 6 : 0;
    std::vector<int32_t> tail(ids_.begin() + from, ids_.end());
    std::vector<int32_t> prev(ids_.begin() + from, ids_.end() - 1);
    const std::string full = tok_->decode(tail, skip_special_);
    const std::string before = tok_->decode(prev, skip_special_);
    std::string delta;
    if (full.size() >= before.size() && full.compare(0, before.size(), before) == 0) delta = full.substr(before.size());
    else delta = full.substr(std::min(common_prefix(full, before), full.size()));
    pending_ += delta;
    // hold back an incomplete UTF-8 tail
    size_t safe = pending_.size();
    for (size_t back = 1; back <= 3 && back <= pending_.size(); ++back) {
      const unsigned char c = (unsigned char)pending_[pending_.size() - back];
      if ((c & 0xC0) == 0x80) continue;
      const size_t need = c >= 0xF0 ? 4 : (c >= 0xE0 ? 3 : (c >= 0xC0 ? 2 : 1));
      if (need > back) safe = pending_.size() - back;
      break;
    }
    // stop strings
    for (auto& s : stops_) {
      const size_t at = pending_.find(s);
      if (at != std::string::npos) {
        std::string out = pending_.substr(0, at);
        pending_.clear();
        stopped_ = true;
        *stopped = true;
        emitted_ += out;
        return out;
      }
    }
    size_t hold = 0;
    for (auto& s : stops_) {
      const size_t maxk = std::min(s.size() - 1, safe);
      for (size_t k = maxk; k > hold; --k)
        if (pending_.compare(safe - k, k, s, 0, k) == 0) { hold = k; break; }
    }
    const size_t release = safe - hold;
    std::string out = pending_.substr(0, release);
    pending_.erase(0, release);
    emitted_ += out;
    return out;
  }

  // Remaining held-back text at end of generation.
  std::string flush() {
    std::string out;
    if (!stopped_) out.swap(pending_);
    emitted_ += out;
    return out;
  }
  const std::string& text() const { return emitted_; }

 private:
  static size_t common_prefix(const std::string& a, const std::string& b) {
    size_t i = 0;
    while (i < a.size() && i < b.size() && a[i] == b[i]) ++i;
    return i;
  }
  const Tokenizer* tok_;
  std::vector<std::string> stops_;
  bool skip_special_;
  size_t max_stop_ = 0;
  std::vector<int32_t> ids_;
  std::string pending_, emitted_;
  bool stopped_ = false;
};

// ------------------------------------------------------------------------------------------------
struct ChatMessage {
  std::string role, content;
  std::string tool_calls_json;   // assistant messages that called tools (JSON array text)
  std::string tool_call_id;      // tool results
};

// Native chat templates for the families the engine ships models for.  Arbitrary Jinja templates
// from tokenizer_config.json are rendered by the Python front end (jinja2); this class covers the
// common cases without leaving C++.
class ChatTemplate {
 public:
  explicit ChatTemplate(std::string family) : family_(std::move(family)) {}

  static std::string detect_family(const std::string& model_type, const std::string& template_text) {
    if (template_text.find("<|im_start|>") != std::string::npos) return "chatml";
    if (template_text.find("<|start_header_id|>") != std::string::npos) return "llama3";
    if (template_text.find("<｜User｜>") != std::string::npos) return "deepseek";
    if (template_text.find("[gMASK]") != std::string::npos || template_text.find("<|user|>") != std::string::npos) return "glm";
    if (model_type.rfind("qwen", 0) == 0) return "chatml";
    if (model_type.rfind("llama", 0) == 0) return "llama3";
    if (model_type.rfind("deepseek", 0) == 0) return "deepseek";
    if (model_type.rfind("glm", 0) == 0) return "glm";
    return "chatml";
  }

  std::string apply(const std::vector<ChatMessage>& msgs, const std::string& tools_json, bool add_generation_prompt,
                    bool enable_thinking) const {
    if (family_ == "llama3") return llama3(msgs, add_generation_prompt);
    if (family_ == "deepseek") return deepseek(msgs, add_generation_prompt);
    if (family_ == "glm") return glm(msgs, add_generation_prompt);
    return chatml(msgs, tools_json, add_generation_prompt, enable_thinking);
  }

 private:
  static std::string chatml(const std::vector<ChatMessage>& msgs, const std::string& tools_json, bool gen,
                            bool enable_thinking) {
    std::string out;
    size_t start = 0;
    const bool has_tools = !tools_json.empty() && tools_json != "[]" && tools_json != "null";
    if (has_tools) {
      out += "<|im_start|>system\n";
      if (!msgs.empty() && msgs[0].role == "system") { out += msgs[0].content + "\n\n"; start = 1; }
      out += "# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
             "You are provided with function signatures within <tools></tools> XML tags:\n<tools>";
      Json tools;
      if (Json::try_parse(tools_json, &tools))
        for (auto& t : tools.items()) out += "\n" + t.dump();
      out += "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
             "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": "
             "<args-json-object>}\n</tool_call><|im_end|>\n";
    } else if (!msgs.empty() && msgs[0].role == "system") {
      out += "<|im_start|>system\n" + msgs[0].content + "<|im_end|>\n";
      start = 1;
    }
    for (size_t i = start; i < msgs.size(); ++i) {
      const ChatMessage& m = msgs[i];
      if (m.role == "tool") {
        const bool first = i == 0 || msgs[i - 1].role != "tool";
        const bool last = i + 1 == msgs.size() || msgs[i + 1].role != "tool";
        if (first) out += "<|im_start|>user";
        out += "\n<tool_response>\n" + m.content + "\n</tool_response>";
        if (last) out += "<|im_end|>\n";
        continue;
      }
      out += "<|im_start|>" + m.role + "\n" + m.content;
      if (m.role == "assistant" && !m.tool_calls_json.empty()) {
        Json calls;
        if (Json::try_parse(m.tool_calls_json, &calls)) {
          for (auto& c : calls.items()) {
            const Json& fn = c.contains("function") ? c["function"] : c;
            std::string args = fn["arguments"].is_string() ? fn["arguments"].as_string() : fn["arguments"].dump();
            out += "\n<tool_call>\n{\"name\": \"" + fn["name"].as_string() + "\", \"arguments\": " + args + "}\n</tool_call>";
          }
        }
      }
      out += "<|im_end|>\n";
    }
    if (gen) {
      out += "<|im_start|>assistant\n";
      if (!enable_thinking) out += "<think>\n\n</think>\n\n";
    }
    return out;
  }
  static std::string llama3(const std::vector<ChatMessage>& msgs, bool gen) {
    std::string out = "<|begin_of_text|>";
    for (auto& m : msgs)
      out += "<|start_header_id|>" + m.role + "<|end_header_id|>\n\n" + m.content + "<|eot_id|>";
    if (gen) out += "<|start_header_id|>assistant<|end_header_id|>\n\n";
    return out;
  }
  static std::string deepseek(const std::vector<ChatMessage>& msgs, bool gen) {
    std::string out = "<｜begin▁of▁sentence｜>";
    for (auto& m : msgs) {
      if (m.role == "system") out += m.content;
      else if (m.role == "user") out += "<｜User｜>" + m.content;
      else if (m.role == "assistant") out += "<｜Assistant｜>" + m.content + "<｜end▁of▁sentence｜>";
      else if (m.role == "tool") out += "<｜tool▁outputs▁begin｜><｜tool▁output▁begin｜>" + m.content + "<｜tool▁output▁end｜><｜tool▁outputs▁end｜>";
    }
    if (gen) out += "<｜Assistant｜>";
    return out;
  }
  static std::string glm(const std::vector<ChatMessage>& msgs, bool gen) {
    std::string out = "[gMASK]<sop>";
    for (auto& m : msgs) out += "<|" + (m.role == "tool" ? std::string("observation") : m.role) + "|>\n" + m.content;
    if (gen) out += "<|assistant|>\n";
    return out;
  }
  std::string family_;
};

}  // namespace xllm
