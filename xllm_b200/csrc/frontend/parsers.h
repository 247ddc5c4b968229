// Streaming reasoning and tool-call parsers.
//
// Parity: xllm/parser/reasoning_parser.h + reasoning_detector.* (<think> splitting for qwen3 /
// deepseek-r1 / glm45) and xllm/function_call/* (FunctionCallParser with per-model detectors
// qwen25, qwen3_coder, kimi_k2, deepseekv3, glm45 and utils.cpp partial-JSON handling).  Each
// detector is a small state machine fed with text deltas; it returns what is plain content, what is
// reasoning, and tool-call items whose argument JSON may still be growing.
#pragma once
#include <string>
#include <vector>

#include "json.h"

namespace xllm {

// Close whatever is open in a truncated JSON text so that it parses (strings, arrays, objects;
// a dangling key or ':' is dropped).  Returns false when nothing usable is there yet.
inline bool complete_partial_json(const std::string& in, std::string* out) {
  std::string s;
  std::vector<char> stack;
  bool in_str = false, esc = false;
  size_t last_safe = 0;        // length of `s` after the last complete value / opener
  std::vector<char> safe_stack;
  for (char c : in) {
    s.push_back(c);
    if (in_str) {
      if (esc) esc = false;
      else if (c == '\\') esc = true;
      else if (c == '"') in_str = false;
      continue;
    }
    if (c == '"') in_str = true;
    else if (c == '{' || c == '[') { stack.push_back(c == '{' ? '}' : ']'); }
    else if (c == '}' || c == ']') { if (!stack.empty()) stack.pop_back(); }
    if (c == '{' || c == '[' || c == '}' || c == ']' || c == ',') { last_safe = s.size(); safe_stack = stack; }
  }
  auto close = [](std::string t, const std::vector<char>& st) {
    // strip trailing comma / whitespace before closing
    while (!t.empty() && (t.back() == ',' || t.back() == ' ' || t.back() == '\n' || t.back() == '\t')) t.pop_back();
    for (auto it = st.rbegin(); it != st.rend(); ++it) t.push_back(*it);
    return t;
  };
  Json tmp;
  std::string cand = s;
  if (in_str) { if (esc) cand.pop_back(); cand.push_back('"'); }
  cand = close(cand, stack);
  if (Json::try_parse(cand, &tmp)) { *out = cand; return true; }
  // fall back to the last point where a value had just ended
  cand = close(s.substr(0, last_safe), safe_stack);
  if (!cand.empty() && Json::try_parse(cand, &tmp)) { *out = cand; return true; }
  return false;
}

// ------------------------------------------------------------------------------------------------
struct ReasoningDelta {
  std::string reasoning, content;
};

// Splits "<think> ... </think> answer".  `starts_in_reasoning`: models whose template already
// opened the think block (deepseek-r1, qwen3 with thinking forced on).
class ReasoningParser {
 public:
  explicit ReasoningParser(const std::string& kind = "qwen3", bool starts_in_reasoning = false)
      : open_("<think>"), close_("</think>"), in_(starts_in_reasoning) {
    if (kind == "deepseek-r1" || kind == "deepseek_r1") in_ = true;
  }
  ReasoningDelta push(const std::string& delta) {
    ReasoningDelta out;
    buf_ += delta;
    while (true) {
      const std::string& tag = in_ ? close_ : open_;
      const size_t at = buf_.find(tag);
      if (at != std::string::npos) {
        (in_ ? out.reasoning : out.content) += buf_.substr(0, at);
        buf_.erase(0, at + tag.size());
        if (in_) { // swallow the newlines that follow </think>
          size_t k = 0;
          while (k < buf_.size() && k < 2 && buf_[k] == '\n') ++k;
          buf_.erase(0, k);
        }
        in_ = !in_;
        seen_ = true;
        continue;
      }
      // hold back a possible tag prefix at the end
      size_t hold = 0;
      for (size_t k = std::min(tag.size() - 1, buf_.size()); k > 0; --k)
        if (buf_.compare(buf_.size() - k, k, tag, 0, k) == 0) { hold = k; break; }
      (in_ ? out.reasoning : out.content) += buf_.substr(0, buf_.size() - hold);
      buf_.erase(0, buf_.size() - hold);
      break;
    }
    return out;
  }
  ReasoningDelta flush() {
    ReasoningDelta out;
    (in_ ? out.reasoning : out.content) = buf_;
    buf_.clear();
    return out;
  }

 private:
  std::string open_, close_, buf_;
  bool in_, seen_ = false;
};

// ------------------------------------------------------------------------------------------------
struct ToolCallItem {
  int index = 0;
  std::string name;        // set on the first item of a call
  std::string arguments;   // full argument JSON text (non-streaming) or the newly added piece
};

struct ToolParseResult {
  std::string content;               // text outside tool calls
  std::vector<ToolCallItem> calls;
};

class ToolCallParser {
 public:
  // kind: qwen25 | qwen3 | hermes | qwen3_coder | deepseekv3 | kimi_k2 | glm45 | glm47
  explicit ToolCallParser(const std::string& kind) : kind_(kind) {
    if (kind == "deepseekv3" || kind == "deepseekv32") {
      begin_ = "<｜tool▁call▁begin｜>"; end_ = "<｜tool▁call▁end｜>";
      outer_begin_ = "<｜tool▁calls▁begin｜>"; outer_end_ = "<｜tool▁calls▁end｜>";
    } else if (kind == "kimi_k2") {
      begin_ = "<|tool_call_begin|>"; end_ = "<|tool_call_end|>";
      outer_begin_ = "<|tool_calls_section_begin|>"; outer_end_ = "<|tool_calls_section_end|>";
    } else {
      begin_ = "<tool_call>"; end_ = "</tool_call>";
    }
  }

  bool has_tool_call(const std::string& text) const { return text.find(begin_) != std::string::npos; }

  // Whole-text parse (non-streaming responses).
  ToolParseResult parse(const std::string& text) const {
    ToolParseResult r;
    size_t pos = 0;
    int idx = 0;
    while (true) {
      const size_t b = text.find(begin_, pos);
      if (b == std::string::npos) { r.content += strip_outer(text.substr(pos)); break; }
      r.content += strip_outer(text.substr(pos, b - pos));
      const size_t e = text.find(end_, b + begin_.size());
      const std::string body = text.substr(b + begin_.size(), e == std::string::npos ? std::string::npos : e - b - begin_.size());
      ToolCallItem item;
      if (parse_body(body, &item)) { item.index = idx++; r.calls.push_back(std::move(item)); }
      if (e == std::string::npos) break;
      pos = e + end_.size();
    }
    trim(r.content);
    return r;
  }

  // Streaming: feed deltas; content outside calls is passed through, each call yields its name once
  // and then argument text increments.
  ToolParseResult push(const std::string& delta) {
    ToolParseResult r;
    buf_ += delta;
    while (true) {
      if (!in_call_) {
        const size_t b = buf_.find(begin_);
        if (b != std::string::npos) {
          r.content += strip_outer(buf_.substr(0, b));
          buf_.erase(0, b + begin_.size());
          in_call_ = true;
          sent_name_ = false;
          sent_args_ = 0;
          continue;
        }
        size_t hold = 0;
        for (const std::string* tag : {&begin_, &outer_begin_}) {
          if (tag->empty()) continue;
          for (size_t k = std::min(tag->size() - 1, buf_.size()); k > hold; --k)
            if (buf_.compare(buf_.size() - k, k, *tag, 0, k) == 0) { hold = k; break; }
        }
        r.content += strip_outer(buf_.substr(0, buf_.size() - hold));
        buf_.erase(0, buf_.size() - hold);
        break;
      }
      const size_t e = buf_.find(end_);
      const std::string body = e == std::string::npos ? buf_ : buf_.substr(0, e);
      ToolCallItem full;
      const bool partial = e == std::string::npos;
      if (parse_body(body, &full, partial)) {
        ToolCallItem item;
        item.index = call_index_;
        // the name goes out once it can no longer grow; argument text of the tag-based formats is
        // rebuilt from key/value pairs and is only final when the call closes
        const bool name_done = !partial || name_complete(body);
        if (partial && (kind_ == "qwen3_coder" || kind_ == "glm45" || kind_ == "glm47")) full.arguments.clear();
        if (!sent_name_ && !full.name.empty() && name_done) { item.name = full.name; sent_name_ = true; }
        if (sent_name_ && full.arguments.size() > sent_args_ && (e != std::string::npos || stable_prefix(full.arguments) > sent_args_)) {
          const size_t upto = e != std::string::npos ? full.arguments.size() : stable_prefix(full.arguments);
          item.arguments = full.arguments.substr(sent_args_, upto - sent_args_);
          sent_args_ = upto;
        }
        if (!item.name.empty() || !item.arguments.empty()) r.calls.push_back(std::move(item));
      }
      if (e == std::string::npos) break;
      buf_.erase(0, e + end_.size());
      in_call_ = false;
      ++call_index_;
    }
    return r;
  }

 private:
  static void trim(std::string& s) {
    while (!s.empty() && (s.back() == '\n' || s.back() == ' ')) s.pop_back();
    size_t k = 0;
    while (k < s.size() && (s[k] == '\n' || s[k] == ' ')) ++k;
    s.erase(0, k);
  }
  std::string strip_outer(std::string s) const {
    for (const std::string* tag : {&outer_begin_, &outer_end_}) {
      if (tag->empty()) continue;
      size_t at;
      while ((at = s.find(*tag)) != std::string::npos) s.erase(at, tag->size());
    }
    return s;
  }
  // A partial argument string is only streamed up to the point that cannot change any more:
  // completing partial JSON appends closers, so drop trailing closers / quotes.
  static size_t stable_prefix(const std::string& args) {
    size_t n = args.size();
    while (n > 0 && (args[n - 1] == '}' || args[n - 1] == ']' || args[n - 1] == '"')) --n;
    return n;
  }

  bool name_complete(const std::string& body) const {
    if (kind_ == "qwen3_coder") { const size_t f = body.find("<function="); return f != std::string::npos && body.find('>', f) != std::string::npos; }
    if (kind_ == "glm45" || kind_ == "glm47") return body.find('\n') != std::string::npos || body.find("<arg_key>") != std::string::npos;
    if (kind_ == "deepseekv3" || kind_ == "deepseekv32") { const size_t s = body.find("<｜tool▁sep｜>"); return s != std::string::npos && body.find('\n', s) != std::string::npos; }
    if (kind_ == "kimi_k2") return body.find("<|tool_call_argument_begin|>") != std::string::npos;
    return body.find("\"arguments\"") != std::string::npos || body.find("\"parameters\"") != std::string::npos;
  }

  bool parse_body(const std::string& body_in, ToolCallItem* out, bool partial = false) const {
    std::string body = body_in;
    trim(body);
    if (kind_ == "qwen3_coder") return parse_xml_function(body, out);
    if (kind_ == "glm45" || kind_ == "glm47") return parse_glm(body, out);
    if (kind_ == "deepseekv3" || kind_ == "deepseekv32") {
      // function<｜tool▁sep｜>NAME\n```json\n{...}\n```
      const std::string sep = "<｜tool▁sep｜>";
      const size_t s = body.find(sep);
      if (s == std::string::npos) return false;
      std::string rest = body.substr(s + sep.size());
      const size_t nl = rest.find('\n');
      out->name = rest.substr(0, nl);
      trim(out->name);
      if (nl == std::string::npos) return !out->name.empty();
      std::string args = rest.substr(nl + 1);
      const size_t f = args.find("```json");
      if (f != std::string::npos) args.erase(0, f + 7);
      const size_t f2 = args.rfind("```");
      if (f2 != std::string::npos && !partial) args.erase(f2);
      trim(args);
      return finish_args(args, out, partial);
    }
    if (kind_ == "kimi_k2") {
      // functions.NAME:IDX<|tool_call_argument_begin|>{...}
      const std::string sep = "<|tool_call_argument_begin|>";
      const size_t s = body.find(sep);
      std::string head = body.substr(0, s);
      trim(head);
      const size_t dot = head.find('.');
      const size_t colon = head.rfind(':');
      out->name = head.substr(dot == std::string::npos ? 0 : dot + 1,
                              colon == std::string::npos ? std::string::npos : colon - (dot == std::string::npos ? 0 : dot + 1));
      if (s == std::string::npos) return false;
      std::string args = body.substr(s + sep.size());
      trim(args);
      return finish_args(args, out, partial);
    }
    // qwen25 / hermes: {"name": ..., "arguments": {...}}
    std::string fixed = body;
    if (partial && !complete_partial_json(body, &fixed)) return false;
    Json j;
    if (!Json::try_parse(fixed, &j) || !j.is_object()) return false;
    out->name = j["name"].as_string();
    const Json& a = j.contains("arguments") ? j["arguments"] : j["parameters"];
    out->arguments = a.is_null() ? std::string(partial ? "" : "{}") : (a.is_string() ? a.as_string() : a.dump());
    return !out->name.empty();
  }
  static bool finish_args(const std::string& args, ToolCallItem* out, bool partial) {
    if (!partial) { out->arguments = args; return !out->name.empty(); }
    std::string fixed;
    out->arguments = complete_partial_json(args, &fixed) ? fixed : std::string();
    return !out->name.empty();
  }
  // <function=NAME>\n<parameter=KEY>\nVALUE\n</parameter>...</function>
  static bool parse_xml_function(const std::string& body, ToolCallItem* out) {
    const size_t f = body.find("<function=");
    if (f == std::string::npos) return false;
    const size_t fe = body.find('>', f);
    if (fe == std::string::npos) return false;
    out->name = body.substr(f + 10, fe - f - 10);
    Json args = Json::object();
    size_t pos = fe;
    while (true) {
      const size_t p = body.find("<parameter=", pos);
      if (p == std::string::npos) break;
      const size_t pe = body.find('>', p);
      if (pe == std::string::npos) break;
      const std::string key = body.substr(p + 11, pe - p - 11);
      const size_t ve = body.find("</parameter>", pe);
      std::string val = body.substr(pe + 1, ve == std::string::npos ? std::string::npos : ve - pe - 1);
      trim(val);
      Json parsed;
      if (Json::try_parse(val, &parsed) && !parsed.is_string()) args.set(key, parsed);
      else args.set(key, val);
      if (ve == std::string::npos) break;
      pos = ve + 12;
    }
    out->arguments = args.dump();
    return !out->name.empty();
  }
  // NAME\n<arg_key>K</arg_key>\n<arg_value>V</arg_value>...
  static bool parse_glm(const std::string& body, ToolCallItem* out) {
    const size_t nl = body.find('\n');
    const size_t ak = body.find("<arg_key>");
    out->name = body.substr(0, std::min(nl, ak));
    trim(out->name);
    Json args = Json::object();
    size_t pos = 0;
    while (true) {
      const size_t k = body.find("<arg_key>", pos);
      if (k == std::string::npos) break;
      const size_t ke = body.find("</arg_key>", k);
      const size_t v = body.find("<arg_value>", ke);
      const size_t ve = body.find("</arg_value>", v);
      if (ke == std::string::npos || v == std::string::npos || ve == std::string::npos) break;
      const std::string key = body.substr(k + 9, ke - k - 9);
      const std::string val = body.substr(v + 11, ve - v - 11);
      Json parsed;
      if (Json::try_parse(val, &parsed) && !parsed.is_string()) args.set(key, parsed);
      else args.set(key, val);
      pos = ve + 12;
    }
    out->arguments = args.dump();
    return !out->name.empty();
  }

  std::string kind_, begin_, end_, outer_begin_, outer_end_, buf_;
  bool in_call_ = false, sent_name_ = false;
  size_t sent_args_ = 0;
  int call_index_ = 0;
};

}  // namespace xllm
