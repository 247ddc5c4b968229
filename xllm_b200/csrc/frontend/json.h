// Minimal JSON value, parser and serialiser for the C++ front end (config files, tokenizer.json,
// safetensors headers, OpenAI request/response bodies, partial-JSON repair for streamed tool calls).
// The reference relies on nlohmann::json and brpc's json2pb; neither is available here.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace xllm {

class Json {
 public:
  enum Type { NUL, BOOL, INT, DOUBLE, STRING, ARRAY, OBJECT };
  using Array = std::vector<Json>;
  using Object = std::vector<std::pair<std::string, Json>>;  // insertion order is kept

  Json() : type_(NUL) {}
  Json(std::nullptr_t) : type_(NUL) {}
  Json(bool b) : type_(BOOL), b_(b) {}
  Json(int v) : type_(INT), i_(v) {}
  Json(int64_t v) : type_(INT), i_(v) {}
  Json(uint64_t v) : type_(INT), i_((int64_t)v) {}
  Json(double v) : type_(DOUBLE), d_(v) {}
  Json(const char* s) : type_(STRING), s_(s) {}
  Json(std::string s) : type_(STRING), s_(std::move(s)) {}
  static Json array() { Json j; j.type_ = ARRAY; return j; }
  static Json object() { Json j; j.type_ = OBJECT; return j; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == NUL; }
  bool is_bool() const { return type_ == BOOL; }
  bool is_number() const { return type_ == INT || type_ == DOUBLE; }
  bool is_int() const { return type_ == INT; }
  bool is_string() const { return type_ == STRING; }
  bool is_array() const { return type_ == ARRAY; }
  bool is_object() const { return type_ == OBJECT; }

  bool as_bool(bool def = false) const { return type_ == BOOL ? b_ : (type_ == INT ? i_ != 0 : def); }
  int64_t as_int(int64_t def = 0) const { return type_ == INT ? i_ : (type_ == DOUBLE ? (int64_t)d_ : (type_ == BOOL ? b_ : def)); }
  double as_double(double def = 0) const { return type_ == DOUBLE ? d_ : (type_ == INT ? (double)i_ : def); }
  const std::string& as_string() const { static const std::string e; return type_ == STRING ? s_ : e; }
  const Array& items() const { static const Array e; return type_ == ARRAY ? a_ : e; }
  Array& items() { if (type_ != ARRAY) { type_ = ARRAY; } return a_; }
  const Object& members() const { static const Object e; return type_ == OBJECT ? o_ : e; }

  size_t size() const { return type_ == ARRAY ? a_.size() : (type_ == OBJECT ? o_.size() : 0); }
  void push_back(Json v) { if (type_ != ARRAY) type_ = ARRAY; a_.push_back(std::move(v)); }
  const Json& at(size_t i) const { static const Json n; return (type_ == ARRAY && i < a_.size()) ? a_[i] : n; }
  const Json& operator[](size_t i) const { return at(i); }
  const Json& operator[](int i) const { return at((size_t)i); }

  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json* find(const std::string& k) const {
    if (type_ != OBJECT) return nullptr;
    for (auto& kv : o_) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const Json& operator[](const std::string& k) const { static const Json n; const Json* p = find(k); return p ? *p : n; }
  const Json& operator[](const char* k) const { return (*this)[std::string(k)]; }
  Json& set(const std::string& k, Json v) {
    if (type_ != OBJECT) type_ = OBJECT;
    for (auto& kv : o_) if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    o_.emplace_back(k, std::move(v));
    return o_.back().second;
  }

  // ---------------------------------------------------------------- serialise
  std::string dump(int indent = -1) const { std::string out; dump_to(out, indent, 0); return out; }

  static void escape_to(std::string& out, const std::string& s) {
    out.push_back('"');
    for (unsigned char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default:
          if (c < 0x20) { char buf[8]; snprintf(buf, sizeof(buf), "\\u%04x", c); out += buf; }
          else out.push_back((char)c);
      }
    }
    out.push_back('"');
  }

  // ---------------------------------------------------------------- parse
  // Throws std::runtime_error on malformed input (message carries the byte offset).
  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json v = parse_value(text, pos, 0);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::runtime_error("json: trailing characters at " + std::to_string(pos));
    return v;
  }
  static bool try_parse(const std::string& text, Json* out) {
    try { *out = parse(text); return true; } catch (const std::exception&) { return false; }
  }

 private:
  void dump_to(std::string& out, int indent, int depth) const {
    auto nl = [&](int d) { if (indent >= 0) { out.push_back('\n'); out.append((size_t)(indent * d), ' '); } };
    switch (type_) {
      case NUL: out += "null"; break;
      case BOOL: out += b_ ? "true" : "false"; break;
      case INT: out += std::to_string(i_); break;
      case DOUBLE: {
        if (!std::isfinite(d_)) { out += "null"; break; }
        char buf[40];
        snprintf(buf, sizeof(buf), "%.17g", d_);
        double back = 0; sscanf(buf, "%lf", &back);
        for (int p = 1; p < 17; ++p) { char b2[40]; snprintf(b2, sizeof(b2), "%.*g", p, d_); sscanf(b2, "%lf", &back); if (back == d_) { snprintf(buf, sizeof(buf), "%s", b2); break; } }
        out += buf;
        if (std::string(buf).find_first_of(".eE") == std::string::npos) out += ".0";
        break;
      }
      case STRING: escape_to(out, s_); break;
      case ARRAY:
        out.push_back('[');
        for (size_t i = 0; i < a_.size(); ++i) { if (i) out.push_back(','); nl(depth + 1); a_[i].dump_to(out, indent, depth + 1); }
        if (!a_.empty()) nl(depth);
        out.push_back(']');
        break;
      case OBJECT:
        out.push_back('{');
        for (size_t i = 0; i < o_.size(); ++i) {
          if (i) out.push_back(',');
          nl(depth + 1);
          escape_to(out, o_[i].first);
          out += indent >= 0 ? ": " : ":";
          o_[i].second.dump_to(out, indent, depth + 1);
        }
        if (!o_.empty()) nl(depth);
        out.push_back('}');
        break;
    }
  }

  static void skip_ws(const std::string& t, size_t& p) {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\r' || t[p] == '\t')) ++p;
  }
  static void append_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) s.push_back((char)cp);
    else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  }
  static uint32_t hex4(const std::string& t, size_t p) {
    if (p + 4 > t.size()) throw std::runtime_error("json: bad \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = t[p + i];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else throw std::runtime_error("json: bad \\u escape");
    }
    return v;
  }
  static std::string parse_string(const std::string& t, size_t& p) {
    std::string s;
    ++p;  // opening quote
    while (true) {
      if (p >= t.size()) throw std::runtime_error("json: unterminated string");
      char c = t[p++];
      if (c == '"') break;
      if (c != '\\') { s.push_back(c); continue; }
      if (p >= t.size()) throw std::runtime_error("json: unterminated escape");
      char e = t[p++];
      switch (e) {
        case 'n': s.push_back('\n'); break;
        case 't': s.push_back('\t'); break;
        case 'r': s.push_back('\r'); break;
        case 'b': s.push_back('\b'); break;
        case 'f': s.push_back('\f'); break;
        case 'u': {
          uint32_t cp = hex4(t, p); p += 4;
          if (cp >= 0xD800 && cp <= 0xDBFF && p + 6 <= t.size() && t[p] == '\\' && t[p + 1] == 'u') {
            uint32_t lo = hex4(t, p + 2);
            if (lo >= 0xDC00 && lo <= 0xDFFF) { cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00); p += 6; }
          }
          append_utf8(s, cp);
          break;
        }
        default: s.push_back(e);
      }
    }
    return s;
  }
  static Json parse_value(const std::string& t, size_t& p, int depth) {
    if (depth > 256) throw std::runtime_error("json: nesting too deep");
    skip_ws(t, p);
    if (p >= t.size()) throw std::runtime_error("json: unexpected end");
    char c = t[p];
    if (c == '{') {
      Json o = object();
      ++p; skip_ws(t, p);
      if (p < t.size() && t[p] == '}') { ++p; return o; }
      while (true) {
        skip_ws(t, p);
        if (p >= t.size() || t[p] != '"') throw std::runtime_error("json: expected key at " + std::to_string(p));
        std::string k = parse_string(t, p);
        skip_ws(t, p);
        if (p >= t.size() || t[p] != ':') throw std::runtime_error("json: expected ':' at " + std::to_string(p));
        ++p;
        o.o_.emplace_back(std::move(k), parse_value(t, p, depth + 1));
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == '}') { ++p; break; }
        throw std::runtime_error("json: expected ',' or '}' at " + std::to_string(p));
      }
      return o;
    }
    if (c == '[') {
      Json a = array();
      ++p; skip_ws(t, p);
      if (p < t.size() && t[p] == ']') { ++p; return a; }
      while (true) {
        a.a_.push_back(parse_value(t, p, depth + 1));
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == ']') { ++p; break; }
        throw std::runtime_error("json: expected ',' or ']' at " + std::to_string(p));
      }
      return a;
    }
    if (c == '"') return Json(parse_string(t, p));
    if (t.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (t.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (t.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    // number
    size_t s = p;
    bool is_double = false;
    if (p < t.size() && (t[p] == '-' || t[p] == '+')) ++p;
    while (p < t.size() && ((t[p] >= '0' && t[p] <= '9') || t[p] == '.' || t[p] == 'e' || t[p] == 'E' || t[p] == '-' || t[p] == '+')) {
      if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_double = true;
      ++p;
    }
    if (p == s) throw std::runtime_error("json: unexpected character at " + std::to_string(p));
    const std::string num = t.substr(s, p - s);
    try {
      if (!is_double) return Json((int64_t)std::stoll(num));
    } catch (const std::exception&) {
    }
    try {
      return Json(std::stod(num));
    } catch (const std::exception&) {
      throw std::runtime_error("json: bad number at " + std::to_string(s));
    }
  }

  Type type_;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  Array a_;
  Object o_;
};

}  // namespace xllm
