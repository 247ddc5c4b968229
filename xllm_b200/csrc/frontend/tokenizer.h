// Byte-level BPE tokenizer reading HuggingFace `tokenizer.json`, plus tiktoken-format vocabularies.
//
// The reference wraps the Rust `tokenizers` crate (xllm/core/framework/tokenizer/tokenizers/src/lib.rs,
// fast_tokenizer.cpp) and has separate tiktoken / sentencepiece classes behind one `Tokenizer`
// interface (tokenizer.h, tokenizer_factory.cpp).  This is a from-scratch C++ implementation of the
// subset LLM serving needs: added/special tokens, the GPT-2 byte<->unicode alphabet, a hand-written
// scanner for the GPT-4 / Qwen pre-tokenisation pattern, rank-ordered BPE merges, exact decode.
#pragma once
#include <algorithm>
#include <climits>
#include <cstdint>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "json.h"

namespace xllm {

namespace utf8 {
inline uint32_t decode(const std::string& s, size_t& i) {
  const unsigned char c = (unsigned char)s[i];
  if (c < 0x80) { i += 1; return c; }
  auto cont = [&](size_t k) { return k < s.size() ? ((unsigned char)s[k] & 0x3F) : 0u; };
  if ((c >> 5) == 0x6) { uint32_t v = ((c & 0x1F) << 6) | cont(i + 1); i += 2; return v; }
  if ((c >> 4) == 0xE) { uint32_t v = ((c & 0x0F) << 12) | (cont(i + 1) << 6) | cont(i + 2); i += 3; return v; }
  if ((c >> 3) == 0x1E) { uint32_t v = ((c & 0x07) << 18) | (cont(i + 1) << 12) | (cont(i + 2) << 6) | cont(i + 3); i += 4; return v; }
  i += 1;
  return 0xFFFD;
}
inline void append(std::string& s, uint32_t cp) {
  if (cp < 0x80) s.push_back((char)cp);
  else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
}
// Coarse Unicode classes: enough for pre-tokenisation boundaries.
inline bool is_space(uint32_t c) {
  return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
         c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
inline bool is_digit(uint32_t c) {
  return (c >= '0' && c <= '9') || (c >= 0x0660 && c <= 0x0669) || (c >= 0x06F0 && c <= 0x06F9) ||
         (c >= 0x0966 && c <= 0x096F) || (c >= 0xFF10 && c <= 0xFF19) || c == 0xB2 || c == 0xB3 || c == 0xB9 ||
         (c >= 0xBC && c <= 0xBE);
}
inline bool is_punct_or_symbol(uint32_t c) {
  if (c < 0x80) return (c >= 33 && c <= 47) || (c >= 58 && c <= 64) || (c >= 91 && c <= 96) || (c >= 123 && c <= 126);
  return (c >= 0xA1 && c <= 0xBF && c != 0xAA && c != 0xB5 && c != 0xBA && !is_digit(c)) || c == 0xD7 || c == 0xF7 ||
         (c >= 0x2010 && c <= 0x2027) || (c >= 0x2030 && c <= 0x205E) || (c >= 0x20A0 && c <= 0x20CF) ||
         (c >= 0x2190 && c <= 0x2BFF) || (c >= 0x3001 && c <= 0x3003) || (c >= 0x3008 && c <= 0x3011) ||
         (c >= 0x3014 && c <= 0x301F) || (c >= 0xFE50 && c <= 0xFE6B) || (c >= 0xFF01 && c <= 0xFF0F) ||
         (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) || (c >= 0xFF5B && c <= 0xFF65) ||
         (c >= 0x1F000 && c <= 0x1FAFF);
}
inline bool is_letter(uint32_t c) {
  if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
  return !is_space(c) && !is_digit(c) && !is_punct_or_symbol(c) && c != 0xFFFD && !(c < 0xA0);
}
}  // namespace utf8

class Tokenizer {
 public:
  virtual ~Tokenizer() = default;
  virtual std::vector<int32_t> encode(const std::string& text, bool add_special = false) const = 0;
  virtual std::string decode(const std::vector<int32_t>& ids, bool skip_special = true) const = 0;
  virtual int32_t vocab_size() const = 0;
  virtual int32_t token_to_id(const std::string& tok) const = 0;
  virtual std::string id_to_token(int32_t id) const = 0;
};

class BpeTokenizer : public Tokenizer {
 public:
  // ---- loading ---------------------------------------------------------------------------
  static std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
  }

  void load_hf_json(const std::string& json_text) {
    Json j = Json::parse(json_text);
    const Json& model = j["model"];
    if (model["type"].as_string() != "BPE" && !model["vocab"].is_object())
      throw std::runtime_error("tokenizer.json: only BPE models are supported");
    init_byte_alphabet();
    for (auto& kv : model["vocab"].members()) add_token(kv.first, (int32_t)kv.second.as_int(), false);
    int32_t rank = 0;
    for (auto& m : model["merges"].items()) {
      std::string a, b;
      if (m.is_string()) {
        const std::string& s = m.as_string();
        const size_t sp = s.find(' ');
        if (sp == std::string::npos) continue;
        a = s.substr(0, sp);
        b = s.substr(sp + 1);
      } else {
        a = m[0].as_string();
        b = m[1].as_string();
      }
      merges_.emplace(a + "\x01" + b, rank++);
    }
    for (auto& t : j["added_tokens"].items())
      add_token(t["content"].as_string(), (int32_t)t["id"].as_int(), true, t["special"].as_bool(false));
    // GPT-2 style pattern (contractions / letters / single or grouped digits) is chosen from the
    // pre_tokenizer description: Qwen / GPT-4 split digits one by one, GPT-2 keeps runs
    const std::string pre = j["pre_tokenizer"].dump();
    single_digits_ = pre.find("\\\\p{N}+") == std::string::npos && pre.find("\\\\p{N}{1,3}") == std::string::npos;
    digits_upto3_ = pre.find("\\\\p{N}{1,3}") != std::string::npos;
    finalize();
  }

  // tiktoken file: one "<base64 token bytes> <rank>" per line; specials given separately
  void load_tiktoken(const std::string& text, const std::vector<std::pair<std::string, int32_t>>& specials) {
    init_byte_alphabet();
    std::istringstream in(text);
    std::string line;
    while (std::getline(in, line)) {
      const size_t sp = line.find(' ');
      if (sp == std::string::npos) continue;
      const std::string bytes = base64_decode(line.substr(0, sp));
      const int32_t id = (int32_t)std::stol(line.substr(sp + 1));
      add_token(bytes_to_alphabet(bytes), id, false);
    }
    rank_is_id_ = true;  // merge priority of a pair = id of the merged token
    for (auto& s : specials) add_token(s.first, s.second, true, true);
    single_digits_ = false;
    digits_upto3_ = true;
    finalize();
  }

  void set_bos_eos(int32_t bos, int32_t eos) { bos_ = bos; eos_ = eos; }

  // ---- interface -------------------------------------------------------------------------
  int32_t vocab_size() const override { return (int32_t)id_to_tok_.size(); }
  int32_t token_to_id(const std::string& t) const override {
    auto it = tok_to_id_.find(t);
    return it == tok_to_id_.end() ? -1 : it->second;
  }
  std::string id_to_token(int32_t id) const override {
    return id >= 0 && id < (int32_t)id_to_tok_.size() ? id_to_tok_[id] : std::string();
  }
  bool is_special(int32_t id) const { return id >= 0 && id < (int32_t)special_.size() && special_[id]; }

  std::vector<int32_t> encode(const std::string& text, bool add_special = false) const override {
    std::vector<int32_t> out;
    if (add_special && bos_ >= 0) out.push_back(bos_);
    // split on added tokens first (longest match at each position)
    size_t i = 0, seg = 0;
    while (i < text.size()) {
      int32_t hit = -1;
      size_t hit_len = 0;
      auto range = added_by_first_.find((unsigned char)text[i]);
      if (range != added_by_first_.end()) {
        for (int32_t idx : range->second) {
          const std::string& a = added_[idx].first;
          if (a.size() > hit_len && text.compare(i, a.size(), a) == 0) { hit = added_[idx].second; hit_len = a.size(); }
        }
      }
      if (hit >= 0) {
        if (i > seg) encode_plain(text.substr(seg, i - seg), out);
        out.push_back(hit);
        i += hit_len;
        seg = i;
      } else {
        ++i;
      }
    }
    if (seg < text.size()) encode_plain(text.substr(seg), out);
    return out;
  }

  std::string decode(const std::vector<int32_t>& ids, bool skip_special = true) const override {
    std::string out;
    for (int32_t id : ids) {
      if (id < 0 || id >= (int32_t)id_to_tok_.size()) continue;
      if (is_added_[id]) {
        if (!(skip_special && special_[id])) out += id_to_tok_[id];
        continue;
      }
      const std::string& t = id_to_tok_[id];
      size_t p = 0;
      while (p < t.size()) {
        const uint32_t cp = utf8::decode(t, p);
        auto it = alpha_to_byte_.find(cp);
        if (it != alpha_to_byte_.end()) out.push_back((char)it->second);
        else utf8::append(out, cp);
      }
    }
    return out;
  }

 private:
  void init_byte_alphabet() {
    if (!byte_to_alpha_.empty()) return;
    // GPT-2 bytes_to_unicode: printable bytes map to themselves, the rest to 256 + n
    std::vector<int> bs;
    for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
    for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
    for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
    std::vector<uint32_t> cs(bs.begin(), bs.end());
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      if (std::find(bs.begin(), bs.end(), b) == bs.end()) { bs.push_back(b); cs.push_back(256 + n); ++n; }
    }
    byte_to_alpha_.assign(256, std::string());
    for (size_t i = 0; i < bs.size(); ++i) {
      std::string s;
      utf8::append(s, cs[i]);
      byte_to_alpha_[bs[i]] = s;
      alpha_to_byte_[cs[i]] = (uint8_t)bs[i];
    }
  }
  std::string bytes_to_alphabet(const std::string& bytes) const {
    std::string s;
    for (unsigned char c : bytes) s += byte_to_alpha_[c];
    return s;
  }
  void add_token(const std::string& tok, int32_t id, bool added, bool special = false) {
    if (id < 0) return;
    if (id >= (int32_t)id_to_tok_.size()) {
      id_to_tok_.resize(id + 1);
      special_.resize(id + 1, false);
      is_added_.resize(id + 1, false);
    }
    id_to_tok_[id] = tok;
    tok_to_id_[tok] = id;
    if (added) {
      is_added_[id] = true;
      special_[id] = special;
      added_.emplace_back(tok, id);
    }
  }
  void finalize() {
    added_by_first_.clear();
    for (size_t i = 0; i < added_.size(); ++i)
      if (!added_[i].first.empty()) added_by_first_[(unsigned char)added_[i].first[0]].push_back((int32_t)i);
  }
  static std::string base64_decode(const std::string& in) {
    static int8_t tbl[256];
    static bool init = false;
    if (!init) {
      for (int i = 0; i < 256; ++i) tbl[i] = -1;
      const char* a = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
      for (int i = 0; i < 64; ++i) tbl[(unsigned char)a[i]] = (int8_t)i;
      init = true;
    }
    std::string out;
    int val = 0, bits = -8;
    for (unsigned char c : in) {
      if (tbl[c] < 0) break;
      val = (val << 6) | tbl[c];
      bits += 6;
      if (bits >= 0) { out.push_back((char)((val >> bits) & 0xFF)); bits -= 8; }
    }
    return out;
  }

  // Pre-tokenisation: the GPT-4 / Qwen pattern
  //   (?i:'s|'t|'re|'ve|'m|'ll|'d) | [^\r\n\p{L}\p{N}]?\p{L}+ | \p{N}{1,k} | ?[^\s\p{L}\p{N}]+[\r\n]* |
  //   \s*[\r\n]+ | \s+(?!\S) | \s+
  // scanned by hand over code points.
  void split_words(const std::string& text, std::vector<std::string>& words) const {
    std::vector<uint32_t> cp;
    std::vector<size_t> off;
    for (size_t i = 0; i < text.size();) { off.push_back(i); cp.push_back(utf8::decode(text, i)); }
    off.push_back(text.size());
    const size_t n = cp.size();
    auto L = [&](size_t k) { return k < n && utf8::is_letter(cp[k]); };
    auto N = [&](size_t k) { return k < n && utf8::is_digit(cp[k]); };
    auto S = [&](size_t k) { return k < n && utf8::is_space(cp[k]); };
    auto NL = [&](size_t k) { return k < n && (cp[k] == '\n' || cp[k] == '\r'); };
    auto lower = [&](size_t k) { return k < n && cp[k] < 128 ? (char)tolower((int)cp[k]) : (char)0; };
    size_t i = 0;
    auto emit = [&](size_t b, size_t e) { words.push_back(text.substr(off[b], off[e] - off[b])); };
    while (i < n) {
      // contractions
      if (cp[i] == '\'' && i + 1 < n) {
        const char a = lower(i + 1), b = lower(i + 2);
        size_t len = 0;
        if (a == 's' || a == 't' || a == 'm' || a == 'd') len = 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) len = 3;
        if (len) { emit(i, i + len); i += len; continue; }
      }
      // [^\r\n\p{L}\p{N}]?\p{L}+
      if (L(i) || (!NL(i) && !N(i) && L(i + 1))) {
        size_t j = L(i) ? i : i + 1;
        while (L(j)) ++j;
        emit(i, j); i = j; continue;
      }
      if (N(i)) {
        size_t j = i + 1;
        const size_t cap = single_digits_ ? 1 : (digits_upto3_ ? 3 : SIZE_MAX);
        while (N(j) && j - i < cap) ++j;
        emit(i, j); i = j; continue;
      }
      //  ?[^\s\p{L}\p{N}]+[\r\n]*
      {
        size_t j = (cp[i] == ' ' && i + 1 < n && !S(i + 1) && !L(i + 1) && !N(i + 1)) ? i + 1 : i;
        if (j < n && !S(j) && !L(j) && !N(j)) {
          while (j < n && !S(j) && !L(j) && !N(j)) ++j;
          while (NL(j)) ++j;
          emit(i, j); i = j; continue;
        }
      }
      // whitespace runs
      if (S(i)) {
        size_t j = i;
        while (S(j)) ++j;
        // \s*[\r\n]+ : up to the last newline of the run
        size_t last_nl = SIZE_MAX;
        for (size_t k = i; k < j; ++k) if (NL(k)) last_nl = k;
        if (last_nl != SIZE_MAX) { emit(i, last_nl + 1); i = last_nl + 1; continue; }
        // \s+(?!\S) : leave the last space to glue onto the next word, unless at end of text
        if (j < n && j - i > 1) { emit(i, j - 1); i = j - 1; continue; }
        if (j < n && j - i == 1 && (L(j) || (!N(j) && !S(j)))) {
          // single space before a letter / punctuation run belongs to that run
          if (L(j)) { size_t k = j; while (L(k)) ++k; emit(i, k); i = k; continue; }
          size_t k = j; while (k < n && !S(k) && !L(k) && !N(k)) ++k; while (NL(k)) ++k;
          emit(i, k); i = k; continue;
        }
        emit(i, j); i = j; continue;
      }
      emit(i, i + 1); ++i;
    }
  }

  int32_t pair_rank(const std::string& a, const std::string& b) const {
    if (rank_is_id_) {
      auto it = tok_to_id_.find(a + b);
      return it == tok_to_id_.end() ? INT_MAX : it->second;
    }
    auto it = merges_.find(a + "\x01" + b);
    return it == merges_.end() ? INT_MAX : it->second;
  }

  void bpe_word(const std::string& word, std::vector<int32_t>& out) const {
    auto whole = tok_to_id_.find(word);
    if (whole != tok_to_id_.end() && !is_added_[whole->second]) { out.push_back(whole->second); return; }
    std::vector<std::string> parts;
    for (size_t p = 0; p < word.size();) { size_t q = p; utf8::decode(word, q); parts.push_back(word.substr(p, q - p)); p = q; }
    while (parts.size() > 1) {
      int32_t best = INT_MAX;
      size_t at = 0;
      for (size_t k = 0; k + 1 < parts.size(); ++k) {
        const int32_t r = pair_rank(parts[k], parts[k + 1]);
        if (r < best) { best = r; at = k; }
      }
      if (best == INT_MAX) break;
      parts[at] += parts[at + 1];
      parts.erase(parts.begin() + at + 1);
    }
    for (auto& p : parts) {
      auto it = tok_to_id_.find(p);
      if (it != tok_to_id_.end()) out.push_back(it->second);
      else if (unk_ >= 0) out.push_back(unk_);
    }
  }

  void encode_plain(const std::string& text, std::vector<int32_t>& out) const {
    std::vector<std::string> words;
    split_words(text, words);
    for (auto& w : words) bpe_word(bytes_to_alphabet(w), out);
  }

  std::vector<std::string> id_to_tok_;
  std::unordered_map<std::string, int32_t> tok_to_id_;
  std::unordered_map<std::string, int32_t> merges_;
  std::vector<bool> special_, is_added_;
  std::vector<std::pair<std::string, int32_t>> added_;
  std::unordered_map<int, std::vector<int32_t>> added_by_first_;
  std::vector<std::string> byte_to_alpha_;
  std::unordered_map<uint32_t, uint8_t> alpha_to_byte_;
  bool single_digits_ = true, digits_upto3_ = false, rank_is_id_ = false;
  int32_t bos_ = -1, eos_ = -1, unk_ = -1;
};

}  // namespace xllm
