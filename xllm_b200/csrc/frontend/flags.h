// Launch-flag registry with the reference's flag names, types and defaults.
//
// Parity: the gflags-based config system (xllm/core/framework/config/*_config.cpp,
// config_utils.cpp:44-208, help_formatter.h): `--name=value`, `--name value`, `--name` / `--noname`
// for booleans, `--config_json_file` whose keys are flag names (values in the file win over the
// command line, as the reference documents), dumping of the resolved non-default configuration,
// grouped `--help`, and the cross-flag validation of xllm.cpp:327-428.
#pragma once
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "json.h"

namespace xllm {

enum class FlagType { STRING, INT, DOUBLE, BOOL };

struct FlagDef {
  std::string category, name;
  FlagType type;
  std::string def;
};

class FlagRegistry {
 public:
  FlagRegistry() {
#define XLLM_FLAG(cat, name, type, def) add(cat, name, FlagType::type, def);
#include "flag_table.inc"
#undef XLLM_FLAG
    // flags of this engine that the reference does not have
    add("B200Config", "devices", FlagType::STRING, "auto");
    add("B200Config", "gemm_backend", FlagType::STRING, "tcgen05");
    add("B200Config", "tp_comm", FlagType::STRING, "fused");
    add("B200Config", "max_model_len", FlagType::INT, "0");
    add("B200Config", "enable_cuda_graph", FlagType::BOOL, "true");
    add("B200Config", "scheduler_policy", FlagType::STRING, "prefill_first");
    add("B200Config", "random_weights", FlagType::BOOL, "false");
  }

  void add(const std::string& cat, const std::string& name, FlagType t, const std::string& def) {
    if (index_.count(name)) return;
    index_[name] = defs_.size();
    defs_.push_back({cat, name, t, def});
    values_.push_back(def);
    set_.push_back(false);
  }

  bool has(const std::string& name) const { return index_.count(name) != 0; }
  const std::vector<FlagDef>& defs() const { return defs_; }

  std::string get(const std::string& name) const {
    auto it = index_.find(name);
    if (it == index_.end()) throw std::invalid_argument("unknown flag --" + name);
    return values_[it->second];
  }
  int64_t get_int(const std::string& n) const { return std::stoll(get(n)); }
  double get_double(const std::string& n) const { return std::stod(get(n)); }
  bool get_bool(const std::string& n) const { const std::string v = get(n); return v == "true" || v == "1"; }
  bool is_set(const std::string& n) const { auto it = index_.find(n); return it != index_.end() && set_[it->second]; }

  void set(const std::string& name, const std::string& value) {
    auto it = index_.find(name);
    if (it == index_.end()) throw std::invalid_argument("unknown flag --" + name);
    values_[it->second] = normalise(defs_[it->second], value);
    set_[it->second] = true;
  }

  // Returns the positional (non-flag) arguments.
  std::vector<std::string> parse_args(const std::vector<std::string>& argv) {
    std::vector<std::string> positional;
    for (size_t i = 0; i < argv.size(); ++i) {
      const std::string& a = argv[i];
      if (a.size() < 2 || a[0] != '-') { positional.push_back(a); continue; }
      std::string body = a.substr(a[1] == '-' ? 2 : 1);
      std::string name = body, value;
      bool has_value = false;
      const size_t eq = body.find('=');
      if (eq != std::string::npos) { name = body.substr(0, eq); value = body.substr(eq + 1); has_value = true; }
      if (name == "help" || name == "h") { help_requested_ = true; continue; }
      auto it = index_.find(name);
      if (it == index_.end() && name.rfind("no", 0) == 0 && index_.count(name.substr(2)) &&
          defs_[index_[name.substr(2)]].type == FlagType::BOOL && !has_value) {
        set(name.substr(2), "false");
        continue;
      }
      if (it == index_.end()) throw std::invalid_argument("unknown flag --" + name);
      const FlagDef& d = defs_[it->second];
      if (!has_value) {
        if (d.type == FlagType::BOOL) {
          // `--flag` alone means true; `--flag true|false` is accepted too
          if (i + 1 < argv.size() && (argv[i + 1] == "true" || argv[i + 1] == "false")) value = argv[++i];
          else value = "true";
        } else {
          if (i + 1 >= argv.size()) throw std::invalid_argument("flag --" + name + " needs a value");
          value = argv[++i];
        }
      }
      set(name, value);
    }
    if (!get("config_json_file").empty()) load_json_file(get("config_json_file"));
    return positional;
  }
  bool help_requested() const { return help_requested_; }

  void load_json_file(const std::string& path) {
    std::ifstream f(path);
    if (!f) throw std::runtime_error("cannot open config json " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    load_json(Json::parse(ss.str()));
  }
  void load_json(const Json& j) {
    if (!j.is_object()) throw std::invalid_argument("config json must be an object");
    for (auto& kv : j.members()) {
      if (!has(kv.first)) throw std::invalid_argument("unknown key in config json: " + kv.first);
      const Json& v = kv.second;
      if (v.is_string()) set(kv.first, v.as_string());
      else if (v.is_bool()) set(kv.first, v.as_bool() ? "true" : "false");
      else if (v.is_int()) set(kv.first, std::to_string(v.as_int()));
      else if (v.is_number()) set(kv.first, v.dump());
      else throw std::invalid_argument("config json value of " + kv.first + " must be a scalar");
    }
  }

  // Flags that differ from their default (all flags when `all`).
  Json to_json(bool all = false) const {
    Json o = Json::object();
    for (size_t i = 0; i < defs_.size(); ++i) {
      if (!all && values_[i] == defs_[i].def) continue;
      const FlagDef& d = defs_[i];
      switch (d.type) {
        case FlagType::STRING: o.set(d.name, values_[i]); break;
        case FlagType::INT: o.set(d.name, (int64_t)std::stoll(values_[i])); break;
        case FlagType::DOUBLE: o.set(d.name, std::stod(values_[i])); break;
        case FlagType::BOOL: o.set(d.name, values_[i] == "true"); break;
      }
    }
    return o;
  }

  std::string help() const {
    std::string out = "xllm_b200 serve --model <PATH> [flags]\n";
    std::string cat;
    for (auto& d : defs_) {
      if (d.category != cat) { cat = d.category; out += "\n" + cat + ":\n"; }
      static const char* tn[] = {"string", "int", "double", "bool"};
      out += "  --" + d.name + " (" + tn[(int)d.type] + ", default " + (d.def.empty() ? "\"\"" : d.def) + ")\n";
    }
    return out;
  }

  // Cross-flag rules. Returns a list of problems (empty = valid).
  std::vector<std::string> validate() const {
    std::vector<std::string> bad;
    auto pos = [&](const char* n) { if (get_int(n) <= 0) bad.push_back(std::string("--") + n + " must be positive"); };
    if (get("model").empty() && !get_bool("random_weights")) bad.push_back("--model is required");
    pos("block_size"); pos("max_tokens_per_batch"); pos("max_seqs_per_batch"); pos("dp_size"); pos("ep_size");
    if (get_int("block_size") % 16 != 0) bad.push_back("--block_size must be a multiple of 16");
    const double u = get_double("max_memory_utilization");
    if (!(u > 0.0 && u <= 1.0)) bad.push_back("--max_memory_utilization must be in (0, 1]");
    if (get_int("nnodes") > 0 && get_int("node_rank") >= get_int("nnodes")) bad.push_back("--node_rank must be < --nnodes");
    if (get_int("nnodes") > 0 && get_int("nnodes") % get_int("dp_size") != 0) bad.push_back("--nnodes must be divisible by --dp_size");
    if (get_int("nnodes") > 0 && get_int("nnodes") % get_int("ep_size") != 0) bad.push_back("--nnodes must be divisible by --ep_size");
    if (get_int("num_speculative_tokens") > 0 && get("draft_model").empty() && get("speculative_algorithm").empty())
      bad.push_back("--num_speculative_tokens needs --draft_model or --speculative_algorithm");
    const std::string role = get("instance_role");
    if (!role.empty() && role != "DEFAULT" && role != "PREFILL" && role != "DECODE" && role != "MIX")
      bad.push_back("--instance_role must be DEFAULT, PREFILL, DECODE or MIX");
    if (get_bool("enable_disagg_pd") && (role.empty() || role == "DEFAULT"))
      bad.push_back("--enable_disagg_pd needs --instance_role PREFILL or DECODE");
    // rules of the reference's option check (xllm/core/distributed_runtime/master.cpp:100-284, xllm.cpp)
    const std::string backend = get("backend");
    if (!backend.empty() && backend != "llm" && backend != "vlm" && backend != "dit" && backend != "rec")
      bad.push_back("--backend must be llm, vlm, dit or rec");
    const std::string task = get("task");
    if (task != "generate" && task != "embed" && task != "mm_embed") bad.push_back("--task must be generate, embed or mm_embed");
    if (backend == "rec" && task != "generate") bad.push_back("--backend rec serves --task generate only");
    if (get_double("host_blocks_factor") > 1.0 || get_double("host_blocks_factor") < 0.0)
      bad.push_back("--host_blocks_factor must be in [0, 1]");
    if (get_int("cp_size") != 1) bad.push_back("--cp_size: context parallelism of the serving engine is not available on this platform (use 1)");
    if (get_int("kv_split_size") != 1) bad.push_back("--kv_split_size: decode context parallelism is not available on this platform (use 1)");
    if (get_int("beam_width") < 1) bad.push_back("--beam_width must be >= 1");
    if (get_int("beam_width") > 1 && get_int("num_speculative_tokens") > 0)
      bad.push_back("--beam_width > 1 cannot be combined with speculative decoding");
    if (get_bool("enable_eplb") && get_int("ep_size") <= 1) bad.push_back("--enable_eplb needs --ep_size > 1");
    if (get_bool("enable_eplb") && get_int("redundant_experts_num") < 0) bad.push_back("--redundant_experts_num must be >= 0");
    const std::string mode = get("kv_cache_transfer_mode");
    if (mode != "PUSH" && mode != "PULL") bad.push_back("--kv_cache_transfer_mode must be PUSH or PULL");
    const std::string kvd = get("kv_cache_dtype");
    if (kvd != "auto" && kvd != "bfloat16" && kvd != "float16" && kvd != "fp8" && kvd != "int8")
      bad.push_back("--kv_cache_dtype must be auto, bfloat16, float16, fp8 or int8");
    if (get_int("max_tokens_per_chunk_for_prefill") == 0) bad.push_back("--max_tokens_per_chunk_for_prefill must be positive (or -1: the batch budget)");
    if (get_int("max_seqs_per_batch") > get_int("max_tokens_per_batch"))
      bad.push_back("--max_seqs_per_batch must not exceed --max_tokens_per_batch (every running sequence needs one token per step)");
    if (get_int("max_concurrent_requests") < 0) bad.push_back("--max_concurrent_requests must be >= 0");
    if (get_int("num_request_handling_threads") < 1 || get_int("num_response_handling_threads") < 1)
      bad.push_back("--num_request_handling_threads and --num_response_handling_threads must be >= 1");
    if (get_bool("enable_disagg_pd") && get_int("num_speculative_tokens") > 0 && role == "PREFILL")
      bad.push_back("a PREFILL instance does not speculate: drop --num_speculative_tokens");
    return bad;
  }

 private:
  static std::string normalise(const FlagDef& d, const std::string& v) {
    switch (d.type) {
      case FlagType::BOOL:
        if (v == "true" || v == "1" || v == "True") return "true";
        if (v == "false" || v == "0" || v == "False") return "false";
        throw std::invalid_argument("flag --" + d.name + " expects true/false, got " + v);
      case FlagType::INT: {
        size_t n = 0;
        long long x = std::stoll(v, &n);
        if (n != v.size()) throw std::invalid_argument("flag --" + d.name + " expects an integer, got " + v);
        return std::to_string(x);
      }
      case FlagType::DOUBLE: {
        size_t n = 0;
        (void)std::stod(v, &n);
        if (n != v.size()) throw std::invalid_argument("flag --" + d.name + " expects a number, got " + v);
        return v;
      }
      default: return v;
    }
  }

  std::vector<FlagDef> defs_;
  std::vector<std::string> values_;
  std::vector<bool> set_;
  std::unordered_map<std::string, size_t> index_;
  bool help_requested_ = false;
};

}  // namespace xllm
