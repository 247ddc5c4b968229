// Bindings of the C++ front end (flags, JSON, safetensors, tokenizer, chat template, parsers).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "flags.h"
#include "json.h"
#include "parsers.h"
#include "safetensors.h"
#include "text.h"
#include "tokenizer.h"

namespace py = pybind11;
using namespace xllm;

static py::object json_to_py(const Json& j) {
  switch (j.type()) {
    case Json::NUL: return py::none();
    case Json::BOOL: return py::bool_(j.as_bool());
    case Json::INT: return py::int_(j.as_int());
    case Json::DOUBLE: return py::float_(j.as_double());
    case Json::STRING: return py::str(j.as_string());
    case Json::ARRAY: {
      py::list l;
      for (auto& v : j.items()) l.append(json_to_py(v));
      return std::move(l);
    }
    default: {
      py::dict d;
      for (auto& kv : j.members()) d[py::str(kv.first)] = json_to_py(kv.second);
      return std::move(d);
    }
  }
}

void bind_frontend(py::module_& m) {
  m.def("json_loads", [](const std::string& s) { return json_to_py(Json::parse(s)); });
  m.def("json_roundtrip", [](const std::string& s, int indent) { return Json::parse(s).dump(indent); },
        py::arg("text"), py::arg("indent") = -1);
  m.def("complete_partial_json", [](const std::string& s) -> py::object {
    std::string out;
    if (!complete_partial_json(s, &out)) return py::none();
    return py::str(out);
  });

  py::class_<FlagRegistry>(m, "FlagRegistry")
      .def(py::init<>())
      .def("parse_args", &FlagRegistry::parse_args)
      .def("load_json_file", &FlagRegistry::load_json_file)
      .def("load_json", [](FlagRegistry& f, const std::string& text) { f.load_json(Json::parse(text)); })
      .def("get", &FlagRegistry::get)
      .def("get_int", &FlagRegistry::get_int)
      .def("get_double", &FlagRegistry::get_double)
      .def("get_bool", &FlagRegistry::get_bool)
      .def("set", &FlagRegistry::set)
      .def("has", &FlagRegistry::has)
      .def("is_set", &FlagRegistry::is_set)
      .def("help", &FlagRegistry::help)
      .def("help_requested", &FlagRegistry::help_requested)
      .def("validate", &FlagRegistry::validate)
      .def("to_json", [](const FlagRegistry& f, bool all, int indent) { return f.to_json(all).dump(indent); },
           py::arg("all") = false, py::arg("indent") = 2)
      .def("names", [](const FlagRegistry& f) {
        std::vector<std::string> out;
        for (auto& d : f.defs()) out.push_back(d.name);
        return out;
      })
      .def("categories", [](const FlagRegistry& f) {
        std::vector<std::pair<std::string, std::string>> out;
        for (auto& d : f.defs()) out.emplace_back(d.category, d.name);
        return out;
      });

  py::class_<SafeTensorsFile, std::shared_ptr<SafeTensorsFile>>(m, "SafeTensorsFile")
      .def(py::init<const std::string&>())
      .def("keys", [](const SafeTensorsFile& f) {
        std::vector<std::string> k;
        for (auto& t : f.tensors()) k.push_back(t.name);
        return k;
      })
      .def("metadata", &SafeTensorsFile::metadata)
      // name -> (dtype string, shape, begin, end) of every tensor
      .def("index", [](const SafeTensorsFile& f) {
        py::dict d;
        for (auto& t : f.tensors()) d[py::str(t.name)] = py::make_tuple(t.dtype, t.shape, t.begin, t.end);
        return d;
      })
      // zero-copy read-only view of the whole data section (kept alive by the file object)
      .def("buffer", [](std::shared_ptr<SafeTensorsFile> f) {
        return py::memoryview::from_memory((const void*)f->data(), (py::ssize_t)f->data_size());
      }, py::keep_alive<0, 1>());

  py::class_<BpeTokenizer, std::shared_ptr<BpeTokenizer>>(m, "BpeTokenizer")
      .def(py::init<>())
      .def("load_hf_json", &BpeTokenizer::load_hf_json)
      .def("load_hf_file", [](BpeTokenizer& t, const std::string& path) { t.load_hf_json(BpeTokenizer::read_file(path)); })
      .def("load_tiktoken", &BpeTokenizer::load_tiktoken)
      .def("load_tiktoken_file", [](BpeTokenizer& t, const std::string& path,
                                    const std::vector<std::pair<std::string, int32_t>>& specials) {
        t.load_tiktoken(BpeTokenizer::read_file(path), specials);
      })
      .def("set_bos_eos", &BpeTokenizer::set_bos_eos)
      .def("encode", &BpeTokenizer::encode, py::arg("text"), py::arg("add_special") = false,
           py::call_guard<py::gil_scoped_release>())
      .def("decode", [](const BpeTokenizer& t, const std::vector<int32_t>& ids, bool skip) {
        const std::string s = t.decode(ids, skip);
        return py::reinterpret_steal<py::str>(PyUnicode_DecodeUTF8(s.data(), (Py_ssize_t)s.size(), "replace"));
      }, py::arg("ids"), py::arg("skip_special") = true)
      .def("decode_bytes", [](const BpeTokenizer& t, const std::vector<int32_t>& ids, bool skip) {
        return py::bytes(t.decode(ids, skip));
      }, py::arg("ids"), py::arg("skip_special") = true)
      .def("token_to_id", &BpeTokenizer::token_to_id)
      .def("id_to_token", &BpeTokenizer::id_to_token)
      .def("is_special", &BpeTokenizer::is_special)
      .def_property_readonly("vocab_size", &BpeTokenizer::vocab_size);

  py::class_<IncrementalDecoder>(m, "IncrementalDecoder")
      .def(py::init([](std::shared_ptr<BpeTokenizer> tok, std::vector<std::string> stops, bool skip) {
        return new IncrementalDecoder(tok.get(), std::move(stops), skip);
      }), py::arg("tokenizer"), py::arg("stops") = std::vector<std::string>(), py::arg("skip_special") = true,
          py::keep_alive<1, 2>())
      .def("push", [](IncrementalDecoder& d, int32_t tok) {
        bool stopped = false;
        std::string s = d.push(tok, &stopped);
        return py::make_tuple(py::reinterpret_steal<py::str>(PyUnicode_DecodeUTF8(s.data(), (Py_ssize_t)s.size(), "replace")), stopped);
      })
      .def("flush", [](IncrementalDecoder& d) {
        std::string s = d.flush();
        return py::reinterpret_steal<py::str>(PyUnicode_DecodeUTF8(s.data(), (Py_ssize_t)s.size(), "replace"));
      })
      .def("text", [](const IncrementalDecoder& d) {
        const std::string& s = d.text();
        return py::reinterpret_steal<py::str>(PyUnicode_DecodeUTF8(s.data(), (Py_ssize_t)s.size(), "replace"));
      });

  py::class_<ChatMessage>(m, "ChatMessage")
      .def(py::init([](std::string role, std::string content, std::string tool_calls_json, std::string tool_call_id) {
        ChatMessage c;
        c.role = std::move(role); c.content = std::move(content);
        c.tool_calls_json = std::move(tool_calls_json); c.tool_call_id = std::move(tool_call_id);
        return c;
      }), py::arg("role"), py::arg("content"), py::arg("tool_calls_json") = "", py::arg("tool_call_id") = "")
      .def_readwrite("role", &ChatMessage::role)
      .def_readwrite("content", &ChatMessage::content);

  py::class_<ChatTemplate>(m, "ChatTemplate")
      .def(py::init<std::string>())
      .def_static("detect_family", &ChatTemplate::detect_family)
      .def("apply", &ChatTemplate::apply, py::arg("messages"), py::arg("tools_json") = "",
           py::arg("add_generation_prompt") = true, py::arg("enable_thinking") = true);

  py::class_<ReasoningParser>(m, "ReasoningParser")
      .def(py::init<const std::string&, bool>(), py::arg("kind") = "qwen3", py::arg("starts_in_reasoning") = false)
      .def("push", [](ReasoningParser& p, const std::string& d) { auto r = p.push(d); return py::make_tuple(r.reasoning, r.content); })
      .def("flush", [](ReasoningParser& p) { auto r = p.flush(); return py::make_tuple(r.reasoning, r.content); });

  auto conv = [](const ToolParseResult& r) {
    py::list calls;
    for (auto& c : r.calls) calls.append(py::make_tuple(c.index, c.name, c.arguments));
    return py::make_tuple(r.content, calls);
  };
  py::class_<ToolCallParser>(m, "ToolCallParser")
      .def(py::init<const std::string&>())
      .def("has_tool_call", &ToolCallParser::has_tool_call)
      .def("parse", [conv](const ToolCallParser& p, const std::string& t) { return conv(p.parse(t)); })
      .def("push", [conv](ToolCallParser& p, const std::string& d) { return conv(p.push(d)); });
}
