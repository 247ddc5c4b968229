// Bindings of the C++ HTTP server and the metrics registry.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "http_server.h"
#include "metrics.h"
#include "response_processor.h"
#include "../runtime/scheduler.h"

namespace py = pybind11;
using namespace xllm;

void bind_server(py::module_& m) {
  py::class_<HttpRequest>(m, "HttpRequest")
      .def_readonly("id", &HttpRequest::id)
      .def_readonly("method", &HttpRequest::method)
      .def_readonly("path", &HttpRequest::path)
      .def_readonly("query", &HttpRequest::query)
      .def_property_readonly("body", [](const HttpRequest& r) { return py::bytes(r.body); })
      .def_readonly("headers", &HttpRequest::headers)
      .def("header", &HttpRequest::header);

  py::class_<HttpServer>(m, "HttpServer")
      .def(py::init<>())
      .def("start", &HttpServer::start, py::arg("host") = "", py::arg("port") = 0)
      .def("stop", &HttpServer::stop, py::call_guard<py::gil_scoped_release>())
      .def("poll", &HttpServer::poll, py::arg("timeout_ms") = 0, py::call_guard<py::gil_scoped_release>())
      .def("respond", &HttpServer::respond, py::arg("id"), py::arg("status"), py::arg("content_type"),
           py::arg("body"), py::arg("extra_headers") = std::vector<std::pair<std::string, std::string>>())
      .def("stream_begin", &HttpServer::stream_begin)
      .def("stream_send", &HttpServer::stream_send)
      .def("stream_end", &HttpServer::stream_end)
      .def("is_disconnected", &HttpServer::is_disconnected)
      // the ids among `ids` whose connection is gone (one lock for all of them)
      .def("disconnected_among", [](HttpServer& s, const std::vector<int64_t>& ids) {
             std::vector<int64_t> gone;
             for (int64_t id : ids)
               if (s.is_disconnected(id)) gone.push_back(id);
             return gone;
           })
      .def("num_connections", &HttpServer::num_connections)
      .def_property_readonly("port", &HttpServer::port);

  py::class_<RespCallSpec>(m, "RespCallSpec")
      .def(py::init<>())
      .def_readwrite("http_id", &RespCallSpec::http_id)
      .def_readwrite("request_id", &RespCallSpec::request_id)
      .def_readwrite("model", &RespCallSpec::model)
      .def_readwrite("kind", &RespCallSpec::kind)
      .def_readwrite("stream", &RespCallSpec::stream)
      .def_readwrite("include_usage", &RespCallSpec::include_usage)
      .def_readwrite("return_token_ids", &RespCallSpec::return_token_ids)
      .def_readwrite("n", &RespCallSpec::n)
      .def_readwrite("prompt_tokens", &RespCallSpec::prompt_tokens)
      .def_readwrite("created", &RespCallSpec::created)
      .def_readwrite("echo_text", &RespCallSpec::echo_text)
      .def_readwrite("stops", &RespCallSpec::stops)
      .def_readwrite("skip_special", &RespCallSpec::skip_special)
      .def_readwrite("t_arrival", &RespCallSpec::t_arrival);

  py::class_<RespDone>(m, "RespDone")
      .def_readonly("request_id", &RespDone::request_id)
      .def_readonly("http_id", &RespDone::http_id)
      .def_readonly("generated", &RespDone::generated)
      .def_readonly("prompt_tokens", &RespDone::prompt_tokens)
      .def_readonly("aborted", &RespDone::aborted)
      .def_readonly("ttft_ms", &RespDone::ttft_ms)
      .def_readonly("e2e_ms", &RespDone::e2e_ms);

  py::class_<ResponseProcessor>(m, "ResponseProcessor")
      .def(py::init([](HttpServer* http, py::object tok, int n_threads) {
             std::shared_ptr<BpeTokenizer> t;
             if (!tok.is_none()) t = tok.cast<std::shared_ptr<BpeTokenizer>>();
             return new ResponseProcessor(http, std::move(t), n_threads);
           }),
           py::arg("http"), py::arg("tokenizer"), py::arg("n_threads") = 4, py::keep_alive<1, 2>())
      .def("open", &ResponseProcessor::open)
      // events of one engine step as parallel lists: handles, sequence indices, tokens, flags
      // (bit 0 finished, bit 1 request_finished, bit 2 aborted), finish reasons
      .def("push",
           [](ResponseProcessor& rp, const std::vector<int64_t>& calls, const std::vector<int32_t>& seq,
              const std::vector<int32_t>& tokens, const std::vector<int32_t>& flags,
              const std::vector<std::string>& reasons) {
             std::vector<RespEvent> ev(calls.size());
             for (size_t i = 0; i < calls.size(); ++i) {
               ev[i].call = calls[i];
               ev[i].seq_index = seq[i];
               ev[i].token = tokens[i];
               ev[i].finished = flags[i] & 1;
               ev[i].request_finished = flags[i] & 2;
               ev[i].aborted = flags[i] & 4;
               if (i < reasons.size()) ev[i].finish_reason = reasons[i];
             }
             py::gil_scoped_release rel;
             rp.push(std::move(ev));
           })
      // The engine's events as they come out of step(): those whose request id is in `handles` go to the
      // workers, the indices of the others are returned (the caller formats them itself).  No per-event
      // attribute access in the interpreter.
      .def("push_events",
           [](ResponseProcessor& rp, const py::list& events, const py::dict& handles) {
             std::vector<RespEvent> ev;
             std::vector<int64_t> rest;
             ev.reserve(events.size());
             int64_t i = 0;
             for (const py::handle& h : events) {
               const OutputEvent* e = nullptr;
               try {
                 e = &h.cast<const OutputEvent&>();
               } catch (const py::cast_error&) {
                 rest.push_back(i++);        // a wrapped event (first token of a disaggregated request, ...)
                 continue;
               }
               py::object key = py::str(e->request_id);
               if (!handles.contains(key)) {
                 rest.push_back(i++);
                 continue;
               }
               RespEvent r;
               r.call = handles[key].cast<int64_t>();
               r.seq_index = e->seq_index;
               r.token = e->token;
               r.finished = e->finished;
               r.request_finished = e->request_finished;
               r.aborted = e->finished && e->finish_reason == "abort";
               if (e->finished) r.finish_reason = e->finish_reason;
               ev.push_back(std::move(r));
               ++i;
             }
             if (!ev.empty()) {
               py::gil_scoped_release rel;
               rp.push(std::move(ev));
             }
             return rest;
           })
      .def("take_done", &ResponseProcessor::take_done)
      .def("drain", &ResponseProcessor::drain, py::arg("timeout_ms") = 5000, py::call_guard<py::gil_scoped_release>())
      .def("stop", &ResponseProcessor::stop, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("pending", &ResponseProcessor::pending)
      .def_property_readonly("processed", &ResponseProcessor::processed)
      .def_property_readonly("num_threads", &ResponseProcessor::num_threads);

  m.def("metric_counter_add", [](const std::string& n, double v) { Metrics::instance().counter_add(n, v); },
        py::arg("name"), py::arg("value") = 1.0);
  m.def("metric_gauge_set", [](const std::string& n, double v) { Metrics::instance().gauge_set(n, v); });
  m.def("metric_histogram_observe", [](const std::string& n, double v) { Metrics::instance().histogram_observe(n, v); });
  m.def("metric_counter", [](const std::string& n) { return Metrics::instance().counter(n); });
  m.def("metric_gauge", [](const std::string& n) { return Metrics::instance().gauge(n); });
  m.def("metric_quantile", [](const std::string& n, double q) { return Metrics::instance().quantile(n, q); });
  m.def("metrics_text", [] { return Metrics::instance().prometheus_text(); });
  m.def("metrics_reset", [] { Metrics::instance().reset(); });
}
