// Bindings of the C++ HTTP server and the metrics registry.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "http_server.h"
#include "metrics.h"

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
      .def("num_connections", &HttpServer::num_connections)
      .def_property_readonly("port", &HttpServer::port);

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
