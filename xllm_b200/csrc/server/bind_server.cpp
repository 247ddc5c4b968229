// Bindings of the C++ HTTP server.
#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_server(py::module_& m) { (void)m; }
