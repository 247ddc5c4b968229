// Additional runtime bindings (filled in as components land).
#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_runtime_extra(py::module_& m) { (void)m; }
