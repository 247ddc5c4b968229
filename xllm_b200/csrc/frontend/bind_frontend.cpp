// Bindings of the C++ front end (tokenizer, chat template, parsers, loaders).
#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_frontend(py::module_& m) { (void)m; }
