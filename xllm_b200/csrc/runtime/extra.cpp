// Additional runtime bindings: the virtual-memory page pool (vmm.h).
#include <pybind11/pybind11.h>

#include <memory>

#include "vmm.h"
namespace py = pybind11;
using namespace xllm;

void bind_runtime_extra(py::module_& m) {
  m.def("vmm_cuda_available", [] { return cuda_driver() != nullptr; });
  py::class_<PhyPagePool, std::shared_ptr<PhyPagePool>>(m, "PhyPagePool")
      .def(py::init([](int device, size_t page_bytes, size_t max_pages, bool fake) {
             return std::make_shared<PhyPagePool>(fake ? fake_driver() : cuda_driver(), device, page_bytes, max_pages);
           }),
           py::arg("device") = 0, py::arg("page_bytes") = size_t(2) << 20, py::arg("max_pages") = 1024,
           py::arg("fake") = false)
      .def("trim", &PhyPagePool::trim)
      .def_property_readonly("page_bytes", &PhyPagePool::page_bytes)
      .def_property_readonly("max_pages", &PhyPagePool::max_pages)
      .def_property_readonly("pages_created", &PhyPagePool::pages_created)
      .def_property_readonly("pages_in_use", &PhyPagePool::pages_in_use)
      .def_property_readonly("pages_free", &PhyPagePool::pages_free)
      .def_property_readonly("driver", [](const PhyPagePool& p) { return std::string(p.driver()->name); });
  py::class_<XTensor>(m, "XTensor")
      .def(py::init([](std::shared_ptr<PhyPagePool> pool, size_t virt_bytes) { return new XTensor(pool.get(), virt_bytes); }),
           py::arg("pool"), py::arg("virt_bytes"), py::keep_alive<1, 2>())
      .def_property_readonly("ptr", &XTensor::ptr)
      .def_property_readonly("virt_bytes", &XTensor::virt_bytes)
      .def_property_readonly("mapped_bytes", &XTensor::mapped_bytes)
      .def("is_mapped", &XTensor::is_mapped)
      .def("map_range", &XTensor::map_range)
      .def("unmap_range", &XTensor::unmap_range)
      .def("ensure", &XTensor::ensure)
      .def("release_all", &XTensor::release_all);
}
