// Test-only Python module: drives host-side policies of the backend against
// fakes, on a machine without a GPU. It is compiled from the product's own
// sources (the allocator and the watchdog) plus the harnesses in this folder,
// and is never loaded by the product.
#include <pybind11/functional.h>
#include <torch/csrc/utils/pybind.h>

namespace torch_gcu {
py::dict allocator_selftest();              // allocator_selftest.cpp
}
namespace c10d_gcu {
void bind_watchdog_selftest(py::module& m);  // watchdog_selftest.cpp
}

PYBIND11_MODULE(_gcu_selftest, m) {
  m.def("allocator_selftest", &torch_gcu::allocator_selftest);
  c10d_gcu::bind_watchdog_selftest(m);
}
