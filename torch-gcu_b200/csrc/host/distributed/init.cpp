// Python bindings of the "eccl" c10d backend: torch_gcu._C._distributed_c10d.
// Constructor signatures and the extra methods follow the reference's binding
// (reference: torch_gcu/csrc/python/dist_py_init.cpp:79-144): (store, rank, size,
// timeout) or (store, rank, size, Options); allreduce_outplace, get_unique_id,
// options.
#include <pybind11/chrono.h>
#include <torch/csrc/utils/pybind.h>

#include "distributed/ProcessGroupECCL.hpp"

namespace torch_gcu {

void init_distributed_bindings(py::module& root) {
  using PG = ::c10d_gcu::ProcessGroupECCL;
  py::module m = root.def_submodule("_distributed_c10d", "c10d bindings of the gcu backend");
  py::module dist = py::module::import("torch._C._distributed_c10d");

  auto pg = py::class_<PG, c10::intrusive_ptr<PG>>(m, "ProcessGroupECCL", dist.attr("Backend"));
  py::class_<PG::Options, c10::intrusive_ptr<PG::Options>>(pg, "Options", dist.attr("Backend").attr("Options"))
      .def(py::init([](bool is_high_priority_stream) { return PG::Options::create(is_high_priority_stream); }),
           py::arg("is_high_priority_stream") = true)
      .def_readwrite("is_high_priority_stream", &PG::Options::is_high_priority_stream)
      .def_readwrite("op_timeout", &PG::Options::timeout);

  pg.def(py::init([](const c10::intrusive_ptr<::c10d::Store>& store, int rank, int size, c10::intrusive_ptr<PG::Options> options) {
           return c10::make_intrusive<PG>(store, rank, size, std::move(options));
         }),
         py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("options"), py::call_guard<py::gil_scoped_release>())
      .def(py::init([](const c10::intrusive_ptr<::c10d::Store>& store, int rank, int size, const std::chrono::milliseconds& timeout) {
             auto options = PG::Options::create(false);
             options->timeout = timeout;
             return c10::make_intrusive<PG>(store, rank, size, options);
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"),
           py::arg("timeout") = ::c10d_gcu::kProcessGroupECCLDefaultTimeout, py::call_guard<py::gil_scoped_release>())
      .def("allreduce_outplace", &PG::allreduce_outplace, py::arg("outputTensor"), py::arg("inputTensor"),
           py::arg("opts") = ::c10d::AllreduceOptions(), py::call_guard<py::gil_scoped_release>())
      .def("get_unique_id", &PG::get_unique_id_hex, py::call_guard<py::gil_scoped_release>())
      .def("abort", &PG::abort, py::call_guard<py::gil_scoped_release>())
      .def("shutdown", &PG::shutdown, py::call_guard<py::gil_scoped_release>())
      .def_static("_check_tensor", [](const at::Tensor& t) { PG::check_tensor(t, "check"); })
      .def("_group_start", &PG::group_start, py::call_guard<py::gil_scoped_release>())
      .def("_group_end", &PG::group_end, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("options", &PG::getOptions);
}

}  // namespace torch_gcu
