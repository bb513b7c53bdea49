// torch_gcu._C: the Python bindings of the gcu backend (reference:
// torch_gcu/csrc/InitGcuBindings.cpp:59-127,251-292, csrc/python/gcu_module.cpp,
// csrc/python/efficient_ops.cpp:11-26, csrc/python/dist_py_init.cpp:79-144).
// Streams and events need no classes of their own: torch.Stream / torch.Event
// drive the registered device guard.
#include <ATen/autocast_mode.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/csrc/utils/tensor_dtypes.h>
#include <torch/extension.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"
#include "runtime/gcu_allocator.h"
#include "runtime/gcu_graph.h"
#include "runtime/gcu_runtime.h"

namespace torch_gcu {
void register_runtime();                              // runtime/gcu_guard_hooks.cpp
const at::Generator& default_generator(c10::DeviceIndex idx);
void init_distributed_bindings(py::module& m);        // distributed/init.cpp
void init_tp_exchange_bindings(py::module& m);        // distributed/tp_exchange.cpp
}  // namespace torch_gcu

using namespace torch_gcu;

static c10::List<std::optional<at::Tensor>> to_index_list(const py::list& indices) {
  c10::List<std::optional<at::Tensor>> out;
  for (const auto& i : indices) {
    if (i.is_none()) out.push_back(std::nullopt);
    else out.push_back(i.cast<at::Tensor>());
  }
  return out;
}

PYBIND11_MODULE(_C, m) {
  register_runtime();
  init_tp_exchange_bindings(m);

  // ---- devices ---------------------------------------------------------------
  m.def("_gcu_getDeviceCount", [] { return static_cast<int>(device_count()); });
  m.def("_gcu_init", [] {
    TORCH_CHECK(device_count() > 0, "no gcu (B200) device is available");
    GCU_CUDA_CHECK(cudaFree(nullptr));
  });
  m.def("_gcu_getDevice", [] { return static_cast<int>(current_device()); });
  m.def("_gcu_setDevice", [](int d) { set_device(static_cast<c10::DeviceIndex>(d)); });
  m.def("_gcu_exchangeDevice", [](int d) { return static_cast<int>(d < 0 ? -1 : exchange_device(static_cast<c10::DeviceIndex>(d))); });
  m.def("_gcu_maybeExchangeDevice", [](int d) { return static_cast<int>(d < 0 ? -1 : exchange_device(static_cast<c10::DeviceIndex>(d))); });
  m.def("_gcu_synchronize", [] {
    py::gil_scoped_release nogil;
    device_synchronize();
  });
  m.def("_gcu_getDeviceProperties", [](int d) {
    cudaDeviceProp p;
    GCU_CUDA_CHECK(cudaGetDeviceProperties(&p, d));
    py::dict r;
    r["name"] = std::string(p.name);
    r["total_memory"] = static_cast<int64_t>(p.totalGlobalMem);
    r["multi_processor_count"] = p.multiProcessorCount;
    r["major"] = p.major;
    r["minor"] = p.minor;
    r["l2_cache_size"] = p.l2CacheSize;
    return r;
  });
  m.def("_gcu_memGetInfo", [](int d) {
    const c10::DeviceIndex prev = exchange_device(static_cast<c10::DeviceIndex>(d));
    size_t free_b = 0, total_b = 0;
    GCU_CUDA_CHECK(cudaMemGetInfo(&free_b, &total_b));
    if (prev != d) set_device(prev);
    return py::make_tuple(free_b, total_b);
  });

  // ---- streams (ids as torch.Stream carries them) ------------------------------
  m.def("_gcu_getCurrentStream", [](int d) {
    GCUStream s = getCurrentGCUStream(static_cast<c10::DeviceIndex>(d));
    return py::make_tuple(static_cast<int64_t>(s.id()), static_cast<int64_t>(s.device_index()),
                          static_cast<int64_t>(kGcuDeviceType));
  });
  m.def("_gcu_getDefaultStream", [](int d) {
    GCUStream s = getDefaultGCUStream(static_cast<c10::DeviceIndex>(d));
    return py::make_tuple(static_cast<int64_t>(s.id()), static_cast<int64_t>(s.device_index()),
                          static_cast<int64_t>(kGcuDeviceType));
  });
  m.def("_gcu_setStream", [](int64_t stream_id, int64_t device_index, int64_t) {
    setCurrentGCUStream(GCUStream(c10::Stream::unpack3(stream_id, static_cast<c10::DeviceIndex>(device_index), kGcuDeviceType)));
  });
  m.def("_gcu_getStreamFromExternal", [](uint64_t handle, int d) {
    GCUStream s = getStreamFromExternal(reinterpret_cast<cudaStream_t>(handle), static_cast<c10::DeviceIndex>(d));
    return py::make_tuple(static_cast<int64_t>(s.id()), static_cast<int64_t>(s.device_index()),
                          static_cast<int64_t>(kGcuDeviceType));
  });
  m.def("_gcu_streamHandle", [](int64_t stream_id, int64_t device_index) {
    GCUStream s(c10::Stream::unpack3(stream_id, static_cast<c10::DeviceIndex>(device_index), kGcuDeviceType));
    return reinterpret_cast<uint64_t>(s.stream());
  });
  m.def("_gcu_streamPriorityRange", [] { return GCUStream::priority_range(); });

  // ---- allocator ---------------------------------------------------------------
  m.def("_gcu_emptyCache", [] { GCUDeviceAllocator::get()->impl().empty_cache(); });
  m.def("_gcu_hostEmptyCache", [] { GCUHostAllocator::get()->empty_cache(); });
  m.def("_gcu_resetPeakMemoryStats", [](int d) { GCUDeviceAllocator::get()->impl().reset_peak_stats(d); });
  m.def("_gcu_memoryStats", [](int d) {
    DeviceStats s = GCUDeviceAllocator::get()->impl().stats(d);
    py::dict r;
    r["allocated_bytes.all.current"] = s.allocated_bytes;
    r["allocated_bytes.all.peak"] = s.allocated_bytes_peak;
    r["reserved_bytes.all.current"] = s.reserved_bytes;
    r["reserved_bytes.all.peak"] = s.reserved_bytes_peak;
    r["num_allocs"] = s.num_allocs;
    r["num_cache_hits"] = s.num_cache_hits;
    r["num_backend_allocs"] = s.num_backend_allocs;
    r["num_backend_frees"] = s.num_backend_frees;
    r["num_alloc_retries"] = s.num_alloc_retries;
    r["num_ooms"] = s.num_ooms;
    r["num_deferred_frees"] = s.num_deferred_frees;
    return r;
  });

  // ---- autocast accessors for the PrivateUse1 key (reference: InitGcuBindings.cpp:59-127)
  m.def("is_autocast_enabled", [] { return at::autocast::is_autocast_enabled(at::kPrivateUse1); });
  m.def("set_autocast_enabled", [](bool on) { at::autocast::set_autocast_enabled(at::kPrivateUse1, on); });
  m.def("get_autocast_dtype", [] {
    return py::reinterpret_borrow<py::object>(
        reinterpret_cast<PyObject*>(torch::getTHPDtype(at::autocast::get_autocast_dtype(at::kPrivateUse1))));
  });
  m.def("set_autocast_dtype", [](py::object dtype) {
    TORCH_CHECK(THPDtype_Check(dtype.ptr()), "dtype must be a torch.dtype");
    at::autocast::set_autocast_dtype(at::kPrivateUse1, reinterpret_cast<THPDtype*>(dtype.ptr())->scalar_type);
  });

  // ---- random ------------------------------------------------------------------
  m.def("_gcu_manualSeed", [](int d, uint64_t seed) {
    at::Generator g = default_generator(static_cast<c10::DeviceIndex>(d));
    std::lock_guard<std::mutex> lock(g.mutex());
    g.set_current_seed(seed);
  });
  m.def("_gcu_initialSeed", [](int d) { return default_generator(static_cast<c10::DeviceIndex>(d)).current_seed(); });

  // ---- efficient ops -------------------------------------------------------------
  m.def("_int32_indices_index", [](const at::Tensor& self, const py::list& indices) {
    return aotops::int32_indices_index(self, to_index_list(indices));
  });
  m.def("_rms_norm_residual", &aotops::rms_norm_residual, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("eps"));
  m.def("_rope", &aotops::rope, py::arg("x"), py::arg("cos"), py::arg("sin"), py::arg("positions") = py::none(),
        py::arg("inplace") = false);
  m.def("_swiglu", &aotops::swiglu);
  m.def("_swiglu_packed", &aotops::swiglu_packed);
  m.def("_linear_swiglu", &aotops::linear_swiglu);
  m.def("_linear_rope", &aotops::linear_rope);
  m.def("_rope_kv_append", &aotops::rope_kv_append, py::arg("qkv"), py::arg("cos"), py::arg("sin"), py::arg("positions"),
        py::arg("q_heads"), py::arg("k_cache"), py::arg("v_cache"));
  m.def("_sdpa_flash", &aotops::sdpa_flash, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("is_causal"),
        py::arg("scale") = py::none());

  // ---- debug ---------------------------------------------------------------------
  m.def("_set_op_sync_mode", &set_op_sync_mode);
  m.def("_get_op_sync_mode", &op_sync_mode);
  m.def("_device_error_fetch", [] {
    uint32_t f = 0;
    check_status(b200_device_error_fetch(&f), "b200_device_error_fetch");
    return f;
  });
  m.def("_kernel_library_version", [] { return std::string(b200_version()); });
  py::class_<GCUGraph>(m, "_GCUGraph")
      .def(py::init<>())
      .def("capture_begin", &GCUGraph::capture_begin)
      .def("capture_end", &GCUGraph::capture_end)
      .def("replay", &GCUGraph::replay, py::call_guard<py::gil_scoped_release>())
      .def("reset", &GCUGraph::reset)
      .def("captured", &GCUGraph::captured)
      .def("num_nodes", &GCUGraph::num_nodes);
  m.def("_gcu_isCurrentStreamCapturing", &current_stream_is_capturing);
  m.def("_kernel_launch_count", [] { return static_cast<uint64_t>(b200_launch_count()); });
  m.def("_set_reserved_sms", [](int n) { b200_set_reserved_sms(n); });
  m.def("_get_reserved_sms", [] { return b200_get_reserved_sms(); });

  m.def("_c10d_gcu_init", [m]() mutable {
    static bool done = false;
    if (!done) {
      init_distributed_bindings(m);
      done = true;
    }
    return true;
  });
}
