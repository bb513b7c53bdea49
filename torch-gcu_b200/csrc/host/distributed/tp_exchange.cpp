// Peer-visible ("symmetric") device buffers and the Python bindings of the kernel library's
// tensor-parallel exchange (b200_tp_sync, b200_tp_reduce_norm).
//
// A symmetric buffer is one plain cudaMalloc allocation per rank whose IPC handle the ranks
// exchange through the c10d store (the Python side does the exchange); every rank then maps the
// others' allocations into its own address space (cudaIpcOpenMemHandle with lazy peer access),
// once, at set-up. The caching allocator is not involved: pool memory cannot be exported, and
// these buffers live as long as the process group does.
//
// The reference reaches peer memory only through its collective library (reference:
// torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:2270-2419 collective<>); this file is what lets
// this backend's own kernels do the exchange instead.
#include <torch/csrc/utils/pybind.h>

#include "aten/bridge.h"
#include "runtime/gcu_runtime.h"

namespace torch_gcu {
namespace {

at::Tensor wrap_bytes(void* ptr, int64_t nbytes, c10::DeviceIndex device, std::function<void(void*)> deleter) {
  const c10::Device dev(c10::DeviceType::PrivateUse1, device);
  return at::for_blob(ptr, {nbytes})
      .deleter(std::move(deleter))
      .options(at::TensorOptions().dtype(at::kByte).device(dev))
      .target_device(dev)
      .make_tensor();
}

// (uint8 tensor over a fresh zeroed allocation on the current device, its IPC handle)
std::pair<at::Tensor, py::bytes> symm_alloc(int64_t nbytes) {
  TORCH_CHECK(nbytes > 0, "symmetric buffer: nbytes must be positive");
  const c10::DeviceIndex device = current_device();
  void* p = nullptr;
  GCU_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(nbytes)));
  GCU_CUDA_CHECK(cudaMemset(p, 0, static_cast<size_t>(nbytes)));
  GCU_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaFree(p);
    TORCH_CHECK(false, "symmetric buffer: cudaIpcGetMemHandle failed: ", cudaGetErrorString(e));
  }
  at::Tensor t = wrap_bytes(p, nbytes, device, [](void* q) { (void)cudaFree(q); });
  return {t, py::bytes(reinterpret_cast<const char*>(&h), sizeof(h))};
}

// Maps another rank's allocation (its handle as published) into this process, on the current device.
at::Tensor symm_open(const std::string& handle, int64_t nbytes) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "symmetric buffer: malformed IPC handle");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  TORCH_CHECK(e == cudaSuccess && p, "symmetric buffer: cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e),
              " (peer access between the two devices is required)");
  return wrap_bytes(p, nbytes, current_device(), [](void* q) { (void)cudaIpcCloseMemHandle(q); });
}

// Table of one buffer per rank, each at `offset` bytes into that rank's symmetric allocation.
b200TpPeers peer_table(const std::vector<at::Tensor>& buffers, int64_t rank, int64_t offset) {
  TORCH_CHECK(!buffers.empty() && buffers.size() <= B200_TP_MAX_RANKS, "tensor-parallel exchange: 1 to ", B200_TP_MAX_RANKS, " ranks");
  TORCH_CHECK(rank >= 0 && rank < static_cast<int64_t>(buffers.size()), "tensor-parallel exchange: rank out of range");
  b200TpPeers t{};
  t.world = static_cast<int32_t>(buffers.size());
  t.rank = static_cast<int32_t>(rank);
  for (size_t r = 0; r < buffers.size(); ++r) {
    const at::Tensor& b = buffers[r];
    TORCH_CHECK(b.device().is_privateuseone() && b.scalar_type() == at::kByte && b.is_contiguous(),
                "tensor-parallel exchange: the symmetric buffers are contiguous uint8 gcu tensors");
    TORCH_CHECK(offset >= 0 && offset < b.numel(), "tensor-parallel exchange: offset outside the buffer");
    t.base[r] = static_cast<char*>(b.data_ptr()) + offset;
  }
  return t;
}

}  // namespace

void init_tp_exchange_bindings(py::module& m) {
  m.def("_symm_alloc", &symm_alloc, py::arg("nbytes"));
  m.def("_symm_open", &symm_open, py::arg("handle"), py::arg("nbytes"));
  m.def("_tp_control_bytes", [] { return static_cast<int64_t>(b200_tp_control_bytes()); });
  m.def(
      "_tp_sync",
      [](const std::vector<at::Tensor>& buffers, int64_t rank, int64_t control_offset, int64_t channel, bool do_signal,
         bool do_wait, double timeout_s) {
        const b200TpPeers ctl = peer_table(buffers, rank, control_offset);
        cudaStream_t stream = current_stream(buffers[static_cast<size_t>(rank)]);
        GCU_KERNEL_CALL(b200_tp_sync, stream, &ctl, static_cast<int32_t>(channel), do_signal ? 1 : 0, do_wait ? 1 : 0,
                        static_cast<uint64_t>(timeout_s * 1e9));
      },
      py::arg("buffers"), py::arg("rank"), py::arg("control_offset"), py::arg("channel"), py::arg("signal"), py::arg("wait"),
      py::arg("timeout_s"));
  m.def(
      "_tp_reduce_norm",
      [](const std::vector<at::Tensor>& buffers, int64_t rank, std::optional<int64_t> partial_offset, int64_t gathered_offset,
         const std::optional<at::Tensor>& residual, const std::optional<at::Tensor>& residual_out,
         const std::optional<at::Tensor>& weight, int64_t row0, int64_t total_rows, double eps, bool normalise, bool gather_all) {
        const b200TpPeers gathered = peer_table(buffers, rank, gathered_offset);
        b200TpPeers partial{};
        if (partial_offset.has_value()) partial = peer_table(buffers, rank, *partial_offset);
        b200Tensor vr{}, vo{}, vw{};
        if (residual.has_value()) vr = to_b200(*residual);
        if (residual_out.has_value()) vo = to_b200(*residual_out);
        if (weight.has_value()) vw = to_b200(*weight);
        cudaStream_t stream = current_stream(buffers[static_cast<size_t>(rank)]);
        GCU_KERNEL_CALL(b200_tp_reduce_norm, stream, partial_offset.has_value() ? &partial : nullptr, &gathered,
                        residual.has_value() ? &vr : nullptr, residual_out.has_value() ? &vo : nullptr,
                        weight.has_value() ? &vw : nullptr, row0, total_rows, eps, normalise ? 1 : 0, gather_all ? 1 : 0);
      },
      py::arg("buffers"), py::arg("rank"), py::arg("partial_offset"), py::arg("gathered_offset"), py::arg("residual"),
      py::arg("residual_out"), py::arg("weight"), py::arg("row0"), py::arg("total_rows"), py::arg("eps"), py::arg("normalise"),
      py::arg("gather_all"));
}

}  // namespace torch_gcu
