// Allocation, metadata and copy operators: the ones every model touches and
// that have no arithmetic (reference: torch_gcu/csrc/aten/aot_ops/
// gcu_empty_tensor.cpp:26-92,175-229, gcu_resize.cpp:13-130, gcu_tensor_shape.cpp:
// 52-199, gcu_copy.cpp:34-442, gcu_scalar.cpp:22-58, gcu_record_stream.cpp:10-22).
#include <ATen/EmptyTensor.h>
#include <ATen/ExpandUtils.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorFactories.h>
#include <ATen/ops/_reshape_alias_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/unfold_native.h>
#include <ATen/ops/view_native.h>
#include <c10/core/TensorOptions.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {

// ------------------------------------------------------------------ empty --
namespace aotops {

at::Tensor empty_memory_format(c10::IntArrayRef size, std::optional<at::ScalarType> dtype,
                               std::optional<at::Layout> layout, std::optional<at::Device> device,
                               std::optional<bool> pin_memory, std::optional<at::MemoryFormat> memory_format) {
  TORCH_CHECK(!pin_memory.value_or(false), "only dense CPU tensors can be pinned");
  TORCH_CHECK(layout.value_or(at::kStrided) == at::kStrided, "the gcu backend supports strided tensors only");
  const at::Device dev = device.value_or(gcu_device(current_device()));
  const c10::DeviceIndex idx = dev.has_index() ? dev.index() : current_device();
  const c10::DeviceIndex prev = exchange_device(idx);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  at::Tensor t = at::detail::empty_generic(size, GCUDeviceAllocator::get(), ks, dtype_or_default(dtype), memory_format);
  if (prev != idx) set_device(prev);
  return t;
}

at::Tensor empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride, std::optional<at::ScalarType> dtype,
                         std::optional<at::Layout> layout, std::optional<at::Device> device,
                         std::optional<bool> pin_memory) {
  TORCH_CHECK(!pin_memory.value_or(false), "only dense CPU tensors can be pinned");
  TORCH_CHECK(layout.value_or(at::kStrided) == at::kStrided, "the gcu backend supports strided tensors only");
  const at::Device dev = device.value_or(gcu_device(current_device()));
  const c10::DeviceIndex idx = dev.has_index() ? dev.index() : current_device();
  const c10::DeviceIndex prev = exchange_device(idx);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  at::Tensor t = at::detail::empty_strided_generic(size, stride, GCUDeviceAllocator::get(), ks, dtype_or_default(dtype));
  if (prev != idx) set_device(prev);
  return t;
}

}  // namespace aotops

// ----------------------------------------------------------------- resize --
// Growing a storage copies the old bytes device-to-device on the current stream
// (reference: gcu_resize.cpp:13-44).
void resize_storage_bytes(c10::StorageImpl* storage, size_t size_bytes) {
  TORCH_CHECK(storage->resizable(), "trying to resize a storage that is not resizable");
  if (size_bytes == 0) {
    storage->set_data_ptr_noswap(c10::DataPtr(nullptr, storage->device()));
    storage->set_nbytes(0);
    return;
  }
  const c10::DeviceIndex idx = storage->device().index();
  const c10::DeviceIndex prev = exchange_device(idx);
  c10::DataPtr fresh = GCUDeviceAllocator::get()->allocate(size_bytes);
  if (storage->data_ptr()) {
    const size_t keep = std::min(storage->nbytes(), size_bytes);
    GCU_CUDA_CHECK(cudaMemcpyAsync(fresh.get(), storage->data(), keep, cudaMemcpyDeviceToDevice,
                                   getCurrentGCUStream(idx).stream()));
  }
  storage->set_data_ptr_noswap(std::move(fresh));
  storage->set_nbytes(size_bytes);
  if (prev != idx) set_device(prev);
}

static void maybe_resize_storage(at::TensorImpl* self, size_t new_size_bytes) {
  if (self->numel() == 0) return;
  const c10::Storage& storage = self->unsafe_storage();
  TORCH_CHECK(storage, "Tensor: invalid null storage");
  if (new_size_bytes > storage.nbytes()) resize_storage_bytes(storage.unsafeGetStorageImpl(), new_size_bytes);
}

namespace aotops {

const at::Tensor& resize_(const at::Tensor& self, c10::IntArrayRef size, std::optional<at::MemoryFormat> memory_format) {
  at::TensorImpl* impl = self.unsafeGetTensorImpl();
  if (impl->sizes() != size) {
    const int64_t storage_offset = impl->storage_offset();
    impl->set_sizes_contiguous(size);
    const size_t need = (impl->numel() + storage_offset) * self.dtype().itemsize();
    maybe_resize_storage(impl, need);
  }
  if (memory_format.has_value() && *memory_format != at::MemoryFormat::Preserve)
    impl->empty_tensor_restride(*memory_format);
  return self;
}

at::Tensor& set__source_Storage_storage_offset(at::Tensor& result, at::Storage storage, int64_t storage_offset,
                                              c10::IntArrayRef size, c10::IntArrayRef stride) {
  at::native::checkSetStorage(result, std::move(storage), storage_offset, size, stride);
  at::TensorImpl* impl = result.unsafeGetTensorImpl();
  impl->set_storage_offset(storage_offset);
  at::OptionalIntArrayRef stride_opt = stride.data() != nullptr ? at::OptionalIntArrayRef(stride) : std::nullopt;
  if (stride_opt.has_value()) impl->set_sizes_and_strides(size, *stride_opt);
  else impl->set_sizes_contiguous(size);
  const size_t need = at::detail::computeStorageNbytes(impl->sizes(), impl->strides(), result.dtype().itemsize(), storage_offset);
  maybe_resize_storage(impl, need);
  return result;
}
at::Tensor& set__source_Storage(at::Tensor& result, at::Storage source) {
  const int64_t n = static_cast<int64_t>(source.nbytes() / result.dtype().itemsize());
  return set__source_Storage_storage_offset(result, std::move(source), 0, {n}, {});
}
at::Tensor& set__source_Tensor(at::Tensor& result, const at::Tensor& source) {
  if (result.unsafeGetTensorImpl() != source.unsafeGetTensorImpl())
    return set__source_Storage_storage_offset(result, source.storage(), source.storage_offset(), source.sizes(),
                                             source.strides());
  return result;
}
at::Tensor& set_(at::Tensor& result) {
  c10::Storage storage(c10::Storage::use_byte_size_t(), 0, GCUDeviceAllocator::get(), true);
  return set__source_Storage_storage_offset(result, std::move(storage), 0, {0}, {});
}

at::Tensor as_strided(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride,
                      std::optional<int64_t> storage_offset) {
  return at::native::as_strided_tensorimpl(self, size, stride, storage_offset);
}
at::Tensor view(const at::Tensor& self, c10::IntArrayRef size) { return at::native::view(self, size); }
at::Tensor _reshape_alias(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride) {
  return at::native::_reshape_alias(self, size, stride);
}
at::Tensor unfold(const at::Tensor& self, int64_t dim, int64_t size, int64_t step) {
  return at::native::unfold(self, dim, size, step);
}

// ------------------------------------------------------------------- copy --
// dst <- src, any pair of {cpu, gcu}; dtype cast and restriding run on the device.
static void device_copy(const at::Tensor& dst, const at::Tensor& src) {
  // same device: one kernel-library call on the source device's current stream
  c10::OptionalDeviceGuard g(src.device());
  at::Tensor s = src.sizes() == dst.sizes() ? src : src.expand(dst.sizes());
  b200Tensor vd = to_b200(dst), vs = to_b200(s);
  cudaStream_t stream = current_stream(dst);
  GCU_KERNEL_CALL(b200_copy, stream, &vd, &vs);
}

static void peer_copy(const at::Tensor& dst, const at::Tensor& src) {
  // different gcu devices: stage to a contiguous same-dtype buffer on the source
  // device, cudaMemcpyPeerAsync, then fix layout/dtype on the destination.
  at::Tensor s = src.expand(dst.sizes()).contiguous();
  at::Tensor stage = (dst.is_contiguous() && dst.dtype() == s.dtype()) ? dst : at::empty(dst.sizes(), s.options().device(dst.device()));
  const int sd = src.device().index(), dd = dst.device().index();
  cudaStream_t sstream = getCurrentGCUStream(sd).stream();
  {
    c10::OptionalDeviceGuard g(src.device());
    // order after pending work on the destination stream
    cudaEvent_t ev;
    {
      c10::OptionalDeviceGuard gd(dst.device());
      GCU_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      GCU_CUDA_CHECK(cudaEventRecord(ev, getCurrentGCUStream(dd).stream()));
    }
    GCU_CUDA_CHECK(cudaStreamWaitEvent(sstream, ev, 0));
    GCU_CUDA_CHECK(cudaMemcpyPeerAsync(stage.data_ptr(), dd, s.data_ptr(), sd, s.nbytes(), sstream));
    GCU_CUDA_CHECK(cudaEventRecord(ev, sstream));
    {
      c10::OptionalDeviceGuard gd(dst.device());
      GCU_CUDA_CHECK(cudaStreamWaitEvent(getCurrentGCUStream(dd).stream(), ev, 0));
    }
    GCU_CUDA_CHECK(cudaEventDestroy(ev));
  }
  GCUDeviceAllocator::get()->impl().record_stream(stage.data_ptr(), sstream);
  if (!stage.is_same(dst)) device_copy(dst, stage);
}

at::Tensor _copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  TORCH_CHECK(self.defined() && dst.defined(), "copy_: undefined tensor");
  if (dst.numel() == 0) return dst;
  if (self.is_same(dst)) return dst;
  const bool src_dev = self.device().is_privateuseone(), dst_dev = dst.device().is_privateuseone();
  TORCH_CHECK(src_dev || dst_dev, "_copy_from reached the gcu backend without a gcu tensor");
  TORCH_CHECK((src_dev || self.device().is_cpu()) && (dst_dev || dst.device().is_cpu()),
              "copies between gcu and ", src_dev ? dst.device() : self.device(), " are not supported");
  if (src_dev && dst_dev) {
    if (self.device() == dst.device()) device_copy(dst, self);
    else peer_copy(dst, self);
    return dst;
  }
  if (dst_dev) {
    // H2D: make the host side contiguous, same dtype; cast / restride on the device
    c10::OptionalDeviceGuard g(dst.device());
    const int idx = dst.device().index();
    cudaStream_t stream = getCurrentGCUStream(idx).stream();
    at::Tensor host = self.expand(dst.sizes()).contiguous();
    const bool direct = dst.is_contiguous() && dst.dtype() == host.dtype();
    at::Tensor target = direct ? dst : at::empty(dst.sizes(), host.options().device(dst.device()));
    const bool pinned = GCUHostAllocator::get()->is_pinned(host.data_ptr());
    GCU_CUDA_CHECK(cudaMemcpyAsync(target.data_ptr(), host.data_ptr(), host.nbytes(), cudaMemcpyHostToDevice, stream));
    if (non_blocking && pinned) GCUHostAllocator::get()->record_event(host.data_ptr(), stream);
    else GCU_CUDA_CHECK(cudaStreamSynchronize(stream));  // pageable or blocking: host buffer may go away
    if (!direct) device_copy(dst, target);
    return dst;
  }
  // D2H: cast / make contiguous on the device, then one copy
  c10::OptionalDeviceGuard g(self.device());
  const int idx = self.device().index();
  cudaStream_t stream = getCurrentGCUStream(idx).stream();
  at::Tensor dev = self.expand(dst.sizes());
  if (dev.dtype() != dst.dtype() || !dev.is_contiguous()) {
    at::Tensor tmp = at::empty(dst.sizes(), self.options().dtype(dst.scalar_type()));
    device_copy(tmp, dev);
    dev = tmp;
  }
  const bool direct = dst.is_contiguous();
  at::Tensor host = direct ? dst : at::empty(dst.sizes(), dst.options());
  GCU_CUDA_CHECK(cudaMemcpyAsync(host.data_ptr(), dev.data_ptr(), dev.nbytes(), cudaMemcpyDeviceToHost, stream));
  const bool pinned = GCUHostAllocator::get()->is_pinned(host.data_ptr());
  if (non_blocking && pinned && direct) GCUHostAllocator::get()->record_event(host.data_ptr(), stream);
  else GCU_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (!direct) dst.copy_(host);
  return dst;
}

at::Tensor _copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  at::native::resize_output(dst, self.sizes());
  return aotops::_copy_from(self, dst, false);
}

// 1-element D2H through pinned memory + stream sync (reference: gcu_scalar.cpp:22-58)
at::Scalar _local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  at::Tensor host = at::empty({}, self.options().device(at::kCPU));
  aotops::_copy_from(self.reshape({}), host, false);
  return host.item();
}

at::Tensor& fill__Scalar(at::Tensor& self, const at::Scalar& value) {
  if (self.numel() == 0) return self;
  c10::OptionalDeviceGuard g(self.device());
  b200Tensor v = to_b200(self);
  cudaStream_t stream = current_stream(self);
  if (self.scalar_type() == at::kLong && value.isIntegral(false)) {
    GCU_KERNEL_CALL(b200_fill_i64, stream, &v, value.toLong());   // exact beyond 2^53, where a double is not
    return self;
  }
  const double x = value.isBoolean() ? static_cast<double>(value.toBool()) : value.toDouble();
  GCU_KERNEL_CALL(b200_fill, stream, &v, x);
  return self;
}
at::Tensor& fill__Tensor(at::Tensor& self, const at::Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "fill_ only supports 0-dimension value tensor but got tensor with ", value.dim(), " dimensions.");
  return fill__Scalar(self, value.item());
}
at::Tensor& zero_(at::Tensor& self) { return fill__Scalar(self, 0); }

void record_stream(at::Tensor& self, c10::Stream s) {
  GCUDeviceAllocator::get()->record_stream(self.storage().data_ptr(), GCUStream(s).stream());
}

}  // namespace aotops
}  // namespace torch_gcu
