// Device guard, PrivateUse1 hooks and the Philox generator of the "gcu" backend
// (reference: torch_gcu/csrc/gcu/gcu_guard_impl.{h:17-99,cpp:99-206},
// gcu_hooks.{h:21-66,cpp:17-139}, gcu_generator_impl.{h,cpp}), over cudart.
#include <ATen/CPUGeneratorImpl.h>
#include <ATen/core/GeneratorForPrivateuseone.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>

#include <deque>
#include <mutex>

#include "runtime/gcu_allocator.h"
#include "runtime/gcu_runtime.h"

namespace torch_gcu {

// ------------------------------------------------------------- guard impl --
struct GCUGuardImpl final : public c10::impl::DeviceGuardImplInterface {
  static constexpr c10::DeviceType static_type = kGcuDeviceType;
  GCUGuardImpl() = default;
  explicit GCUGuardImpl(c10::DeviceType t) { TORCH_INTERNAL_ASSERT(t == kGcuDeviceType); }

  c10::DeviceType type() const override { return kGcuDeviceType; }
  c10::Device exchangeDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.is_privateuseone());
    return gcu_device(exchange_device(d.index()));
  }
  c10::Device getDevice() const override { return gcu_device(current_device()); }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.is_privateuseone());
    if (d.index() != current_device()) set_device(d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override { (void)cudaSetDevice(d.index()); }
  c10::Stream getStream(c10::Device d) const override { return getCurrentGCUStream(d.index()).unwrap(); }
  c10::Stream getDefaultStream(c10::Device d) const override { return getDefaultGCUStream(d.index()).unwrap(); }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool high = false) const override {
    return getStreamFromPool(high, d.index()).unwrap();
  }
  c10::Stream getNewStream(c10::Device d, int priority = 0) const override {
    return getStreamFromPool(priority, d.index()).unwrap();
  }
  c10::Stream exchangeStream(c10::Stream s) const override {
    GCUStream cs(s);
    c10::Stream old = getCurrentGCUStream(s.device_index()).unwrap();
    setCurrentGCUStream(cs);
    return old;
  }
  void* getStreamNativeHandle(const c10::Stream s) const override { return GCUStream(s).stream(); }
  c10::DeviceIndex deviceCount() const noexcept override { return device_count(); }

  // Events: created lazily on first record, always on the stream's device
  // (reference: gcu_guard_impl.cpp:99-145).
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag flag) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "event device ", device_index,
                " does not match the recording stream's device ", stream.device_index());
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    cudaEvent_t ev = static_cast<cudaEvent_t>(*event);
    if (!ev) {
      unsigned int f = cudaEventDisableTiming;
      if (flag == c10::EventFlag::BACKEND_DEFAULT) f = cudaEventDefault;  // timing enabled
      GCU_CUDA_CHECK(cudaEventCreateWithFlags(&ev, f));
      *event = ev;
    }
    GCU_CUDA_CHECK(cudaEventRecord(ev, GCUStream(stream).stream()));
    if (prev != stream.device_index()) set_device(prev);
  }
  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    GCU_CUDA_CHECK(cudaStreamWaitEvent(GCUStream(stream).stream(), static_cast<cudaEvent_t>(event), 0));
    if (prev != stream.device_index()) set_device(prev);
  }
  bool queryEvent(void* event) const override {
    if (!event) return true;
    cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (e == cudaErrorNotReady) {
      (void)cudaGetLastError();
      return false;
    }
    GCU_CUDA_CHECK(e);
    return true;
  }
  void destroyEvent(void* event, const c10::DeviceIndex) const noexcept override {
    if (event) (void)cudaEventDestroy(static_cast<cudaEvent_t>(event));
  }
  void synchronizeEvent(void* event) const override {
    if (event) GCU_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  }
  double elapsedTime(void* e1, void* e2, const c10::DeviceIndex) const override {
    TORCH_CHECK(e1 && e2, "both events must be recorded before elapsed_time");
    float ms = 0;
    GCU_CUDA_CHECK(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(e1), static_cast<cudaEvent_t>(e2)));
    return ms;
  }
  bool queryStream(const c10::Stream& s) const override { return GCUStream(s).query(); }
  void synchronizeStream(const c10::Stream& s) const override { GCUStream(s).synchronize(); }
  void synchronizeDevice(const c10::DeviceIndex idx) const override {
    const c10::DeviceIndex prev = exchange_device(idx);
    device_synchronize();
    if (prev != idx) set_device(prev);
  }
  void recordDataPtrOnStream(const c10::DataPtr& p, const c10::Stream& s) const override {
    GCUDeviceAllocator::get()->record_stream(p, GCUStream(s).stream());
  }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, GCUGuardImpl);

// -------------------------------------------------------------- generator --
// A CPU-seeded Philox-style generator object for the device: the ops on the hot
// path draw nothing, so it only has to carry seed/offset state for the
// torch.gcu.manual_seed / get_rng_state API.
struct GCUGeneratorImpl : public at::CPUGeneratorImpl {
  explicit GCUGeneratorImpl(c10::DeviceIndex idx) : at::CPUGeneratorImpl() {
    device_ = gcu_device(idx);
    key_set_ = c10::DispatchKeySet(c10::DispatchKey::PrivateUse1);
  }
};

namespace {
std::mutex g_gen_mutex;
std::deque<at::Generator> g_default_gens;
}  // namespace

const at::Generator& default_generator(c10::DeviceIndex idx) {
  std::lock_guard<std::mutex> g(g_gen_mutex);
  if (idx < 0) idx = device_count() > 0 ? current_device() : 0;
  while (static_cast<c10::DeviceIndex>(g_default_gens.size()) <= idx) {
    g_default_gens.push_back(at::make_generator<GCUGeneratorImpl>(static_cast<c10::DeviceIndex>(g_default_gens.size())));
    g_default_gens.back().seed();
  }
  return g_default_gens[idx];
}

at::Generator new_generator(c10::DeviceIndex idx) {
  if (idx < 0) idx = device_count() > 0 ? current_device() : 0;
  return at::make_generator<GCUGeneratorImpl>(idx);
}

// ------------------------------------------------------------------ hooks --
struct GCUHooks final : public at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return device_count() > 0; }
  bool hasPrimaryContext(c10::DeviceIndex idx) const override {
    unsigned int flags = 0;
    int active = 0;
    // cudart has no direct query; a device that was made current has a context
    (void)flags;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) (void)cudaGetLastError();
    active = (cur == idx);
    return active != 0;
  }
  void init() const override {
    TORCH_CHECK(device_count() > 0, "no gcu (B200) device is available");
    (void)cudaFree(nullptr);  // create the primary context of the current device
  }
  c10::DeviceIndex deviceCount() const override { return device_count(); }
  void setCurrentDevice(c10::DeviceIndex d) const override { set_device(d); }
  c10::DeviceIndex getCurrentDevice() const override { return current_device(); }
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex d) const override { return exchange_device(d); }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex d) const override { return exchange_device(d); }
  const at::Generator& getDefaultGenerator(c10::DeviceIndex idx) const override { return default_generator(idx); }
  at::Generator getNewGenerator(c10::DeviceIndex idx = -1) const override { return new_generator(idx); }
  at::Device getDeviceFromPtr(void* data) const override {
    cudaPointerAttributes attr;
    GCU_CUDA_CHECK(cudaPointerGetAttributes(&attr, data));
    TORCH_CHECK(attr.type == cudaMemoryTypeDevice, "the pointer is not device memory");
    return gcu_device(static_cast<c10::DeviceIndex>(attr.device));
  }
  bool isPinnedPtr(const void* data) const override { return GCUHostAllocator::get()->is_pinned(data); }
  c10::Allocator* getPinnedMemoryAllocator() const override { return GCUHostAllocator::get(); }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override;
};

void resize_storage_bytes(c10::StorageImpl* storage, size_t size_bytes);  // aten/gcu_empty_resize.cpp
void GCUHooks::resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const {
  resize_storage_bytes(storage.unsafeGetStorageImpl(), newsize);
}

void register_runtime() {
  static std::once_flag once;
  std::call_once(once, [] {
    c10::SetAllocator(kGcuDeviceType, GCUDeviceAllocator::get());
    at::RegisterPrivateUse1HooksInterface(new GCUHooks());
  });
}

}  // namespace torch_gcu
