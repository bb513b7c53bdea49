// Device runtime of the PrivateUse1 ("gcu") backend over the CUDA runtime:
// device selection, the stream pool, events. It keeps the surface of the
// reference's csrc/gcu layer (reference: torch_gcu/csrc/gcu/gcu_functions.cpp,
// gcu_stream.{h,cpp}, gcu_event.h) with cudart underneath instead of the vendor
// runtime.
#pragma once

#include <c10/core/Device.h>
#include <c10/core/Stream.h>
#include <c10/util/Exception.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <tuple>

namespace torch_gcu {

constexpr c10::DeviceType kGcuDeviceType = c10::DeviceType::PrivateUse1;

#define GCU_CUDA_CHECK(EXPR)                                                                   \
  do {                                                                                         \
    cudaError_t _e = (EXPR);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      (void)cudaGetLastError();                                                                \
      TORCH_CHECK(false, "GCU(B200) runtime error: ", cudaGetErrorString(_e), " at ", __FILE__, ":", __LINE__); \
    }                                                                                          \
  } while (0)

// ---- devices (reference: gcu_functions.cpp:176-252) -------------------------
// device_count never throws: no driver / no GPU gives 0.
c10::DeviceIndex device_count();
c10::DeviceIndex current_device();
void set_device(c10::DeviceIndex index);
// Sets the device only when it differs; returns the previous one.
c10::DeviceIndex exchange_device(c10::DeviceIndex index);
void device_synchronize();
inline c10::Device gcu_device(c10::DeviceIndex i) { return c10::Device(kGcuDeviceType, i); }

// ---- streams (reference: gcu_stream.h:66-148, gcu_stream.cpp:240-291) --------
// Value wrapper around c10::Stream that knows how to reach the cudaStream_t.
// Stream ids: 0 = the device's default (legacy null) stream; 1..32 = normal-
// priority pool; 33..64 = high-priority pool; >= kExternalBase = streams created
// elsewhere and registered with getStreamFromExternal.
class GCUStream {
 public:
  enum Unchecked { UNCHECKED };
  explicit GCUStream(c10::Stream stream) : stream_(stream) {
    TORCH_CHECK(stream_.device_type() == kGcuDeviceType, "expected a gcu stream, got ", stream_);
  }
  explicit GCUStream(Unchecked, c10::Stream stream) : stream_(stream) {}
  bool operator==(const GCUStream& o) const noexcept { return stream_ == o.stream_; }
  bool operator!=(const GCUStream& o) const noexcept { return stream_ != o.stream_; }
  operator cudaStream_t() const { return stream(); }
  operator c10::Stream() const { return stream_; }
  c10::DeviceType device_type() const { return kGcuDeviceType; }
  c10::DeviceIndex device_index() const { return stream_.device_index(); }
  c10::Device device() const { return gcu_device(device_index()); }
  c10::StreamId id() const { return stream_.id(); }
  bool query() const;
  void synchronize() const;
  int priority() const;
  cudaStream_t stream() const;
  c10::Stream unwrap() const { return stream_; }
  static std::tuple<int, int> priority_range();  // (least, greatest) as cudart reports them

 private:
  c10::Stream stream_;
};

constexpr int kStreamsPerPool = 32;
constexpr c10::StreamId kExternalBase = 1 << 20;

GCUStream getStreamFromPool(bool high_priority = false, c10::DeviceIndex device = -1);
GCUStream getStreamFromPool(int priority, c10::DeviceIndex device = -1);
GCUStream getStreamFromExternal(cudaStream_t ext, c10::DeviceIndex device);
GCUStream getDefaultGCUStream(c10::DeviceIndex device = -1);
GCUStream getCurrentGCUStream(c10::DeviceIndex device = -1);  // thread-local per device
void setCurrentGCUStream(GCUStream stream);
// Synchronises the stream when the op_sync_mode debug switch is on
// (reference: maybeGCUStreamSynchronize, gcu_stream.cpp:382-386).
void maybe_stream_synchronize(cudaStream_t stream);
void set_op_sync_mode(bool on);
bool op_sync_mode();

}  // namespace torch_gcu
