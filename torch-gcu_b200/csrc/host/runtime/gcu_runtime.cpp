#include "runtime/gcu_runtime.h"

#include <array>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace torch_gcu {

// ------------------------------------------------------------------ devices --
c10::DeviceIndex device_count() {
  static const int n = [] {
    int c = 0;
    if (cudaGetDeviceCount(&c) != cudaSuccess) {
      (void)cudaGetLastError();
      c = 0;
    }
    return c;
  }();
  return static_cast<c10::DeviceIndex>(n);
}

c10::DeviceIndex current_device() {
  int d = 0;
  GCU_CUDA_CHECK(cudaGetDevice(&d));
  return static_cast<c10::DeviceIndex>(d);
}

void set_device(c10::DeviceIndex index) {
  TORCH_CHECK(index >= 0 && index < device_count(), "invalid gcu device index ", static_cast<int>(index),
              " (", static_cast<int>(device_count()), " devices)");
  GCU_CUDA_CHECK(cudaSetDevice(index));
}

c10::DeviceIndex exchange_device(c10::DeviceIndex index) {
  const c10::DeviceIndex cur = current_device();
  if (index >= 0 && index != cur) set_device(index);
  return cur;
}

void device_synchronize() { GCU_CUDA_CHECK(cudaDeviceSynchronize()); }

// ------------------------------------------------------------------ streams --
namespace {

constexpr int kMaxDevices = 64;

struct DevicePools {
  std::once_flag once;
  std::array<cudaStream_t, kStreamsPerPool> low{};
  std::array<cudaStream_t, kStreamsPerPool> high{};
  std::atomic<uint32_t> next_low{0}, next_high{0};
  int least_prio = 0, greatest_prio = 0;
};

DevicePools& pools(c10::DeviceIndex d) {
  static std::array<DevicePools, kMaxDevices> all;
  TORCH_CHECK(d >= 0 && d < kMaxDevices, "gcu device index out of range");
  return all[d];
}

void init_pools(c10::DeviceIndex d) {
  DevicePools& p = pools(d);
  std::call_once(p.once, [&] {
    const c10::DeviceIndex prev = exchange_device(d);
    GCU_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&p.least_prio, &p.greatest_prio));
    for (int i = 0; i < kStreamsPerPool; ++i) {
      GCU_CUDA_CHECK(cudaStreamCreateWithPriority(&p.low[i], cudaStreamNonBlocking, p.least_prio));
      GCU_CUDA_CHECK(cudaStreamCreateWithPriority(&p.high[i], cudaStreamNonBlocking, p.greatest_prio));
    }
    if (prev != d) set_device(prev);
  });
}

std::mutex g_ext_mutex;
std::unordered_map<c10::StreamId, cudaStream_t> g_ext_streams;  // id -> handle
c10::StreamId g_ext_next = kExternalBase;

// Current stream ids, thread-local per device; 0 = default stream.
thread_local std::array<c10::StreamId, kMaxDevices> tl_current{};

std::atomic<bool> g_op_sync{false};

c10::DeviceIndex resolve(c10::DeviceIndex d) { return d < 0 ? current_device() : d; }

c10::Stream make_stream(c10::DeviceIndex d, c10::StreamId id) {
  return c10::Stream(c10::Stream::UNSAFE, gcu_device(d), id);
}

}  // namespace

cudaStream_t GCUStream::stream() const {
  const c10::StreamId id = stream_.id();
  if (id == 0) return nullptr;  // legacy default stream
  if (id >= kExternalBase) {
    std::lock_guard<std::mutex> g(g_ext_mutex);
    auto it = g_ext_streams.find(id);
    TORCH_CHECK(it != g_ext_streams.end(), "unknown external gcu stream id ", id);
    return it->second;
  }
  TORCH_CHECK(id >= 1 && id <= 2 * kStreamsPerPool, "invalid gcu stream id ", id);
  init_pools(device_index());
  DevicePools& p = pools(device_index());
  return id <= kStreamsPerPool ? p.low[id - 1] : p.high[id - 1 - kStreamsPerPool];
}

bool GCUStream::query() const {
  const c10::DeviceIndex prev = exchange_device(device_index());
  cudaError_t e = cudaStreamQuery(stream());
  if (prev != device_index()) set_device(prev);
  if (e == cudaSuccess) return true;
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return false;
  }
  GCU_CUDA_CHECK(e);
  return false;
}

void GCUStream::synchronize() const {
  const c10::DeviceIndex prev = exchange_device(device_index());
  GCU_CUDA_CHECK(cudaStreamSynchronize(stream()));
  if (prev != device_index()) set_device(prev);
}

int GCUStream::priority() const {
  const c10::StreamId id = stream_.id();
  if (id > kStreamsPerPool && id <= 2 * kStreamsPerPool) return -1;  // high priority, as torch numbers it
  return 0;
}

std::tuple<int, int> GCUStream::priority_range() {
  int least = 0, greatest = 0;
  GCU_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  return std::make_tuple(least, greatest);
}

GCUStream getStreamFromPool(bool high_priority, c10::DeviceIndex device) {
  const c10::DeviceIndex d = resolve(device);
  init_pools(d);
  DevicePools& p = pools(d);
  const uint32_t i = (high_priority ? p.next_high : p.next_low).fetch_add(1) % kStreamsPerPool;
  return GCUStream(GCUStream::UNCHECKED, make_stream(d, 1 + (high_priority ? kStreamsPerPool : 0) + i));
}

GCUStream getStreamFromPool(int priority, c10::DeviceIndex device) { return getStreamFromPool(priority < 0, device); }

GCUStream getStreamFromExternal(cudaStream_t ext, c10::DeviceIndex device) {
  if (ext == nullptr) return getDefaultGCUStream(device);
  std::lock_guard<std::mutex> g(g_ext_mutex);
  for (auto& kv : g_ext_streams)
    if (kv.second == ext) return GCUStream(GCUStream::UNCHECKED, make_stream(resolve(device), kv.first));
  const c10::StreamId id = g_ext_next++;
  g_ext_streams[id] = ext;
  return GCUStream(GCUStream::UNCHECKED, make_stream(resolve(device), id));
}

GCUStream getDefaultGCUStream(c10::DeviceIndex device) {
  return GCUStream(GCUStream::UNCHECKED, make_stream(resolve(device), 0));
}

GCUStream getCurrentGCUStream(c10::DeviceIndex device) {
  const c10::DeviceIndex d = resolve(device);
  TORCH_CHECK(d < kMaxDevices, "gcu device index out of range");
  return GCUStream(GCUStream::UNCHECKED, make_stream(d, tl_current[d]));
}

void setCurrentGCUStream(GCUStream stream) {
  const c10::DeviceIndex d = stream.device_index();
  TORCH_CHECK(d >= 0 && d < kMaxDevices, "gcu device index out of range");
  tl_current[d] = stream.id();
}

void set_op_sync_mode(bool on) { g_op_sync.store(on); }
bool op_sync_mode() {
  static std::once_flag once;
  std::call_once(once, [] {
    // ENFLAME_PT_OP_DEBUG_CONFIG="op_sync_mode=true ..." (reference: op_debug_config.cpp:25-118)
    const char* cfg = std::getenv("ENFLAME_PT_OP_DEBUG_CONFIG");
    if (cfg && std::strstr(cfg, "op_sync_mode=true")) g_op_sync.store(true);
  });
  return g_op_sync.load();
}
void maybe_stream_synchronize(cudaStream_t stream) {
  if (op_sync_mode()) GCU_CUDA_CHECK(cudaStreamSynchronize(stream));
}

}  // namespace torch_gcu
