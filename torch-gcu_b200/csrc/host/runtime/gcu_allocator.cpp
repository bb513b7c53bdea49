#include "runtime/gcu_allocator.h"

#include <c10/util/Exception.h>

#include <algorithm>
#include <cstring>
#include <limits>

#include "runtime/gcu_runtime.h"

namespace torch_gcu {

// ------------------------------------------------------------ CUDA backend --
namespace {

class CudaBackend final : public MemoryBackend {
 public:
  void* alloc(int device, size_t bytes, cudaStream_t stream) override {
    ensure_pool(device);
    DeviceSwitch sw(device);
    void* p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, bytes, stream);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      if (e == cudaErrorMemoryAllocation) return nullptr;
      TORCH_CHECK(false, "cudaMallocAsync failed: ", cudaGetErrorString(e));
    }
    return p;
  }
  void free(int device, void* ptr, cudaStream_t stream) override {
    DeviceSwitch sw(device);
    cudaError_t e = cudaFreeAsync(ptr, stream);
    if (e != cudaSuccess) (void)cudaGetLastError();  // teardown after the context is gone: ignore
  }
  void* record_event(int device, cudaStream_t stream) override {
    DeviceSwitch sw(device);
    cudaEvent_t ev;
    GCU_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    GCU_CUDA_CHECK(cudaEventRecord(ev, stream));
    return ev;
  }
  bool event_done(void* event) override {
    cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (e == cudaErrorNotReady) {
      (void)cudaGetLastError();
      return false;
    }
    if (e != cudaSuccess) (void)cudaGetLastError();
    // anything but success keeps the block parked: an event that cannot be queried (recorded on a
    // capturing stream, a lost context) is no proof that the other stream is done with the memory
    return e == cudaSuccess;
  }
  void destroy_event(void* event) override { (void)cudaEventDestroy(static_cast<cudaEvent_t>(event)); }
  void synchronize(int device) override {
    DeviceSwitch sw(device);
    (void)cudaDeviceSynchronize();
  }
  void* alloc_plain(int device, size_t bytes) override {
    DeviceSwitch sw(device);
    // cudaMalloc is refused on a capturing thread unless the thread's capture mode is relaxed
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    (void)cudaThreadExchangeStreamCaptureMode(&mode);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    (void)cudaThreadExchangeStreamCaptureMode(&mode);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      if (e == cudaErrorMemoryAllocation) return nullptr;
      TORCH_CHECK(false, "cudaMalloc failed: ", cudaGetErrorString(e));
    }
    return p;
  }
  void free_plain(int device, void* ptr) override {
    DeviceSwitch sw(device);
    if (cudaFree(ptr) != cudaSuccess) (void)cudaGetLastError();
  }
  bool stream_is_capturing(cudaStream_t stream) override {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    return st == cudaStreamCaptureStatusActive;
  }

 private:
  struct DeviceSwitch {
    int prev = -1, want;
    explicit DeviceSwitch(int d) : want(d) {
      if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
      if (prev != want) (void)cudaSetDevice(want);
    }
    ~DeviceSwitch() {
      if (prev >= 0 && prev != want) (void)cudaSetDevice(prev);
    }
  };
  void ensure_pool(int device) {
    std::lock_guard<std::mutex> g(m_);
    if (device < static_cast<int>(ready_.size()) && ready_[device]) return;
    if (device >= static_cast<int>(ready_.size())) ready_.resize(device + 1, false);
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
      uint64_t keep = std::numeric_limits<uint64_t>::max();  // never trim behind our back
      (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    } else {
      (void)cudaGetLastError();
    }
    ready_[device] = true;
  }
  std::mutex m_;
  std::vector<bool> ready_;
};

}  // namespace

std::unique_ptr<MemoryBackend> make_cuda_backend() { return std::make_unique<CudaBackend>(); }

// -------------------------------------------------------------- allocator --
StreamOrderedCachingAllocator::StreamOrderedCachingAllocator(std::unique_ptr<MemoryBackend> backend)
    : backend_(std::move(backend)) {}

StreamOrderedCachingAllocator::~StreamOrderedCachingAllocator() {
  // Process teardown: the driver reclaims everything; touching it now may run
  // after the context is destroyed.
}

size_t StreamOrderedCachingAllocator::round_size(size_t bytes) {
  constexpr size_t kSmall = 512, kLargeStep = 2u << 20, kSmallLimit = 1u << 20;
  if (bytes <= kSmallLimit) return (bytes + kSmall - 1) / kSmall * kSmall;
  return (bytes + kLargeStep - 1) / kLargeStep * kLargeStep;
}

StreamOrderedCachingAllocator::PerDevice& StreamOrderedCachingAllocator::dev(int device) { return devices_[device]; }

void StreamOrderedCachingAllocator::process_pending_locked() {
  if (capturing_.empty() && !parked_.empty()) {
    for (Block* b : parked_) record_deferred_locked(b);
    parked_.clear();
  }
  while (!pending_.empty()) {
    auto [event, block] = pending_.front();
    if (!backend_->event_done(event)) break;
    backend_->destroy_event(event);
    pending_.pop_front();
    if (--block->pending_events == 0) {
      block->other_streams.clear();
      dev(block->device).cache.emplace(Key(block->stream, block->size), block);
    }
  }
}

void StreamOrderedCachingAllocator::release_cached_locked(int device) {
  PerDevice& d = dev(device);
  for (auto& kv : d.cache) {
    Block* b = kv.second;
    backend_->free(device, b->ptr, b->stream);
    d.stats.reserved_bytes -= static_cast<int64_t>(b->size);
    d.stats.num_backend_frees++;
    delete b;
  }
  d.cache.clear();
}

void* StreamOrderedCachingAllocator::malloc(int device, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) return nullptr;
  const size_t size = round_size(bytes);
  std::lock_guard<std::mutex> g(mutex_);
  if (capturing_.empty()) process_pending_locked();   // event queries are not legal while a capture is open
  PerDevice& d = dev(device);
  d.stats.num_allocs++;
  Block* block = nullptr;
  auto cap = capturing_.find({device, stream});
  if (cap == capturing_.end() && !capturing_.empty() && backend_->stream_is_capturing(stream)) {
    // a side stream that joined a capture (it waited on an event of the capturing stream): its allocations
    // belong to that capture's pool too, never to the stream-ordered cache that eager code shares
    for (auto it = capturing_.begin(); it != capturing_.end(); ++it)
      if (it->first.first == device) {
        cap = it;
        break;
      }
  }
  if (cap != capturing_.end()) {
    Pool& pool = pools_[cap->second];
    // reuse inside the pool only along one stream: two streams of a graph are parallel branches, and nothing
    // orders a block freed on one of them before its next use on the other
    auto pit = pool.cache.lower_bound(size);
    while (pit != pool.cache.end() && pit->first <= size + size / 4 && pit->second->stream != stream) ++pit;
    if (pit != pool.cache.end() && pit->first <= size + size / 4) {
      block = pit->second;
      pool.cache.erase(pit);
      d.stats.num_cache_hits++;
    } else {
      void* p = backend_->alloc_plain(device, size);
      if (!p) {
        d.stats.num_ooms++;
        TORCH_CHECK_WITH(OutOfMemoryError, false, "GCU(B200) out of memory during graph capture: tried to allocate ", size,
                         " bytes on device ", device);
      }
      d.stats.num_backend_allocs++;
      d.stats.reserved_bytes += static_cast<int64_t>(size);
      d.stats.reserved_bytes_peak = std::max(d.stats.reserved_bytes_peak, d.stats.reserved_bytes);
      block = new Block{p, size, device, stream, {}, 0, cap->second};
    }
    pool.live++;
    d.stats.allocated_bytes += static_cast<int64_t>(block->size);
    d.stats.allocated_bytes_peak = std::max(d.stats.allocated_bytes_peak, d.stats.allocated_bytes);
    live_[block->ptr] = block;
    return block->ptr;
  }
  auto it = d.cache.lower_bound(Key(stream, size));
  if (it != d.cache.end() && it->first.first == stream && it->first.second <= size + size / 4) {
    block = it->second;
    d.cache.erase(it);
    d.stats.num_cache_hits++;
  } else {
    void* p = backend_->alloc(device, size, stream);
    if (!p) {
      // give the backend its memory back and try once more
      d.stats.num_alloc_retries++;
      release_cached_locked(device);
      backend_->synchronize(device);
      process_pending_locked();
      release_cached_locked(device);
      p = backend_->alloc(device, size, stream);
    }
    if (!p) {
      d.stats.num_ooms++;
      TORCH_CHECK_WITH(OutOfMemoryError, false, "GCU(B200) out of memory: tried to allocate ", size,
                       " bytes on device ", device, " (", d.stats.allocated_bytes, " bytes allocated, ",
                       d.stats.reserved_bytes, " reserved)");
    }
    d.stats.num_backend_allocs++;
    d.stats.reserved_bytes += static_cast<int64_t>(size);
    d.stats.reserved_bytes_peak = std::max(d.stats.reserved_bytes_peak, d.stats.reserved_bytes);
    block = new Block{p, size, device, stream, {}, 0, 0};
  }
  d.stats.allocated_bytes += static_cast<int64_t>(block->size);
  d.stats.allocated_bytes_peak = std::max(d.stats.allocated_bytes_peak, d.stats.allocated_bytes);
  live_[block->ptr] = block;
  return block->ptr;
}

void StreamOrderedCachingAllocator::free(void* ptr) {
  if (!ptr) return;
  std::lock_guard<std::mutex> g(mutex_);
  auto it = live_.find(ptr);
  TORCH_CHECK(it != live_.end(), "gcu allocator: freeing a pointer it does not own");
  Block* b = it->second;
  live_.erase(it);
  PerDevice& d = dev(b->device);
  d.stats.allocated_bytes -= static_cast<int64_t>(b->size);
  if (b->pool != 0) {
    // a capture pool's block: order inside the graph is fixed by the captured dependencies,
    // so no events; it stays with its pool until the graph is gone
    Pool& pool = pools_[b->pool];
    pool.live--;
    b->other_streams.clear();
    if (pool.released) {
      const uint64_t pool_id = b->pool;        // read before the block (and then the pool) go away
      const bool last = pool.live == 0;
      backend_->free_plain(b->device, b->ptr);
      d.stats.reserved_bytes -= static_cast<int64_t>(b->size);
      d.stats.num_backend_frees++;
      delete b;
      if (last) pools_.erase(pool_id);
    } else {
      pool.cache.emplace(b->size, b);
    }
    return;
  }
  if (b->other_streams.empty()) {
    d.cache.emplace(Key(b->stream, b->size), b);
  } else {
    // other streams may still be using the block: wait for events recorded on them now
    d.stats.num_deferred_frees++;
    if (!capturing_.empty()) {
      // an event recorded now could land inside a capture and never become queryable: park the
      // block and record its events when no capture is open any more
      parked_.push_back(b);
      return;
    }
    record_deferred_locked(b);
  }
}

void StreamOrderedCachingAllocator::record_deferred_locked(Block* b) {
  for (cudaStream_t s : b->other_streams) {
    pending_.emplace_back(backend_->record_event(b->device, s), b);
    b->pending_events++;
  }
}

void StreamOrderedCachingAllocator::record_stream(void* ptr, cudaStream_t stream) {
  if (!ptr) return;
  std::lock_guard<std::mutex> g(mutex_);
  auto it = live_.find(ptr);
  if (it == live_.end()) return;  // not ours (e.g. an external buffer)
  Block* b = it->second;
  if (stream == b->stream) return;
  if (std::find(b->other_streams.begin(), b->other_streams.end(), stream) == b->other_streams.end())
    b->other_streams.push_back(stream);
}

uint64_t StreamOrderedCachingAllocator::begin_capture(int device, cudaStream_t stream) {
  std::lock_guard<std::mutex> g(mutex_);
  TORCH_CHECK(capturing_.find({device, stream}) == capturing_.end(), "gcu allocator: this stream is already capturing");
  const uint64_t id = next_pool_++;
  pools_[id].device = device;
  capturing_[{device, stream}] = id;
  return id;
}

void StreamOrderedCachingAllocator::end_capture(int device, cudaStream_t stream) {
  std::lock_guard<std::mutex> g(mutex_);
  capturing_.erase({device, stream});
  if (capturing_.empty()) process_pending_locked();   // blocks parked during the capture get their events now
}

void StreamOrderedCachingAllocator::release_pool(uint64_t id) {
  std::lock_guard<std::mutex> g(mutex_);
  auto it = pools_.find(id);
  if (it == pools_.end()) return;
  Pool& pool = it->second;
  PerDevice& d = dev(pool.device);
  for (auto& kv : pool.cache) {
    Block* b = kv.second;
    backend_->free_plain(b->device, b->ptr);
    d.stats.reserved_bytes -= static_cast<int64_t>(b->size);
    d.stats.num_backend_frees++;
    delete b;
  }
  pool.cache.clear();
  pool.released = true;   // blocks still held by tensors are returned as those tensors die
  if (pool.live == 0) pools_.erase(it);
}

void StreamOrderedCachingAllocator::empty_cache() {
  std::lock_guard<std::mutex> g(mutex_);
  process_pending_locked();
  for (auto& kv : devices_) release_cached_locked(kv.first);
}

DeviceStats StreamOrderedCachingAllocator::stats(int device) {
  std::lock_guard<std::mutex> g(mutex_);
  return dev(device).stats;
}

void StreamOrderedCachingAllocator::reset_peak_stats(int device) {
  std::lock_guard<std::mutex> g(mutex_);
  DeviceStats& s = dev(device).stats;
  s.allocated_bytes_peak = s.allocated_bytes;
  s.reserved_bytes_peak = s.reserved_bytes;
}

// --------------------------------------------------- c10 device allocator --
namespace {
StreamOrderedCachingAllocator* device_impl() {
  static StreamOrderedCachingAllocator* a = new StreamOrderedCachingAllocator(make_cuda_backend());  // leaked on purpose
  return a;
}
void device_deleter(void* ptr) { device_impl()->free(ptr); }
}  // namespace

GCUDeviceAllocator* GCUDeviceAllocator::get() {
  static GCUDeviceAllocator a;
  return &a;
}
StreamOrderedCachingAllocator& GCUDeviceAllocator::impl() { return *device_impl(); }

c10::DataPtr GCUDeviceAllocator::allocate(size_t nbytes) {
  const c10::DeviceIndex d = current_device();
  void* p = nullptr;
  if (nbytes > 0) p = device_impl()->malloc(d, nbytes, getCurrentGCUStream(d).stream());
  return {p, p, &device_deleter, gcu_device(d)};
}
c10::DeleterFnPtr GCUDeviceAllocator::raw_deleter() const { return &device_deleter; }
void GCUDeviceAllocator::copy_data(void* dest, const void* src, std::size_t count) const {
  GCU_CUDA_CHECK(cudaMemcpy(dest, src, count, cudaMemcpyDeviceToDevice));
}
void GCUDeviceAllocator::record_stream(const c10::DataPtr& ptr, cudaStream_t stream) {
  device_impl()->record_stream(ptr.get(), stream);
}

// ------------------------------------------------------ pinned host memory --
namespace {
struct HostBlock {
  void* ptr;
  size_t size;
  std::vector<cudaEvent_t> events;
};
struct HostState {
  std::mutex m;
  std::unordered_map<void*, HostBlock*> live;
  std::multimap<size_t, HostBlock*> cache;
  std::deque<HostBlock*> waiting;  // freed, events outstanding
};
HostState& host_state() {
  static HostState* s = new HostState();
  return *s;
}
bool host_events_done(HostBlock* b) {
  while (!b->events.empty()) {
    cudaError_t e = cudaEventQuery(b->events.back());
    if (e == cudaErrorNotReady) {
      (void)cudaGetLastError();
      return false;
    }
    (void)cudaEventDestroy(b->events.back());
    b->events.pop_back();
  }
  return true;
}
void host_process_waiting(HostState& s) {
  for (auto it = s.waiting.begin(); it != s.waiting.end();) {
    if (host_events_done(*it)) {
      s.cache.emplace((*it)->size, *it);
      it = s.waiting.erase(it);
    } else {
      ++it;
    }
  }
}
void host_deleter(void* ptr) {
  if (!ptr) return;
  HostState& s = host_state();
  std::lock_guard<std::mutex> g(s.m);
  auto it = s.live.find(ptr);
  if (it == s.live.end()) return;
  HostBlock* b = it->second;
  s.live.erase(it);
  if (host_events_done(b)) s.cache.emplace(b->size, b);
  else s.waiting.push_back(b);
}
}  // namespace

GCUHostAllocator* GCUHostAllocator::get() {
  static GCUHostAllocator a;
  return &a;
}
c10::DataPtr GCUHostAllocator::allocate(size_t nbytes) {
  if (nbytes == 0) return {nullptr, nullptr, &host_deleter, c10::Device(c10::DeviceType::CPU)};
  const size_t size = (nbytes + 4095) / 4096 * 4096;
  HostState& s = host_state();
  std::lock_guard<std::mutex> g(s.m);
  host_process_waiting(s);
  HostBlock* b = nullptr;
  auto it = s.cache.lower_bound(size);
  if (it != s.cache.end() && it->first <= size * 2) {
    b = it->second;
    s.cache.erase(it);
  } else {
    void* p = nullptr;
    GCU_CUDA_CHECK(cudaHostAlloc(&p, size, cudaHostAllocDefault));
    b = new HostBlock{p, size, {}};
  }
  s.live[b->ptr] = b;
  return {b->ptr, b->ptr, &host_deleter, c10::Device(c10::DeviceType::CPU)};
}
c10::DeleterFnPtr GCUHostAllocator::raw_deleter() const { return &host_deleter; }
void GCUHostAllocator::copy_data(void* dest, const void* src, std::size_t count) const { std::memcpy(dest, src, count); }
void GCUHostAllocator::record_event(void* ptr, cudaStream_t stream) {
  HostState& s = host_state();
  std::lock_guard<std::mutex> g(s.m);
  // ptr may point inside a block (a slice of a pinned tensor)
  for (auto& kv : s.live) {
    HostBlock* b = kv.second;
    if (ptr >= b->ptr && ptr < static_cast<char*>(b->ptr) + b->size) {
      cudaEvent_t ev;
      GCU_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      GCU_CUDA_CHECK(cudaEventRecord(ev, stream));
      b->events.push_back(ev);
      return;
    }
  }
}
bool GCUHostAllocator::is_pinned(const void* ptr) {
  if (!ptr || device_count() == 0) return false;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost;
}
void GCUHostAllocator::empty_cache() {
  HostState& s = host_state();
  std::lock_guard<std::mutex> g(s.m);
  host_process_waiting(s);
  for (auto& kv : s.cache) {
    (void)cudaFreeHost(kv.second->ptr);
    delete kv.second;
  }
  s.cache.clear();
}

}  // namespace torch_gcu
