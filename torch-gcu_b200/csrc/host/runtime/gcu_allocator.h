// Stream-ordered caching allocator for device memory, and the pinned host
// allocator. It replaces the reference's block-splitting caching allocator
// (reference: torch_gcu/csrc/gcu/gcu_caching_allocator.{h:231-305,cpp:593,815})
// with a design that leans on stream order:
//   * a freed block goes back to a per-stream cache and is handed out again to
//     the same stream with no synchronisation and no driver call (work on one
//     stream is ordered, so reuse is safe by construction);
//   * a cache miss calls the backend's stream-ordered allocation
//     (cudaMallocAsync from the device's pool, release threshold unlimited);
//   * a block that other streams touched (recordStream) is parked until events
//     recorded on those streams have completed;
//   * out of memory: cached blocks are returned to the backend and the request
//     retried once before an OutOfMemoryError is raised;
//   * while a stream captures a graph, its allocations come from a private pool
//     (plain device allocations, legal during capture) that keeps every block it
//     ever handed out until the graph is destroyed: blocks freed during capture
//     are reused later in the same capture, never by eager code, so a replay
//     never writes into memory someone else has been given
//     (reference: gcu_caching_allocator.h:247-261 private pools for GCUGraph).
// The device backend is an interface so the policy can be unit-tested on a
// machine without a GPU against a fake backend.
#pragma once

#include <c10/core/Allocator.h>
#include <c10/core/Device.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace torch_gcu {

struct DeviceStats {
  int64_t allocated_bytes = 0, allocated_bytes_peak = 0;  // handed out to tensors
  int64_t reserved_bytes = 0, reserved_bytes_peak = 0;    // handed out + cached
  int64_t num_allocs = 0, num_cache_hits = 0, num_backend_allocs = 0, num_backend_frees = 0;
  int64_t num_alloc_retries = 0, num_ooms = 0, num_deferred_frees = 0;
};

// What the allocator needs from the device runtime.
class MemoryBackend {
 public:
  virtual ~MemoryBackend() = default;
  virtual void* alloc(int device, size_t bytes, cudaStream_t stream) = 0;  // nullptr when out of memory
  virtual void free(int device, void* ptr, cudaStream_t stream) = 0;
  virtual void* record_event(int device, cudaStream_t stream) = 0;         // opaque event handle
  virtual bool event_done(void* event) = 0;
  virtual void destroy_event(void* event) = 0;
  virtual void synchronize(int device) = 0;
  // Plain (not stream-ordered) allocation, usable while the calling thread captures a graph.
  virtual void* alloc_plain(int device, size_t bytes) = 0;   // nullptr when out of memory
  virtual void free_plain(int device, void* ptr) = 0;
  // True when work issued to `stream` is being recorded into a graph (the stream started the capture or
  // joined it by waiting on an event of a capturing stream).
  virtual bool stream_is_capturing(cudaStream_t stream) = 0;
};
std::unique_ptr<MemoryBackend> make_cuda_backend();

class StreamOrderedCachingAllocator {
 public:
  explicit StreamOrderedCachingAllocator(std::unique_ptr<MemoryBackend> backend);
  ~StreamOrderedCachingAllocator();
  void* malloc(int device, size_t bytes, cudaStream_t stream);
  void free(void* ptr);
  void record_stream(void* ptr, cudaStream_t stream);
  void empty_cache();
  // Graph capture: allocations made on `stream` between begin and end come from pool `id`
  // (returned by begin); release_pool gives the pool's memory back once no graph replays into it.
  uint64_t begin_capture(int device, cudaStream_t stream);
  void end_capture(int device, cudaStream_t stream);
  void release_pool(uint64_t id);
  DeviceStats stats(int device);
  void reset_peak_stats(int device);
  static size_t round_size(size_t bytes);

 private:
  struct Block {
    void* ptr;
    size_t size;
    int device;
    cudaStream_t stream;
    std::vector<cudaStream_t> other_streams;
    int pending_events = 0;
    uint64_t pool = 0;   // 0: the general allocator; otherwise the capture pool that owns the block
  };
  struct Pool {
    int device;
    std::multimap<size_t, Block*> cache;   // freed blocks, reusable inside this pool only
    int64_t live = 0;                      // blocks handed out and not yet freed
    bool released = false;                 // graph gone: blocks leave as they are freed
  };
  using Key = std::pair<cudaStream_t, size_t>;
  struct PerDevice {
    std::multimap<Key, Block*> cache;
    DeviceStats stats;
  };
  void process_pending_locked();
  void record_deferred_locked(Block* b);   // one event per other stream that used the block
  void release_cached_locked(int device);
  PerDevice& dev(int device);

  std::unique_ptr<MemoryBackend> backend_;
  std::mutex mutex_;
  std::unordered_map<void*, Block*> live_;
  std::unordered_map<int, PerDevice> devices_;
  std::deque<std::pair<void*, Block*>> pending_;  // (event, block)
  std::vector<Block*> parked_;   // freed with other streams recorded while a capture was open: events not recorded yet
  std::map<std::pair<int, cudaStream_t>, uint64_t> capturing_;   // (device, stream) -> pool
  std::unordered_map<uint64_t, Pool> pools_;
  uint64_t next_pool_ = 1;
};

// The process-wide device allocator registered with c10 for PrivateUse1.
class GCUDeviceAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t nbytes) override;
  c10::DeleterFnPtr raw_deleter() const override;
  void copy_data(void* dest, const void* src, std::size_t count) const override;
  static GCUDeviceAllocator* get();
  StreamOrderedCachingAllocator& impl();
  void record_stream(const c10::DataPtr& ptr, cudaStream_t stream);
};

// Pinned host memory (reference: gcu_caching_host_allocator.cpp): blocks are
// cached by size and reused once the copies that used them have completed.
class GCUHostAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t nbytes) override;
  c10::DeleterFnPtr raw_deleter() const override;
  void copy_data(void* dest, const void* src, std::size_t count) const override;
  static GCUHostAllocator* get();
  // Notes that an async copy on `stream` reads or writes the pinned block at ptr.
  void record_event(void* ptr, cudaStream_t stream);
  bool is_pinned(const void* ptr);
  void empty_cache();
};

}  // namespace torch_gcu
