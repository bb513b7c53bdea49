// Exercises the stream-ordered caching policy against a fake device backend
// (host malloc, manually completed events), so the allocator logic is testable
// on a machine without a GPU. Returns the observations as a dict; the Python
// test asserts on them. Built into the test-only module (selftest_module.cpp),
// never into the product extension.
#include <torch/csrc/utils/pybind.h>

#include <algorithm>
#include <algorithm>
#include <cstdlib>
#include <set>

#include "runtime/gcu_allocator.h"

namespace torch_gcu {
namespace {

struct FakeEvent {
  bool done = false;
};

class FakeBackend final : public MemoryBackend {
 public:
  size_t capacity = 1 << 20, used = 0;
  int allocs = 0, frees = 0, syncs = 0;
  std::unordered_map<void*, size_t> sizes;
  std::vector<FakeEvent*> events;
  void* alloc(int, size_t bytes, cudaStream_t) override {
    if (used + bytes > capacity) return nullptr;
    void* p = std::malloc(bytes);
    sizes[p] = bytes;
    used += bytes;
    ++allocs;
    return p;
  }
  void free(int, void* ptr, cudaStream_t) override {
    used -= sizes[ptr];
    sizes.erase(ptr);
    std::free(ptr);
    ++frees;
  }
  void* record_event(int, cudaStream_t) override {
    events.push_back(new FakeEvent());
    return events.back();
  }
  bool event_done(void* e) override { return static_cast<FakeEvent*>(e)->done; }
  void destroy_event(void* e) override {
    events.erase(std::remove(events.begin(), events.end(), static_cast<FakeEvent*>(e)), events.end());
    delete static_cast<FakeEvent*>(e);
  }
  void synchronize(int) override {
    ++syncs;
    for (FakeEvent* e : events) e->done = true;
  }
  std::set<cudaStream_t> capturing_streams;
  bool stream_is_capturing(cudaStream_t s) override { return capturing_streams.count(s) != 0; }
  int plain_allocs = 0, plain_frees = 0;
  void* alloc_plain(int, size_t bytes) override {
    if (used + bytes > capacity) return nullptr;
    void* p = std::malloc(bytes);
    sizes[p] = bytes;
    used += bytes;
    ++plain_allocs;
    return p;
  }
  void free_plain(int, void* ptr) override {
    used -= sizes[ptr];
    sizes.erase(ptr);
    std::free(ptr);
    ++plain_frees;
  }
};

}  // namespace

py::dict allocator_selftest() {
  py::dict r;
  auto backend = std::make_unique<FakeBackend>();
  FakeBackend* fb = backend.get();
  StreamOrderedCachingAllocator a(std::move(backend));
  cudaStream_t s1 = reinterpret_cast<cudaStream_t>(0x10), s2 = reinterpret_cast<cudaStream_t>(0x20);

  r["round_small"] = StreamOrderedCachingAllocator::round_size(1000);       // 1024
  r["round_large"] = StreamOrderedCachingAllocator::round_size((1 << 20) + 1);  // 2 MiB

  // 1. same-stream reuse: free then malloc of the same size hits the cache
  void* p1 = a.malloc(0, 1000, s1);
  a.free(p1);
  void* p2 = a.malloc(0, 900, s1);  // rounds to 1024 too
  r["same_stream_reuse"] = (p1 == p2);
  r["backend_allocs_after_reuse"] = fb->allocs;  // 1

  // 2. another stream must not get the cached block of s1
  a.free(p2);
  void* p3 = a.malloc(0, 1000, s2);
  r["cross_stream_no_reuse"] = (p3 != p1);
  a.free(p3);

  // 3. record_stream defers reuse until the recorded stream's event completed
  void* p4 = a.malloc(0, 1000, s1);  // the cached s1 block again
  r["cached_block_back"] = (p4 == p1);
  a.record_stream(p4, s2);
  a.free(p4);
  void* p5 = a.malloc(0, 1000, s1);
  r["deferred_not_reused"] = (p5 != p4);
  for (FakeEvent* e : fb->events) e->done = true;  // the other stream finished
  a.free(p5);
  std::set<void*> seen;
  void* p6 = a.malloc(0, 1000, s1);
  void* p7 = a.malloc(0, 1000, s1);
  seen.insert(p6);
  seen.insert(p7);
  r["deferred_reused_after_event"] = seen.count(p4) == 1;
  a.free(p6);
  a.free(p7);

  // 4. out of memory: cached blocks go back to the backend and the request is retried
  DeviceStats before = a.stats(0);
  r["reserved_before_oom"] = before.reserved_bytes;
  void* big = a.malloc(0, (1 << 20) - 512, s1);  // only fits once the cache is released
  r["oom_retry_succeeded"] = big != nullptr;
  DeviceStats after = a.stats(0);
  r["num_alloc_retries"] = after.num_alloc_retries;
  a.free(big);
  bool threw = false;
  try {
    a.malloc(0, 4 << 20, s1);
  } catch (const c10::OutOfMemoryError&) {
    threw = true;
  }
  r["oom_raises"] = threw;
  r["num_ooms"] = a.stats(0).num_ooms;

  // 4b. graph-capture pool: private blocks, reused inside the pool only, returned with the pool
  {
    void* eager = a.malloc(0, 2000, s1);
    a.free(eager);                                   // sits in the general cache of s1
    const uint64_t pool = a.begin_capture(0, s1);
    void* c1 = a.malloc(0, 2000, s1);
    r["capture_ignores_general_cache"] = (c1 != eager);
    a.free(c1);
    void* c2 = a.malloc(0, 2000, s1);                // later in the same capture: same block again
    r["capture_reuses_own_block"] = (c2 == c1);
    void* out = a.malloc(0, 4000, s1);               // stays alive past the capture (a graph output)
    a.free(c2);
    a.end_capture(0, s1);
    void* after = a.malloc(0, 2000, s1);             // eager code never gets the pool's block
    r["eager_does_not_get_pool_block"] = (after != c1);
    r["eager_gets_general_block"] = (after == eager);
    a.free(after);
    r["plain_allocs_in_capture"] = fb->plain_allocs;  // 2
    a.release_pool(pool);
    r["plain_frees_after_release"] = fb->plain_frees; // 1: the cached block; `out` is still alive
    a.free(out);
    r["plain_frees_after_output_died"] = fb->plain_frees;  // 2
  }

  // 4c. a block that another stream used, freed while a capture is open: no event may be recorded
  // then (it could land inside the capture and never become queryable), so the block is parked and
  // gets its events when the capture has closed
  {
    void* shared = a.malloc(0, 3000, s1);
    a.record_stream(shared, s2);
    const size_t events_before = fb->events.size();
    const uint64_t pool = a.begin_capture(0, s1);
    a.free(shared);
    r["no_event_recorded_during_capture"] = fb->events.size() == events_before;
    a.end_capture(0, s1);
    r["event_recorded_after_capture"] = fb->events.size() == events_before + 1;
    void* other = a.malloc(0, 3000, s1);     // the event has not completed: the block stays away
    r["parked_block_not_reused_early"] = (other != shared);
    for (FakeEvent* e : fb->events) e->done = true;
    a.free(other);
    void* again1 = a.malloc(0, 3000, s1);
    void* again2 = a.malloc(0, 3000, s1);
    r["parked_block_reused_after_event"] = (again1 == shared || again2 == shared);
    a.free(again1);
    a.free(again2);
    a.release_pool(pool);
  }

  // 4d. a side stream that joined the capture: its blocks come from the capture's pool, and a block freed on
  // one stream of the graph is not handed to the other stream (parallel branches)
  {
    const uint64_t pool = a.begin_capture(0, s1);
    fb->capturing_streams = {s1, s2};
    const int plain_before = fb->plain_allocs, async_before = fb->allocs;
    void* on_main = a.malloc(0, 5000, s1);
    void* on_side = a.malloc(0, 5000, s2);
    r["side_stream_allocates_from_pool"] = fb->plain_allocs == plain_before + 2 && fb->allocs == async_before;
    a.free(on_main);
    void* side2 = a.malloc(0, 5000, s2);
    r["no_cross_stream_reuse_inside_pool"] = (side2 != on_main);
    void* main2 = a.malloc(0, 5000, s1);
    r["same_stream_reuse_inside_pool"] = (main2 == on_main);
    a.free(on_side);
    a.free(side2);
    a.free(main2);
    fb->capturing_streams.clear();
    a.end_capture(0, s1);
    a.release_pool(pool);
  }

  // 5. stats and empty_cache
  a.empty_cache();
  DeviceStats fin = a.stats(0);
  r["allocated_after_all_freed"] = fin.allocated_bytes;
  r["reserved_after_empty_cache"] = fin.reserved_bytes;
  r["backend_outstanding"] = static_cast<int64_t>(fb->used);
  r["peak_allocated"] = fin.allocated_bytes_peak;
  r["cache_hits"] = fin.num_cache_hits;
  return r;
}

}  // namespace torch_gcu
