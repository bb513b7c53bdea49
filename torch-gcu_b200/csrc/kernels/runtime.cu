// Library-level queries and the small amount of process state the kernel
// library keeps: a thread-local error message and the per-device SM count.
#include "common.cuh"

#include <atomic>

namespace b200 {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

static std::atomic<unsigned long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

int sm_count_current_device();
// SMs the persistent GEMM kernels leave free (for a collective running beside them).
static std::atomic<int> g_reserved_sms{0};
int gemm_sm_budget() {
  const int n = sm_count_current_device() - g_reserved_sms.load(std::memory_order_relaxed);
  return n < 2 ? 2 : n;
}

int sm_count_current_device() {
  // Immutable once written; racing writers store the same value.
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
    n = 148;
  cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace b200

extern "C" {

const char* b200_last_error(void) { return b200::error_buffer(); }

const char* b200_version(void) { return "b200ops 0.1 (sm_100a)"; }

unsigned long long b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }
void b200_set_reserved_sms(int n) { b200::g_reserved_sms.store(n < 0 ? 0 : n, std::memory_order_relaxed); }
int b200_get_reserved_sms(void) { return b200::g_reserved_sms.load(std::memory_order_relaxed); }

int b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int b200_sm_count(int device) {
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}

size_t b200_dtype_size(int32_t dtype) { return b200::dtype_size(dtype); }

}  // extern "C"
