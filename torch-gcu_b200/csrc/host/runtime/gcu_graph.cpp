#include "runtime/gcu_graph.h"

#include <c10/util/Exception.h>

#include "runtime/gcu_allocator.h"
#include "runtime/gcu_runtime.h"

namespace torch_gcu {

bool current_stream_is_capturing() {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  cudaStream_t s = getCurrentGCUStream().stream();
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st == cudaStreamCaptureStatusActive;
}

GCUGraph::~GCUGraph() {
  try {
    reset();
  } catch (...) {
  }
}

void GCUGraph::capture_begin() {
  TORCH_CHECK(!capturing_ && !exec_, "GCUGraph: already capturing or captured; call reset() first");
  device_ = current_device();
  GCUStream stream = getCurrentGCUStream(static_cast<c10::DeviceIndex>(device_));
  capture_stream_ = stream.stream();
  TORCH_CHECK(capture_stream_ != nullptr && capture_stream_ != cudaStreamLegacy && capture_stream_ != cudaStreamPerThread,
              "GCUGraph: capture needs a non-default stream current (use torch.gcu.graph, which switches to a side stream)");
  pool_ = GCUDeviceAllocator::get()->impl().begin_capture(device_, capture_stream_);
  // thread-local mode: other threads (the process group's watchdog) keep calling the runtime
  cudaError_t e = cudaStreamBeginCapture(capture_stream_, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    GCUDeviceAllocator::get()->impl().end_capture(device_, capture_stream_);
    GCUDeviceAllocator::get()->impl().release_pool(pool_);
    pool_ = 0;
    TORCH_CHECK(false, "cudaStreamBeginCapture failed: ", cudaGetErrorString(e));
  }
  capturing_ = true;
}

void GCUGraph::capture_end() {
  TORCH_CHECK(capturing_, "GCUGraph: capture_end without capture_begin");
  TORCH_CHECK(getCurrentGCUStream(static_cast<c10::DeviceIndex>(device_)).stream() == capture_stream_,
              "GCUGraph: the capturing stream must be current when the capture ends");
  capturing_ = false;
  cudaError_t e = cudaStreamEndCapture(capture_stream_, &graph_);
  GCUDeviceAllocator::get()->impl().end_capture(device_, capture_stream_);
  if (e != cudaSuccess || graph_ == nullptr) {
    (void)cudaGetLastError();
    graph_ = nullptr;
    reset();
    TORCH_CHECK(false, "cudaStreamEndCapture failed: ", cudaGetErrorString(e),
                " (an operator that synchronises or allocates outside the pool ran during the capture)");
  }
  size_t n = 0;
  if (cudaGraphGetNodes(graph_, nullptr, &n) == cudaSuccess) num_nodes_ = static_cast<int64_t>(n);
  e = cudaGraphInstantiate(&exec_, graph_, 0);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    exec_ = nullptr;
    reset();
    TORCH_CHECK(false, "cudaGraphInstantiate failed: ", cudaGetErrorString(e));
  }
}

void GCUGraph::replay() {
  TORCH_CHECK(exec_, "GCUGraph: nothing captured");
  c10::DeviceIndex prev = current_device();
  if (prev != device_) set_device(static_cast<c10::DeviceIndex>(device_));
  cudaError_t e = cudaGraphLaunch(exec_, getCurrentGCUStream(static_cast<c10::DeviceIndex>(device_)).stream());
  if (prev != device_) set_device(prev);
  TORCH_CHECK(e == cudaSuccess, "cudaGraphLaunch failed: ", cudaGetErrorString(e));
}

void GCUGraph::reset() {
  if (capturing_) {
    // abandon a half-made capture
    cudaGraph_t g = nullptr;
    (void)cudaStreamEndCapture(capture_stream_, &g);
    (void)cudaGetLastError();
    if (g) (void)cudaGraphDestroy(g);
    GCUDeviceAllocator::get()->impl().end_capture(device_, capture_stream_);
    capturing_ = false;
  }
  if (exec_) {
    (void)cudaGraphExecDestroy(exec_);
    exec_ = nullptr;
  }
  if (graph_) {
    (void)cudaGraphDestroy(graph_);
    graph_ = nullptr;
  }
  if (pool_) {
    GCUDeviceAllocator::get()->impl().release_pool(pool_);
    pool_ = 0;
  }
  num_nodes_ = 0;
}

}  // namespace torch_gcu
