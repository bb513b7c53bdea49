// Graph capture and replay (reference: torch_gcu/csrc/gcu/gcu_graph.cpp,
// torch_gcu/gcu/graphs.py:50-226). A launch-bound sequence of operators (one decode
// step: ~17 small kernels per layer) is recorded once from the current stream into
// a CUDA graph and replayed with one launch. Memory handed out while capturing
// comes from a private pool of the allocator that lives as long as the graph, so
// every replay reads and writes the addresses the capture saw.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace torch_gcu {

class GCUGraph {
 public:
  GCUGraph() = default;
  ~GCUGraph();
  GCUGraph(const GCUGraph&) = delete;
  GCUGraph& operator=(const GCUGraph&) = delete;

  // Starts capturing the current stream of the current device (not the default stream).
  void capture_begin();
  // Ends the capture and instantiates the executable graph.
  void capture_end();
  // Launches the captured work on the current stream.
  void replay();
  // Drops the executable graph and gives the pool back.
  void reset();
  bool captured() const { return exec_ != nullptr; }
  int64_t num_nodes() const { return num_nodes_; }

 private:
  cudaGraph_t graph_ = nullptr;
  cudaGraphExec_t exec_ = nullptr;
  cudaStream_t capture_stream_ = nullptr;
  int device_ = -1;
  uint64_t pool_ = 0;
  bool capturing_ = false;
  int64_t num_nodes_ = 0;
};

// True while the current stream of the current device is being captured.
bool current_stream_is_capturing();

}  // namespace torch_gcu
