// c10d backend "eccl" for gcu (B200) tensors, over NCCL / NVLink.
//
// Same structure as the reference's ProcessGroupECCL (reference:
// torch_gcu/csrc/distributed/ProcessGroupECCL.hpp:233-1064, .cpp collective<>
// 2270-2419, getECCLComm 1801-2019, broadcastUniqueECCLID 1721-1779, WorkECCL
// 598-648, watchdogHandler 1485-1616), reduced to what the tensor-parallel path
// and init_process_group need: one communicator per device, created on first use
// with the unique id published through the c10d Store; one dedicated comm stream
// per device; the compute stream hands over to the comm stream through an event
// and Work::wait() makes the current stream wait for the end event (no host
// block unless blocking wait is on); a watchdog thread (work_watchdog.h) polls the
// communicator for asynchronous errors, times works out and aborts the communicator. The allocator is stream-ordered, so instead of recordStream
// the Work object keeps its tensors alive until it completes.
#pragma once

#include <nccl.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "distributed/work_watchdog.h"
#include "runtime/gcu_runtime.h"

namespace c10d_gcu {

constexpr const char* ECCL_BACKEND_NAME = "eccl";
constexpr auto kProcessGroupECCLDefaultTimeout = std::chrono::milliseconds(10 * 60 * 1000);

class ProcessGroupECCL : public c10d::Backend {
 public:
  struct Options : public c10d::Backend::Options {
    explicit Options(bool is_high_priority_stream = true)
        : c10d::Backend::Options(ECCL_BACKEND_NAME, kProcessGroupECCLDefaultTimeout),
          is_high_priority_stream(is_high_priority_stream) {}
    static c10::intrusive_ptr<Options> create(bool is_high_priority_stream = true) {
      return c10::make_intrusive<Options>(is_high_priority_stream);
    }
    bool is_high_priority_stream;
  };

  class WorkECCL : public c10d::Work {
   public:
    WorkECCL(int rank, c10d::OpType op, uint64_t seq, c10::Device device, std::chrono::milliseconds timeout, bool blocking);
    ~WorkECCL() override;
    bool isCompleted() override;
    bool isSuccess() const override;
    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
    void synchronize() override;
    void blockCurrentStream() override { synchronizeStream(); }
    void abort() override;
    std::vector<at::Tensor> result() override { return outputs_; }
    uint64_t getSequencenumber() const override { return seq_; }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
    bool timedOut(std::chrono::steady_clock::time_point now) const;
    void setException(std::exception_ptr e);
    void markFinished();   // success seen by the watchdog: fulfil the future, release the tensors
    std::chrono::milliseconds timeout() const { return timeout_; }

   private:
    friend class ProcessGroupECCL;
    void synchronizeStream();
    uint64_t seq_;
    c10::Device device_;
    bool captured_ = false;   // issued while the compute stream was capturing a graph
    cudaEvent_t end_event_ = nullptr;
    std::chrono::milliseconds timeout_;
    std::chrono::steady_clock::time_point start_;
    bool blocking_;
    std::vector<at::Tensor> stashed_;   // inputs/outputs kept alive until completion
    std::vector<at::Tensor> outputs_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
    mutable std::mutex mutex_;
    std::exception_ptr exception_;
  };

  ProcessGroupECCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                   c10::intrusive_ptr<Options> options = Options::create());
  ProcessGroupECCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout)
      : ProcessGroupECCL(store, rank, size, make_options(timeout)) {}
  ~ProcessGroupECCL() override;

  const std::string getBackendName() const override { return ECCL_BACKEND_NAME; }
  c10::intrusive_ptr<Options> getOptions() { return options_; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts = c10d::AllreduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> allreduce_outplace(at::Tensor& output, at::Tensor& input,
                                                    const c10d::AllreduceOptions& opts = c10d::AllreduceOptions());
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                           const c10d::BroadcastOptions& opts = c10d::BroadcastOptions()) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors,
                                        const c10d::ReduceOptions& opts = c10d::ReduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& outputSplitSizes,
                                               std::vector<int64_t>& inputSplitSizes,
                                               const c10d::AllToAllOptions& opts = c10d::AllToAllOptions()) override;
  // Coalescing: the collectives issued between the two calls go out as one NCCL group
  // (reference: ProcessGroupECCL.cpp:3976-4048, Python _group_start / _group_end).
  void startCoalescing() override;
  c10::intrusive_ptr<c10d::Work> endCoalescing() override;
  void group_start();
  void group_end();
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts = c10d::BarrierOptions()) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dstRank, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int srcRank, int tag) override;

  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }
  void abort() override;
  void shutdown() override;
  std::string get_unique_id_hex();  // the id of the communicator of the current device (creates it)

  // Argument checks shared by every collective; public so they are testable
  // without a device: throws on an empty list, a non-gcu, sparse or
  // non-contiguous tensor.
  static void check_tensor(const at::Tensor& t, const char* op);

 private:
  static c10::intrusive_ptr<Options> make_options(std::chrono::milliseconds timeout) {
    auto o = Options::create();
    o->timeout = timeout;
    return o;
  }
  struct Comm {
    ncclComm_t comm = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t handoff = nullptr;  // compute -> comm, re-recorded for every collective
    ncclUniqueId id;
    bool aborted = false;
  };
  Comm& get_comm(c10::Device device);
  template <typename Fn>
  c10::intrusive_ptr<c10d::Work> collective(std::vector<at::Tensor> inputs, std::vector<at::Tensor> outputs, Fn fn,
                                            c10d::OpType op);
  void enqueue(const c10::intrusive_ptr<WorkECCL>& work);
  std::string poll_async_error();   // "" while every communicator is healthy (ncclCommGetAsyncError)

  c10::intrusive_ptr<c10d::Store> store_;
  c10::intrusive_ptr<Options> options_;
  std::mutex mutex_;
  std::unordered_map<int, Comm> comms_;  // by device index
  uint64_t seq_ = 0;
  int coalescing_depth_ = 0;
  c10::intrusive_ptr<c10d::Work> last_coalesced_;
  std::vector<std::pair<c10::intrusive_ptr<WorkECCL>, cudaStream_t>> coalesced_;
  uint64_t comm_counter_ = 0;
  bool blocking_wait_ = false;
  c10::Device last_device_ = c10::Device(c10::DeviceType::PrivateUse1, 0);

  std::unique_ptr<WorkWatchdog> watchdog_;
  std::atomic<bool> stop_{false};
};

ncclDataType_t to_nccl_dtype(at::ScalarType t);
ncclRedOp_t to_nccl_op(const c10d::ReduceOp& op, at::ScalarType t);

}  // namespace c10d_gcu
