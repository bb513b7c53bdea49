#include "distributed/ProcessGroupECCL.hpp"

#include <c10/core/DeviceGuard.h>
#include <c10/util/env.h>

#include <cstring>
#include <sstream>

namespace c10d_gcu {

using torch_gcu::getCurrentGCUStream;
using torch_gcu::getStreamFromPool;

#define ECCL_CHECK(EXPR)                                                                         \
  do {                                                                                           \
    ncclResult_t _r = (EXPR);                                                                    \
    TORCH_CHECK(_r == ncclSuccess || _r == ncclInProgress, "ECCL(NCCL) error in " #EXPR ": ",    \
                ncclGetErrorString(_r), " (", ncclGetLastError(nullptr), ")");                   \
  } while (0)

ncclDataType_t to_nccl_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return ncclFloat;
    case at::kBFloat16: return ncclBfloat16;
    case at::kHalf: return ncclHalf;
    case at::kDouble: return ncclDouble;
    case at::kLong: return ncclInt64;
    case at::kInt: return ncclInt32;
    case at::kChar: return ncclInt8;
    case at::kByte: return ncclUint8;
    case at::kBool: return ncclUint8;
    default: TORCH_CHECK(false, "dtype ", t, " is not supported by the eccl backend");
  }
}

ncclRedOp_t to_nccl_op(const c10d::ReduceOp& op, at::ScalarType t) {
  if (t == at::kBool) {
    // bool: SUM acts as OR, PRODUCT/MIN as AND, like the NCCL backend of PyTorch
    if (op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::MAX) return ncclMax;
    if (op == c10d::ReduceOp::PRODUCT || op == c10d::ReduceOp::MIN) return ncclMin;
  }
  switch (op) {
    case c10d::ReduceOp::SUM: return ncclSum;
    case c10d::ReduceOp::AVG: return ncclAvg;
    case c10d::ReduceOp::PRODUCT: return ncclProd;
    case c10d::ReduceOp::MIN: return ncclMin;
    case c10d::ReduceOp::MAX: return ncclMax;
    default: TORCH_CHECK(false, "reduce op ", static_cast<int>(op), " is not supported by the eccl backend");
  }
}

void ProcessGroupECCL::check_tensor(const at::Tensor& t, const char* op) {
  TORCH_CHECK(t.defined(), op, ": undefined tensor");
  TORCH_CHECK(t.device().is_privateuseone(), op, ": tensors must be on a gcu device, got ", t.device());
  TORCH_CHECK(!t.is_sparse(), op, ": sparse tensors are not supported");
  TORCH_CHECK(t.is_contiguous(), op, ": tensors must be contiguous");
}

// ------------------------------------------------------------------- Work --
ProcessGroupECCL::WorkECCL::WorkECCL(int rank, c10d::OpType op, uint64_t seq, c10::Device device,
                                     std::chrono::milliseconds timeout, bool blocking)
    : c10d::Work(rank, op), seq_(seq), device_(device), timeout_(timeout), start_(std::chrono::steady_clock::now()),
      blocking_(blocking) {
  c10::OptionalDeviceGuard g(device_);
  GCU_CUDA_CHECK(cudaEventCreateWithFlags(&end_event_, cudaEventDisableTiming));
  future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), std::vector<c10::Device>{device_});
}

ProcessGroupECCL::WorkECCL::~WorkECCL() {
  if (end_event_) (void)cudaEventDestroy(end_event_);
}

bool ProcessGroupECCL::WorkECCL::isCompleted() {
  if (captured_) return true;
  {
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) return true;
  }
  cudaError_t e = cudaEventQuery(end_event_);
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return false;
  }
  return true;
}

bool ProcessGroupECCL::WorkECCL::isSuccess() const {
  std::lock_guard<std::mutex> g(mutex_);
  return !exception_;
}

void ProcessGroupECCL::WorkECCL::setException(std::exception_ptr e) {
  std::lock_guard<std::mutex> g(mutex_);
  if (!exception_) exception_ = e;
}

bool ProcessGroupECCL::WorkECCL::timedOut(std::chrono::steady_clock::time_point now) const {
  return timeout_.count() > 0 && now - start_ >= timeout_;
}

void ProcessGroupECCL::WorkECCL::synchronizeStream() {
  // the current stream of the work's device waits for the collective; no host block
  c10::OptionalDeviceGuard g(device_);
  GCU_CUDA_CHECK(cudaStreamWaitEvent(getCurrentGCUStream(device_.index()).stream(), end_event_, 0));
}

void ProcessGroupECCL::WorkECCL::synchronize() {
  {
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) std::rethrow_exception(exception_);
  }
  synchronizeStream();
  if (blocking_) {
    while (!isCompleted()) {
      if (timedOut(std::chrono::steady_clock::now())) {
        auto e = std::make_exception_ptr(c10::DistBackendError(
            c10::SourceLocation{__func__, __FILE__, static_cast<uint32_t>(__LINE__)},
            c10::str("eccl work (seq ", seq_, ") timed out after ", timeout_.count(), " ms")));
        setException(e);
        std::rethrow_exception(e);
      }
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) std::rethrow_exception(exception_);
  }
}

bool ProcessGroupECCL::WorkECCL::wait(std::chrono::milliseconds) {
  synchronize();
  return true;
}

void ProcessGroupECCL::WorkECCL::markFinished() {
  future_->markCompleted(c10::IValue(outputs_));
  stashed_.clear();
}

void ProcessGroupECCL::WorkECCL::abort() {
  setException(std::make_exception_ptr(
      c10::DistBackendError(c10::SourceLocation{__func__, __FILE__, static_cast<uint32_t>(__LINE__)}, "eccl work aborted")));
}

// ---------------------------------------------------------- process group --
ProcessGroupECCL::ProcessGroupECCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                   c10::intrusive_ptr<Options> options)
    : c10d::Backend(rank, size), store_(store), options_(std::move(options)) {
  TORCH_CHECK(size >= 1 && rank >= 0 && rank < size, "eccl: invalid rank ", rank, " for world size ", size);
  TORCH_CHECK(store_, "eccl: a c10d store is required to exchange the communicator id");
  // TORCH_ECCL_BLOCKING_WAIT (reference: ProcessGroupECCL.hpp:44-149, .cpp:719-756)
  auto bw = c10::utils::get_env("TORCH_ECCL_BLOCKING_WAIT");
  blocking_wait_ = bw.has_value() && (*bw == "1" || *bw == "true" || *bw == "TRUE");
  watchdog_ = std::make_unique<WorkWatchdog>([this] { return poll_async_error(); }, [this] { abort(); });
}

ProcessGroupECCL::~ProcessGroupECCL() { shutdown(); }

void ProcessGroupECCL::shutdown() {
  if (!stop_.exchange(true) && watchdog_) watchdog_->stop();   // before the communicators go away
  std::lock_guard<std::mutex> g(mutex_);
  for (auto& kv : comms_) {
    Comm& c = kv.second;
    if (c.comm) {
      if (c.aborted) (void)ncclCommAbort(c.comm);
      else {
        (void)cudaStreamSynchronize(c.stream);
        (void)ncclCommDestroy(c.comm);
      }
      c.comm = nullptr;
    }
    if (c.handoff) (void)cudaEventDestroy(c.handoff);
    c.handoff = nullptr;
  }
  comms_.clear();
}

void ProcessGroupECCL::abort() {
  std::lock_guard<std::mutex> g(mutex_);
  for (auto& kv : comms_)
    if (kv.second.comm && !kv.second.aborted) {
      (void)ncclCommAbort(kv.second.comm);
      kv.second.comm = nullptr;
      kv.second.aborted = true;
    }
}

// First use of a device: rank 0 creates the unique id and publishes it in the
// store, every rank joins the communicator, a comm stream is taken from the pool.
ProcessGroupECCL::Comm& ProcessGroupECCL::get_comm(c10::Device device) {
  std::lock_guard<std::mutex> g(mutex_);
  const int key = device.index();
  auto it = comms_.find(key);
  if (it != comms_.end()) {
    TORCH_CHECK(!it->second.aborted && it->second.comm, "eccl: the communicator was aborted");
    return it->second;
  }
  TORCH_CHECK(comms_.empty(), "eccl: one process drives one device; this group already uses gcu:", comms_.begin()->first,
              " and cannot also use gcu:", key);
  c10::OptionalDeviceGuard dg(device);
  Comm c;
  const std::string store_key = "eccl_unique_id/" + std::to_string(comm_counter_++);
  if (rank_ == 0) {
    ECCL_CHECK(ncclGetUniqueId(&c.id));
    std::vector<uint8_t> bytes(reinterpret_cast<uint8_t*>(&c.id), reinterpret_cast<uint8_t*>(&c.id) + sizeof(c.id));
    store_->set(store_key, bytes);
  } else {
    std::vector<uint8_t> bytes = store_->get(store_key);  // blocks until rank 0 published it (store timeout applies)
    TORCH_CHECK(bytes.size() == sizeof(c.id), "eccl: malformed unique id in the store");
    std::memcpy(&c.id, bytes.data(), sizeof(c.id));
  }
  ECCL_CHECK(ncclCommInitRank(&c.comm, size_, c.id, rank_));
  c.stream = getStreamFromPool(options_->is_high_priority_stream, device.index()).stream();
  GCU_CUDA_CHECK(cudaEventCreateWithFlags(&c.handoff, cudaEventDisableTiming));
  last_device_ = device;
  return comms_.emplace(key, c).first->second;
}

std::string ProcessGroupECCL::get_unique_id_hex() {
  Comm& c = get_comm(c10::Device(c10::DeviceType::PrivateUse1, torch_gcu::current_device()));
  std::ostringstream os;
  const unsigned char* p = reinterpret_cast<const unsigned char*>(&c.id);
  for (size_t i = 0; i < sizeof(c.id); ++i) os << std::hex << (p[i] >> 4) << (p[i] & 15);
  return os.str();
}

namespace {
// What the watchdog sees of a WorkECCL.
struct WatchedWork final : public Watched {
  explicit WatchedWork(c10::intrusive_ptr<ProcessGroupECCL::WorkECCL> w) : w_(std::move(w)) {}
  bool poll_completed() override { return w_->isCompleted(); }
  bool failed() const override { return !w_->isSuccess(); }
  bool timed_out(std::chrono::steady_clock::time_point now) const override { return w_->timedOut(now); }
  void fail(std::exception_ptr e) override { w_->setException(e); }
  void finish() override { w_->markFinished(); }
  uint64_t sequence() const override { return w_->getSequencenumber(); }
  std::chrono::milliseconds timeout() const override { return w_->timeout(); }
  c10::intrusive_ptr<ProcessGroupECCL::WorkECCL> w_;
};
}  // namespace

void ProcessGroupECCL::enqueue(const c10::intrusive_ptr<WorkECCL>& work) {
  watchdog_->watch(std::make_shared<WatchedWork>(work));
}

// Asked by the watchdog on every sweep (reference: checkForECCLErrors,
// ProcessGroupECCL.cpp:1682-1700): a communicator that reports anything but success or
// "in progress" is broken for every outstanding work.
std::string ProcessGroupECCL::poll_async_error() {
  std::lock_guard<std::mutex> g(mutex_);
  for (auto& kv : comms_) {
    Comm& c = kv.second;
    if (!c.comm || c.aborted) continue;
    ncclResult_t state = ncclSuccess;
    if (ncclCommGetAsyncError(c.comm, &state) != ncclSuccess) continue;
    if (state != ncclSuccess && state != ncclInProgress)
      return std::string(ncclGetErrorString(state)) + " (" + ncclGetLastError(c.comm) + ")";
  }
  return std::string();
}

template <typename Fn>
c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::collective(std::vector<at::Tensor> inputs, std::vector<at::Tensor> outputs,
                                                            Fn fn, c10d::OpType op) {
  const c10::Device device = (outputs.empty() ? inputs : outputs)[0].device();
  Comm& c = get_comm(device);
  c10::OptionalDeviceGuard dg(device);
  ++seq_;
  auto work = c10::make_intrusive<WorkECCL>(rank_, op, seq_, device, options_->timeout, blocking_wait_);
  // compute stream -> comm stream (one reusable event: re-recording a CUDA event is cheap)
  cudaStream_t compute = getCurrentGCUStream(device.index()).stream();
  GCU_CUDA_CHECK(cudaEventRecord(c.handoff, compute));
  GCU_CUDA_CHECK(cudaStreamWaitEvent(c.stream, c.handoff, 0));
  fn(c.comm, c.stream);
  work->outputs_ = outputs;
  work->stashed_ = std::move(inputs);
  work->stashed_.insert(work->stashed_.end(), outputs.begin(), outputs.end());
  if (coalescing_depth_ > 0) {
    // inside an open group nothing has been launched yet: the end event is recorded, and the
    // work handed to the watchdog, when the group closes
    coalesced_.emplace_back(work, c.stream);
    last_coalesced_ = work;
    return work;
  }
  GCU_CUDA_CHECK(cudaEventRecord(work->end_event_, c.stream));
  // A collective recorded into a graph has no completion of its own to watch: its event belongs
  // to the capture and may not be queried; only the stream hand-off in wait() applies.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(compute, &cap) != cudaSuccess) (void)cudaGetLastError();
  if (cap == cudaStreamCaptureStatusActive) {
    work->captured_ = true;
    return work;
  }
  enqueue(work);
  return work;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "eccl allreduce: expecting one tensor only but got multiple (one process drives one device)");
  at::Tensor t = tensors[0];
  check_tensor(t, "allreduce");
  return collective({t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclAllReduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), to_nccl_dtype(t.scalar_type()),
                             to_nccl_op(opts.reduceOp, t.scalar_type()), comm, s));
  }, c10d::OpType::ALLREDUCE);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::allreduce_outplace(at::Tensor& output, at::Tensor& input,
                                                                    const c10d::AllreduceOptions& opts) {
  check_tensor(input, "allreduce_outplace");
  check_tensor(output, "allreduce_outplace");
  TORCH_CHECK(input.numel() == output.numel() && input.scalar_type() == output.scalar_type(),
              "allreduce_outplace: input and output must agree in size and dtype");
  at::Tensor in = input, out = output;
  return collective({in}, {out}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclAllReduce(in.data_ptr(), out.data_ptr(), static_cast<size_t>(in.numel()), to_nccl_dtype(in.scalar_type()),
                             to_nccl_op(opts.reduceOp, in.scalar_type()), comm, s));
  }, c10d::OpType::ALLREDUCE);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "eccl broadcast: expecting one tensor only but got multiple");
  at::Tensor t = tensors[0];
  check_tensor(t, "broadcast");
  const int root = static_cast<int>(opts.rootRank + opts.rootTensor);
  TORCH_CHECK(root >= 0 && root < size_, "broadcast: invalid root rank ", root);
  return collective({t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclBroadcast(t.data_ptr(), t.data_ptr(), t.nbytes(), ncclUint8, root, comm, s));
  }, c10d::OpType::BROADCAST);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::_allgather_base(at::Tensor& output, at::Tensor& input, const c10d::AllgatherOptions&) {
  check_tensor(input, "_allgather_base");
  check_tensor(output, "_allgather_base");
  TORCH_CHECK(input.scalar_type() == output.scalar_type(), "_allgather_base: output tensor must have the same type as input tensor");
  TORCH_CHECK(input.numel() * size_ == output.numel(), "_allgather_base: output tensor size must be equal to world_size times input tensor size");
  at::Tensor in = input, out = output;
  return collective({in}, {out}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclAllGather(in.data_ptr(), out.data_ptr(), in.nbytes(), ncclUint8, comm, s));
  }, c10d::OpType::_ALLGATHER_BASE);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                                           const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "eccl allgather: expecting one input tensor and one output list");
  at::Tensor in = inputs[0];
  check_tensor(in, "allgather");
  std::vector<at::Tensor>& outs = outputs[0];
  TORCH_CHECK(static_cast<int>(outs.size()) == size_, "allgather: output list must have world_size tensors");
  for (auto& o : outs) {
    check_tensor(o, "allgather");
    TORCH_CHECK(o.numel() == in.numel() && o.scalar_type() == in.scalar_type(), "allgather: all tensors must agree in size and dtype");
  }
  at::Tensor flat = at::empty({size_, in.numel()}, in.options());
  auto work = _allgather_base(flat, in, opts);
  // unpack on the compute stream once the gather is visible to it
  work->wait();
  for (int r = 0; r < size_; ++r) outs[r].copy_(flat[r].view_as(outs[r]));
  return work;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::_reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                                     const c10d::ReduceScatterOptions& opts) {
  check_tensor(input, "_reduce_scatter_base");
  check_tensor(output, "_reduce_scatter_base");
  TORCH_CHECK(input.scalar_type() == output.scalar_type(), "_reduce_scatter_base: input and output must have the same type");
  TORCH_CHECK(output.numel() * size_ == input.numel(), "_reduce_scatter_base: input tensor must be world_size times the output size");
  at::Tensor in = input, out = output;
  return collective({in}, {out}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclReduceScatter(in.data_ptr(), out.data_ptr(), static_cast<size_t>(out.numel()), to_nccl_dtype(in.scalar_type()),
                                 to_nccl_op(opts.reduceOp, in.scalar_type()), comm, s));
  }, c10d::OpType::_REDUCE_SCATTER_BASE);
}

// List form: the inputs of all ranks are packed into one buffer first
// (reference: ProcessGroupECCL.cpp:3168-3330).
c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::reduce_scatter(std::vector<at::Tensor>& outputs,
                                                               std::vector<std::vector<at::Tensor>>& inputs,
                                                               const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1, "eccl reduce_scatter: expecting one output tensor and one input list");
  TORCH_CHECK(static_cast<int>(inputs[0].size()) == size_, "eccl reduce_scatter: the input list must have world_size entries");
  at::Tensor out = outputs[0];
  check_tensor(out, "reduce_scatter");
  for (const auto& t : inputs[0]) {
    check_tensor(t, "reduce_scatter");
    TORCH_CHECK(t.numel() == out.numel() && t.scalar_type() == out.scalar_type(), "eccl reduce_scatter: every input must match the output");
  }
  at::Tensor flat = at::empty({size_, out.numel()}, out.options());
  for (int r = 0; r < size_; ++r) flat[r].copy_(inputs[0][r].reshape({-1}));
  return _reduce_scatter_base(out, flat, opts);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "eccl reduce: expecting one tensor");
  at::Tensor t = tensors[0];
  check_tensor(t, "reduce");
  const int root = static_cast<int>(opts.rootRank);
  TORCH_CHECK(root >= 0 && root < size_, "eccl reduce: invalid root rank ", root);
  return collective({t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclReduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), to_nccl_dtype(t.scalar_type()),
                          to_nccl_op(opts.reduceOp, t.scalar_type()), root, comm, s));
  }, c10d::OpType::REDUCE);
}

// Equal or explicit splits along dim 0, as grouped sends and receives.
c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::alltoall_base(at::Tensor& output, at::Tensor& input,
                                                              std::vector<int64_t>& outputSplitSizes,
                                                              std::vector<int64_t>& inputSplitSizes, const c10d::AllToAllOptions&) {
  check_tensor(input, "alltoall_base");
  check_tensor(output, "alltoall_base");
  TORCH_CHECK(input.scalar_type() == output.scalar_type(), "eccl alltoall_base: input and output must have the same type");
  auto splits = [&](const at::Tensor& t, const std::vector<int64_t>& given, const char* what) {
    std::vector<int64_t> v = given;
    if (v.empty()) {
      TORCH_CHECK(t.dim() >= 1 && t.size(0) % size_ == 0, "eccl alltoall_base: ", what, " dim 0 must divide by world_size");
      v.assign(size_, t.size(0) / size_);
    }
    TORCH_CHECK(static_cast<int>(v.size()) == size_, "eccl alltoall_base: ", what, " split list must have world_size entries");
    int64_t total = 0;
    for (int64_t x : v) { TORCH_CHECK(x >= 0, "eccl alltoall_base: negative split"); total += x; }
    TORCH_CHECK(total == (t.dim() ? t.size(0) : 0), "eccl alltoall_base: ", what, " splits do not sum to dim 0");
    return v;
  };
  const std::vector<int64_t> in_s = splits(input, inputSplitSizes, "input"), out_s = splits(output, outputSplitSizes, "output");
  at::Tensor in = input, out = output;
  const int64_t in_row = in.size(0) ? in.nbytes() / in.size(0) : 0, out_row = out.size(0) ? out.nbytes() / out.size(0) : 0;
  return collective({in}, {out}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclGroupStart());
    int64_t io = 0, oo = 0;
    for (int r = 0; r < size_; ++r) {
      if (in_s[r]) ECCL_CHECK(ncclSend(static_cast<const char*>(in.data_ptr()) + io * in_row, in_s[r] * in_row, ncclUint8, r, comm, s));
      if (out_s[r]) ECCL_CHECK(ncclRecv(static_cast<char*>(out.data_ptr()) + oo * out_row, out_s[r] * out_row, ncclUint8, r, comm, s));
      io += in_s[r];
      oo += out_s[r];
    }
    ECCL_CHECK(ncclGroupEnd());
  }, c10d::OpType::ALLTOALL_BASE);
}

void ProcessGroupECCL::group_start() {
  ECCL_CHECK(ncclGroupStart());
  ++coalescing_depth_;
}
void ProcessGroupECCL::group_end() {
  TORCH_CHECK(coalescing_depth_ > 0, "eccl: _group_end without a matching _group_start");
  --coalescing_depth_;
  ECCL_CHECK(ncclGroupEnd());
  if (coalescing_depth_ == 0) {
    for (auto& [work, stream] : coalesced_) {
      c10::OptionalDeviceGuard dg(work->device_);
      GCU_CUDA_CHECK(cudaEventRecord(work->end_event_, stream));
      enqueue(work);
    }
    coalesced_.clear();
  }
}
void ProcessGroupECCL::startCoalescing() {
  last_coalesced_.reset();
  group_start();
}
c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::endCoalescing() {
  group_end();
  // every collective of the group completes with the group: the last one's work stands for all
  auto w = last_coalesced_;
  last_coalesced_.reset();
  return w;
}

// A 1-element allreduce on the group's device, waited for on the host
// (reference: ProcessGroupECCL.cpp:3462).
c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::barrier(const c10d::BarrierOptions& opts) {
  c10::Device device = last_device_;
  if (!opts.device_ids.empty()) device = c10::Device(c10::DeviceType::PrivateUse1, static_cast<c10::DeviceIndex>(opts.device_ids[0]));
  else if (comms_.empty()) device = c10::Device(c10::DeviceType::PrivateUse1, torch_gcu::current_device());
  c10::OptionalDeviceGuard dg(device);
  at::Tensor t = at::zeros({1}, at::TensorOptions().device(device).dtype(at::kFloat));
  std::vector<at::Tensor> ts{t};
  auto work = allreduce(ts);
  work->wait();
  GCU_CUDA_CHECK(cudaStreamSynchronize(getCurrentGCUStream(device.index()).stream()));
  return work;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::send(std::vector<at::Tensor>& tensors, int dstRank, int) {
  TORCH_CHECK(tensors.size() == 1, "eccl send: expecting one tensor");
  at::Tensor t = tensors[0];
  check_tensor(t, "send");
  return collective({t}, {}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclSend(t.data_ptr(), t.nbytes(), ncclUint8, dstRank, comm, s));
  }, c10d::OpType::SEND);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupECCL::recv(std::vector<at::Tensor>& tensors, int srcRank, int) {
  TORCH_CHECK(tensors.size() == 1, "eccl recv: expecting one tensor");
  at::Tensor t = tensors[0];
  check_tensor(t, "recv");
  return collective({}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    ECCL_CHECK(ncclRecv(t.data_ptr(), t.nbytes(), ncclUint8, srcRank, comm, s));
  }, c10d::OpType::RECV);
}

}  // namespace c10d_gcu
