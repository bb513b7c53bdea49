// Fake works and a fake communicator for the backend's watchdog
// (distributed/work_watchdog.h). The completion query of a FakeWork, the
// asynchronous-error poll and the abort hook are Python callables, so a test can
// make a collective "never complete" or a communicator "report an error" without
// any device, any NCCL call or anything that hangs.
#include <pybind11/functional.h>
#include <torch/csrc/utils/pybind.h>

#include "distributed/work_watchdog.h"

namespace c10d_gcu {
namespace {

class FakeWork final : public Watched {
 public:
  FakeWork(py::function completed, int64_t timeout_ms, uint64_t seq)
      : completed_(std::move(completed)), timeout_(timeout_ms), seq_(seq), start_(std::chrono::steady_clock::now()) {}
  ~FakeWork() override {
    py::gil_scoped_acquire gil;
    completed_ = py::function();
  }
  bool poll_completed() override {
    {
      std::lock_guard<std::mutex> g(m_);
      if (exception_) return true;
    }
    py::gil_scoped_acquire gil;
    return completed_().cast<bool>();
  }
  bool failed() const override {
    std::lock_guard<std::mutex> g(m_);
    return static_cast<bool>(exception_);
  }
  bool timed_out(std::chrono::steady_clock::time_point now) const override {
    return timeout_.count() > 0 && now - start_ >= timeout_;
  }
  void fail(std::exception_ptr e) override {
    std::lock_guard<std::mutex> g(m_);
    if (!exception_) exception_ = e;
  }
  void finish() override { finished_ = true; }
  uint64_t sequence() const override { return seq_; }
  std::chrono::milliseconds timeout() const override { return timeout_; }

  bool finished() const { return finished_; }
  std::string exception_text() const {
    std::exception_ptr e;
    {
      std::lock_guard<std::mutex> g(m_);
      e = exception_;
    }
    if (!e) return std::string();
    try {
      std::rethrow_exception(e);
    } catch (const c10::DistBackendError& err) {
      return std::string("DistBackendError: ") + err.what_without_backtrace();
    } catch (const std::exception& err) {
      return err.what();
    }
  }

 private:
  py::function completed_;
  std::chrono::milliseconds timeout_;
  uint64_t seq_;
  std::chrono::steady_clock::time_point start_;
  mutable std::mutex m_;
  std::exception_ptr exception_;
  std::atomic<bool> finished_{false};
};

}  // namespace

void bind_watchdog_selftest(py::module& m) {
  py::class_<FakeWork, std::shared_ptr<FakeWork>>(m, "FakeWork")
      .def(py::init<py::function, int64_t, uint64_t>(), py::arg("completed"), py::arg("timeout_ms"), py::arg("seq"))
      .def_property_readonly("finished", &FakeWork::finished)
      .def_property_readonly("failed", &FakeWork::failed)
      .def_property_readonly("exception_text", &FakeWork::exception_text);
  py::class_<WorkWatchdog, std::shared_ptr<WorkWatchdog>>(m, "Watchdog")
      .def(py::init([](py::function poll, py::function abort_hook, int64_t idle_ms) {
             // the watchdog thread holds no GIL of its own: take it around each call into Python
             auto poll_sp = std::make_shared<py::function>(std::move(poll));
             auto abort_sp = std::make_shared<py::function>(std::move(abort_hook));
             return std::make_shared<WorkWatchdog>(
                 [poll_sp] {
                   py::gil_scoped_acquire gil;
                   return (*poll_sp)().cast<std::string>();
                 },
                 [abort_sp] {
                   py::gil_scoped_acquire gil;
                   (*abort_sp)();
                 },
                 std::chrono::milliseconds(idle_ms));
           }),
           py::arg("poll_async_error"), py::arg("abort_hook"), py::arg("idle_ms") = 20)
      // every call that takes the watchdog's lock drops the GIL first: the watchdog thread holds that
      // lock while it calls back into Python
      .def("watch", [](WorkWatchdog& w, std::shared_ptr<FakeWork> work) { w.watch(std::move(work)); },
           py::call_guard<py::gil_scoped_release>())
      .def("stop", &WorkWatchdog::stop, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("has_failed", &WorkWatchdog::has_failed)
      .def("failure", &WorkWatchdog::failure, py::call_guard<py::gil_scoped_release>())
      .def("outstanding", &WorkWatchdog::outstanding, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("abort_calls", &WorkWatchdog::abort_calls);
}

}  // namespace c10d_gcu
