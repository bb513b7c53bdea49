// Failure detection of the "eccl" backend, kept free of any device call so the
// whole policy runs on a machine without a GPU.
//
// The reference's watchdog thread walks the list of outstanding works and, for
// each one, (1) asks the communicator for an asynchronous error, (2) checks the
// work's timeout, and on either aborts the communicators so that no rank stays
// blocked inside a collective (reference:
// torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:533-556 checkTimeout,
// :1485-1616 watchdogHandler, :1682-1700 checkForECCLErrors). This class is that
// loop. What it watches is an interface (`Watched`), the communicator's health is
// a callable and the abort is a callable, so a test can drive it with a work that
// never completes or a communicator that reports an error.
//
// Policy:
//  - a completed work is finished (future fulfilled, tensors released) and dropped;
//  - a work that outlives its timeout gets a DistBackendError naming its sequence
//    number and timeout; the abort hook runs ONCE; the watchdog is then "failed";
//  - a non-empty answer of the async-error poll fails EVERY outstanding work with
//    that text (the communicator is broken for all of them) and aborts the same way;
//  - once failed, watch() refuses new works with the text of the first failure.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>

namespace c10d_gcu {

class Watched {
 public:
  virtual ~Watched() = default;
  virtual bool poll_completed() = 0;  // host-side and non-blocking; true once the work is over
  virtual bool failed() const = 0;    // an exception was set (by anyone)
  virtual bool timed_out(std::chrono::steady_clock::time_point now) const = 0;
  virtual void fail(std::exception_ptr e) = 0;  // first exception wins
  virtual void finish() = 0;                    // success: fulfil the future, release the tensors
  virtual uint64_t sequence() const = 0;
  virtual std::chrono::milliseconds timeout() const = 0;
};

class WorkWatchdog {
 public:
  using AsyncErrorPoll = std::function<std::string()>;  // "" while the communicator is healthy
  using AbortHook = std::function<void()>;

  WorkWatchdog(AsyncErrorPoll poll, AbortHook abort_hook,
               std::chrono::milliseconds idle_period = std::chrono::milliseconds(100));
  ~WorkWatchdog();
  WorkWatchdog(const WorkWatchdog&) = delete;
  WorkWatchdog& operator=(const WorkWatchdog&) = delete;

  void watch(std::shared_ptr<Watched> work);  // throws c10::DistBackendError once failed
  void stop();                                // joins the thread; outstanding works stay as they are
  bool has_failed() const { return failed_.load(); }
  std::string failure() const;
  size_t outstanding() const;
  int abort_calls() const { return abort_calls_.load(); }

 private:
  void run();
  bool sweep(std::string* why);  // one pass over the list under the lock; true if something failed

  AsyncErrorPoll poll_;
  AbortHook abort_hook_;
  std::chrono::milliseconds idle_period_;
  mutable std::mutex mutex_;
  std::condition_variable cv_;
  std::deque<std::shared_ptr<Watched>> works_;
  std::string failure_;
  std::atomic<bool> failed_{false};
  std::atomic<bool> stop_{false};
  std::atomic<int> abort_calls_{0};
  std::thread thread_;
};

}  // namespace c10d_gcu
