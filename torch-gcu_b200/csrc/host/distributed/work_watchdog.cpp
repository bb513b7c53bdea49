#include "distributed/work_watchdog.h"

#include <c10/util/Exception.h>
#include <c10/util/StringUtil.h>

namespace c10d_gcu {

namespace {
std::exception_ptr backend_error(const std::string& msg) {
  return std::make_exception_ptr(
      c10::DistBackendError(c10::SourceLocation{__func__, __FILE__, static_cast<uint32_t>(__LINE__)}, msg));
}
}  // namespace

WorkWatchdog::WorkWatchdog(AsyncErrorPoll poll, AbortHook abort_hook, std::chrono::milliseconds idle_period)
    : poll_(std::move(poll)), abort_hook_(std::move(abort_hook)), idle_period_(idle_period) {
  thread_ = std::thread(&WorkWatchdog::run, this);
}

WorkWatchdog::~WorkWatchdog() { stop(); }

void WorkWatchdog::stop() {
  if (!stop_.exchange(true)) {
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
  }
}

std::string WorkWatchdog::failure() const {
  std::lock_guard<std::mutex> g(mutex_);
  return failure_;
}

size_t WorkWatchdog::outstanding() const {
  std::lock_guard<std::mutex> g(mutex_);
  return works_.size();
}

void WorkWatchdog::watch(std::shared_ptr<Watched> work) {
  {
    std::lock_guard<std::mutex> g(mutex_);
    if (failed_.load()) {
      const std::string msg = "eccl: the communicator was aborted after an earlier failure (" + failure_ +
                              "); no further collective can be issued on this group";
      work->fail(backend_error(msg));
      TORCH_CHECK_WITH(DistBackendError, false, msg);
    }
    works_.push_back(std::move(work));
  }
  cv_.notify_one();
}

bool WorkWatchdog::sweep(std::string* why) {
  // communicator health first: an asynchronous error explains every work that is still out
  const std::string async = poll_ ? poll_() : std::string();
  const auto now = std::chrono::steady_clock::now();
  bool bad = false;
  for (auto it = works_.begin(); it != works_.end();) {
    Watched& w = **it;
    if (w.poll_completed()) {
      if (!w.failed()) w.finish();
      it = works_.erase(it);
    } else if (!async.empty()) {
      const std::string msg = c10::str("eccl watchdog: the communicator reported an asynchronous error while collective (seq ",
                                       w.sequence(), ") was outstanding: ", async);
      w.fail(backend_error(msg));
      if (!bad) *why = msg;
      bad = true;
      it = works_.erase(it);
    } else if (w.timed_out(now)) {
      const std::string msg = c10::str("eccl watchdog: collective (seq ", w.sequence(), ") did not complete within ",
                                       w.timeout().count(), " ms");
      w.fail(backend_error(msg));
      if (!bad) *why = msg;
      bad = true;
      it = works_.erase(it);
    } else {
      ++it;
    }
  }
  if (!bad && !async.empty()) {  // nothing outstanding, but the communicator is broken all the same
    *why = "eccl watchdog: the communicator reported an asynchronous error: " + async;
    bad = true;
  }
  return bad;
}

void WorkWatchdog::run() {
  while (!stop_.load()) {
    std::string why;
    bool bad = false;
    {
      std::unique_lock<std::mutex> lk(mutex_);
      cv_.wait_for(lk, idle_period_, [&] { return stop_.load() || !works_.empty(); });
      if (stop_.load()) break;
      if (failed_.load()) {
        // after the abort nothing new is accepted, and what was still out on the aborted
        // communicator cannot complete any more: it fails with the cause of the abort
        for (auto& w : works_) {
          if (w->poll_completed()) {
            if (!w->failed()) w->finish();
          } else {
            w->fail(backend_error(c10::str("eccl watchdog: collective (seq ", w->sequence(),
                                           ") was outstanding when the communicator was aborted: ", failure_)));
          }
        }
        works_.clear();
      } else {
        bad = sweep(&why);
        if (bad) {
          failure_ = why;
          failed_.store(true);
        }
      }
    }
    if (bad) {
      // outside the lock: the hook takes the process group's own lock and calls into the library
      abort_calls_.fetch_add(1);
      if (abort_hook_) abort_hook_();
    } else {
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  }
}

}  // namespace c10d_gcu
