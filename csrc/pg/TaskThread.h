// A FIFO worker thread: tasks run in submission order on one background thread. The CPU backend
// uses one for collectives (all ranks issue them in the same order) and one per peer and
// direction for point-to-point transfers. The reference keeps one such thread per device stub
// (src/cpu/cpu_ccl.cpp:255-304), but runs the op on the caller thread and only waits on the
// worker; here the whole op runs on the worker, so issuing a collective never blocks the caller.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>

namespace ccl {

class TaskThread {
 public:
  TaskThread() : th_([this] { loop(); }) {}
  ~TaskThread() { drain_and_stop(); }

  void post(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> g(mu_);
      q_.push_back(std::move(fn));
      pending_.fetch_add(1, std::memory_order_release);
    }
    // a worker that is still polling (see loop) picks the task up without a futex wake
    if (!polling_.load(std::memory_order_acquire)) cv_.notify_all();
  }

  void drain_and_stop() {
    {
      std::unique_lock<std::mutex> l(mu_);
      if (stopped_) return;
      stop_ = true;
    }
    cv_.notify_all();
    if (th_.joinable()) th_.join();
    stopped_ = true;
  }

 private:
  void loop() {
    std::unique_lock<std::mutex> l(mu_);
    while (true) {
      if (q_.empty() && !stop_) {
        // Collectives usually arrive back to back: poll for the next one for a few tens of
        // microseconds before sleeping, which saves the wake-up latency of the condition
        // variable (the larger part of a small collective's cost).
        polling_.store(true, std::memory_order_release);
        l.unlock();
        const auto t0 = std::chrono::steady_clock::now();
        while (pending_.load(std::memory_order_acquire) == 0 &&
               std::chrono::steady_clock::now() - t0 < std::chrono::microseconds(kPollMicros)) {
#if defined(__x86_64__)
          __builtin_ia32_pause();
#endif
        }
        l.lock();
        polling_.store(false, std::memory_order_release);
      }
      cv_.wait(l, [this] { return stop_ || !q_.empty(); });
      if (q_.empty()) {
        if (stop_) return;
        continue;
      }
      auto fn = std::move(q_.front());
      q_.pop_front();
      pending_.fetch_sub(1, std::memory_order_relaxed);
      l.unlock();
      fn();  // tasks catch their own exceptions
      l.lock();
    }
  }

  static constexpr int kPollMicros = 50;
  std::atomic<int> pending_{0};
  std::atomic<bool> polling_{false};
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void()>> q_;
  bool stop_ = false;
  bool stopped_ = false;
  std::thread th_;
};

}  // namespace ccl
