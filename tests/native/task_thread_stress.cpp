// ThreadSanitizer target for csrc/pg/TaskThread.h: several producers post tasks with gaps that
// straddle the worker's polling window (so that posts land while it polls, while it is about to
// sleep and while it sleeps), every task must run exactly once and in per-producer order, and
// destruction must drain the queue.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <random>
#include <thread>
#include <vector>

#include "pg/TaskThread.h"

int main() {
  constexpr int kProducers = 3, kPerProducer = 400;
  std::atomic<int> ran{0};
  std::vector<int> last(kProducers, -1);  // written only by the worker thread
  std::atomic<int> order_violations{0};
  {
    ccl::TaskThread worker;
    std::vector<std::thread> producers;
    for (int p = 0; p < kProducers; ++p) {
      producers.emplace_back([&, p] {
        std::mt19937 rng(p * 31 + 7);
        for (int i = 0; i < kPerProducer; ++i) {
          worker.post([&, p, i] {
            if (last[p] != i - 1) order_violations.fetch_add(1);
            last[p] = i;
            ran.fetch_add(1);
          });
          const int gap = rng() % 4;  // 0: back to back, 1: inside the polling window, 2: around its end, 3: well after
          if (gap == 1) std::this_thread::sleep_for(std::chrono::microseconds(10));
          if (gap == 2) std::this_thread::sleep_for(std::chrono::microseconds(45 + rng() % 15));
          if (gap == 3) std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
      });
    }
    for (auto& t : producers) t.join();
  }  // ~TaskThread drains
  const bool ok = ran.load() == kProducers * kPerProducer && order_violations.load() == 0;
  std::printf("%s (%d tasks ran, %d order violations)\n", ok ? "PASS" : "FAIL", ran.load(), order_violations.load());
  return ok ? 0 : 1;
}
