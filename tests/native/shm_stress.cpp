// Sanitizer target for the CPU shared-memory backend: the ranks are THREADS of one process, each
// with its own ShmComm (own mapping of the same POSIX segment) bootstrapped through an in-process
// key-value store, running a mixed sequence of every collective plus ring send/recv with value
// checks. Built twice by tests/test_native_probes.py: with -fsanitize=address,undefined (buffer
// overruns in the staging copies, misaligned or overflowing arithmetic) and with
// -fsanitize=thread (the bootstrap, barrier and channel code; accesses through two different
// mappings of the segment are outside what ThreadSanitizer can relate).
//
// The reference builds without any sanitizer (CMakeLists.txt:5-8 of intel/torch-ccl adds only
// -fstack-protector and -Wformat-security) and has no native test of its CPU path.
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "cpu/CpuCollectives.h"
#include "cuda/kernels/collectives.h"

namespace {

using namespace ccl::cpu;

struct MemStore {
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, std::vector<uint8_t>> kv;
  std::map<std::string, int64_t> counters;

  ShmStore handle() {
    ShmStore s;
    s.set = [this](const std::string& k, const std::vector<uint8_t>& v) {
      std::lock_guard<std::mutex> g(mu);
      kv[k] = v;
      cv.notify_all();
    };
    s.get = [this](const std::string& k) {
      std::unique_lock<std::mutex> g(mu);
      cv.wait(g, [&] { return kv.count(k) > 0; });
      return kv[k];
    };
    s.add = [this](const std::string& k, int64_t d) {
      std::lock_guard<std::mutex> g(mu);
      counters[k] += d;
      return counters[k];
    };
    return s;
  }
};

std::atomic<int> g_failures{0};

#define EXPECT(cond, ...)                       \
  do {                                          \
    if (!(cond)) {                              \
      std::fprintf(stderr, "FAILED: " __VA_ARGS__); \
      std::fprintf(stderr, "\n");               \
      g_failures.fetch_add(1);                  \
    }                                           \
  } while (0)

float val(int rank, size_t i, int step) { return (float)((i % 7) + rank + 1 + (step % 3)); }

void rank_main(MemStore* store, int rank, int world, int rounds) {
  const Ms tmo(20000);
  ShmComm comm(store->handle(), rank, world, /*slot_bytes=*/64 << 10, tmo);
  ReduceDesc sum{ccl::kF32, ccl::kSum};
  const size_t sizes[] = {1, 7, 1000, 16384, 16385, 50000};  // 64 KB slots: the last two need several rounds
  for (int step = 0; step < rounds; ++step) {
    const size_t n = sizes[step % 6];
    // all_reduce
    std::vector<float> x(n);
    for (size_t i = 0; i < n; ++i) x[i] = val(rank, i, step);
    allreduce(comm, x.data(), n, sum, tmo);
    for (size_t i = 0; i < n; i += 97) {
      float want = 0;
      for (int r = 0; r < world; ++r) want += val(r, i, step);
      EXPECT(x[i] == want, "allreduce step %d n %zu i %zu: %f != %f", step, n, i, x[i], want);
    }
    // broadcast from a rotating root
    const int root = step % world;
    std::vector<float> b(n, (float)rank);
    if (rank == root)
      for (size_t i = 0; i < n; ++i) b[i] = val(root, i, step);
    broadcast(comm, b.data(), n * sizeof(float), root, tmo);
    EXPECT(b[n - 1] == val(root, n - 1, step), "broadcast step %d", step);
    // all_gather with uneven pieces (rank r contributes n + r elements)
    std::vector<std::vector<float>> pieces(world);
    std::vector<void*> outs(world);
    std::vector<size_t> bytes(world);
    for (int r = 0; r < world; ++r) {
      pieces[r].assign(n + r, -1.f);
      outs[r] = pieces[r].data();
      bytes[r] = (n + r) * sizeof(float);
    }
    std::vector<float> mine(n + rank);
    for (size_t i = 0; i < mine.size(); ++i) mine[i] = val(rank, i, step);
    allgatherv(comm, mine.data(), outs, bytes, tmo);
    for (int r = 0; r < world; ++r) EXPECT(pieces[r].back() == val(r, n + r - 1, step), "allgatherv step %d from %d", step, r);
    // reduce_scatter: piece p has n + p elements
    std::vector<std::vector<float>> rs_in(world);
    std::vector<const void*> rs_ptr(world);
    std::vector<size_t> counts(world);
    for (int p = 0; p < world; ++p) {
      rs_in[p].resize(n + p);
      for (size_t i = 0; i < rs_in[p].size(); ++i) rs_in[p][i] = val(rank, i + p, step);
      rs_ptr[p] = rs_in[p].data();
      counts[p] = n + p;
    }
    std::vector<float> rs_out(n + rank, 0.f);
    reduce_scatterv(comm, rs_ptr, rs_out.data(), counts, sum, tmo);
    {
      float want = 0;
      for (int r = 0; r < world; ++r) want += val(r, (n + rank - 1) + rank, step);
      EXPECT(rs_out.back() == want, "reduce_scatterv step %d: %f != %f", step, rs_out.back(), want);
    }
    // all_to_all: rank r sends (r + p + 1) * 3 floats to rank p
    std::vector<std::vector<float>> a_in(world), a_out(world);
    std::vector<const void*> a_inp(world);
    std::vector<void*> a_outp(world);
    std::vector<size_t> sb(world), rb(world);
    for (int p = 0; p < world; ++p) {
      a_in[p].assign((size_t)(rank + p + 1) * 3, (float)(rank * 100 + p));
      a_out[p].assign((size_t)(p + rank + 1) * 3, -1.f);
      a_inp[p] = a_in[p].data();
      a_outp[p] = a_out[p].data();
      sb[p] = a_in[p].size() * sizeof(float);
      rb[p] = a_out[p].size() * sizeof(float);
    }
    alltoallv(comm, a_inp, sb, a_outp, rb, tmo);
    for (int p = 0; p < world; ++p) EXPECT(a_out[p].back() == (float)(p * 100 + rank), "alltoallv step %d from %d", step, p);
    // ring send / recv (even ranks send first)
    if (world > 1) {
      const int next = (rank + 1) % world, prev = (rank + world - 1) % world;
      std::vector<float> out(n, (float)rank + 0.5f), in(n, -1.f);
      if (rank % 2 == 0) {
        comm.send(out.data(), n * sizeof(float), next, tmo);
        comm.recv(in.data(), n * sizeof(float), prev, tmo);
      } else {
        comm.recv(in.data(), n * sizeof(float), prev, tmo);
        comm.send(out.data(), n * sizeof(float), next, tmo);
      }
      EXPECT(in[n - 1] == (float)prev + 0.5f, "ring step %d", step);
    }
    barrier(comm, tmo);
  }
}

}  // namespace

int main(int argc, char** argv) {
  const int world = argc > 1 ? std::atoi(argv[1]) : 4;
  const int rounds = argc > 2 ? std::atoi(argv[2]) : 24;
  MemStore store;
  std::vector<std::thread> ts;
  for (int r = 0; r < world; ++r) ts.emplace_back(rank_main, &store, r, world, rounds);
  for (auto& t : ts) t.join();
  std::printf("%s (%d ranks, %d rounds, %d failures)\n", g_failures.load() == 0 ? "PASS" : "FAIL", world, rounds, g_failures.load());
  return g_failures.load() == 0 ? 0 : 1;
}
