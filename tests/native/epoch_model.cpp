// Host-thread model of the device synchronisation protocol of the CUDA collectives, small enough
// to run under ThreadSanitizer: every rank is a thread, its arena halves are plain arrays (so a
// missing happens-before edge is a data race that TSan reports, and a value check fails), its
// flags are std::atomic words written with release and polled with acquire, exactly like
// st.release.sys / ld.acquire.sys on the device.
//
// Modelled rules (csrc/cuda/kernels/comm.cuh, collectives.cu):
//   * flags[phase][source] only ever grow: round r of a kernel that started at epoch e signals
//     e + r + 1 and waiters spin until flag >= e + r + 1 (bounded; a timeout fails the test);
//   * round r uses arena half (e + r) & 1; a kernel of R rounds advances the epoch by R;
//   * one-shot all_reduce: push to every peer, signal all, wait all, reduce locally;
//   * all_gather (pull): stage locally, signal all, wait all, read every peer's half, exit
//     without a trailing synchronisation;
//   * broadcast: root pushes and signals; the others copy out and acknowledge; the root waits
//     for every acknowledgement and then RELEASES the others, who wait for that release;
//   * broadcast through the switch: the root stores into EVERY rank's half (its own included, as
//     multimem.st does), then all ranks signal all and wait for all, like the unrooted kernels,
//     and the others copy out of their own half; no acknowledgement and no release;
//   * low-latency exchange (the fused decode kernels, ll_norm.cuh): every 8-byte unit carries
//     {payload, flag of the round}; a rank stores its units into slot [parity][own rank] of EVERY
//     rank (itself included) and then polls the units of all sources until they carry the flag.
//     No separate flag, no trailing synchronisation: a slot of parity p is rewritten two launches
//     later, which its writer can only reach after the launch in between, whose gather needed a
//     unit from every rank, i.e. after every rank has finished reading the older round. A unit
//     that was overwritten too early would carry a newer flag and the poll would time out.
//     On the device these stores and loads are plain / volatile; what orders them against the
//     NEIGHBOURING kernels is the kernel boundary (a kernel's peer accesses start after
//     griddepcontrol.wait, i.e. after the previous kernel of the stream has completed and flushed).
//     The model has no kernel boundaries, so it gives the unit store release and the unit load
//     acquire semantics to stand for them.
//
// The release step is what makes "a rank has left kernel k" imply "every rank has entered
// kernel k" also for rooted kernels. Without it (run with `norelease`) this sequence corrupts
// data: all_gather, broadcast(root 1), broadcast(root 0) with rank 2 slow inside the all_gather -
// rank 0 gets through both broadcasts and overwrites the half of rank 1 that rank 2 still reads.
// `epoch_model norelease` demonstrates it (exit code 3 = corruption detected, as expected).
//
// The reference argues its protocol by construction only (triple buffering with a counter reset
// one slot ahead, src/gpu/allreduce_small.h:275-285); it has no model or test of it.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <thread>
#include <vector>

namespace {

constexpr int kPhases = 3;
constexpr int kMaxW = 8;
constexpr size_t kSlot = 256;  // words per rank slot inside a half
constexpr size_t kLL = 64;     // 8-byte units per source in a low-latency slot

struct Rank {
  std::vector<uint32_t> half[2];
  std::atomic<uint32_t> flags[kPhases][kMaxW];
  std::vector<std::atomic<uint64_t>> ll[2];  // [parity][source * kLL + unit] = payload | flag << 32
  Rank() : ll{std::vector<std::atomic<uint64_t>>(kLL * kMaxW), std::vector<std::atomic<uint64_t>>(kLL * kMaxW)} {
    for (auto& v : ll)
      for (auto& u : v) u.store(0);
    for (auto& h : half) h.assign(kSlot * kMaxW, 0);
    for (auto& p : flags)
      for (auto& f : p) f.store(0);
  }
};

enum Op { kAllReduce, kAllGather, kBroadcast, kBroadcastSwitch, kLowLatency, kNumOps };
struct Step {
  Op op;
  int root;
  int slow_rank;  // this rank sleeps in the middle of the step (-1: nobody)
};

struct World {
  int W;
  bool release;
  std::vector<Rank> ranks;
  std::atomic<int> failures{0};
  std::atomic<int> timeouts{0};
  World(int w, bool rel) : W(w), release(rel), ranks(w) {}
};

bool wait_flag(World& w, int me, int phase, int src, uint32_t want) {
  const auto t0 = std::chrono::steady_clock::now();
  while (w.ranks[me].flags[phase][src].load(std::memory_order_acquire) < want) {
    if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
      w.timeouts.fetch_add(1);
      return false;
    }
    std::this_thread::yield();
  }
  return true;
}
void signal(World& w, int me, int dst, int phase, uint32_t v) {
  w.ranks[dst].flags[phase][me].store(v, std::memory_order_release);
}

uint32_t payload(int rank, int step, size_t i) { return (uint32_t)(rank * 1000003u + step * 7919u + i); }

void rank_main(World* wp, int me, const std::vector<Step>* prog) {
  World& w = *wp;
  const int W = w.W;
  uint32_t epoch = 0;
  std::mt19937 rng(me * 977 + 5);
  auto jitter = [&] {
    if (rng() % 4 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
  };
  for (size_t s = 0; s < prog->size(); ++s) {
    const Step st = (*prog)[s];
    const int h = epoch & 1;
    const uint32_t tag = epoch + 1;
    jitter();
    if (st.op == kAllReduce) {
      for (int p = 0; p < W; ++p)
        if (p != me)
          for (size_t i = 0; i < kSlot; ++i) w.ranks[p].half[h][me * kSlot + i] = payload(me, (int)s, i);
      for (int p = 0; p < W; ++p)
        if (p != me) signal(w, me, p, 0, tag);
      for (int p = 0; p < W; ++p)
        if (p != me && !wait_flag(w, me, 0, p, tag)) return;
      if (st.slow_rank == me) std::this_thread::sleep_for(std::chrono::milliseconds(30));
      for (size_t i = 0; i < kSlot; ++i) {
        uint32_t acc = payload(me, (int)s, i), want = 0;
        for (int p = 0; p < W; ++p) {
          if (p != me) acc += w.ranks[me].half[h][p * kSlot + i];
          want += payload(p, (int)s, i);
        }
        if (acc != want) w.failures.fetch_add(1);
      }
    } else if (st.op == kAllGather) {
      for (size_t i = 0; i < kSlot; ++i) w.ranks[me].half[h][i] = payload(me, (int)s, i);
      for (int p = 0; p < W; ++p)
        if (p != me) signal(w, me, p, 0, tag);
      for (int p = 0; p < W; ++p)
        if (p != me && !wait_flag(w, me, 0, p, tag)) return;
      for (int q = 1; q < W; ++q) {
        const int p = (me + q) % W;
        if (st.slow_rank == me && q == 1) std::this_thread::sleep_for(std::chrono::milliseconds(60));
        for (size_t i = 0; i < kSlot; ++i)
          if (w.ranks[p].half[h][i] != payload(p, (int)s, i)) w.failures.fetch_add(1);
      }
    } else if (st.op == kLowLatency) {
      for (int p = 0; p < W; ++p)
        for (size_t i = 0; i < kLL; ++i)
          w.ranks[p].ll[h][me * kLL + i].store((uint64_t)payload(me, (int)s, i) | ((uint64_t)tag << 32), std::memory_order_release);
      const auto t0 = std::chrono::steady_clock::now();
      for (int p = 0; p < W; ++p) {
        if (st.slow_rank == me && p == W / 2) std::this_thread::sleep_for(std::chrono::milliseconds(30));
        for (size_t i = 0; i < kLL; ++i) {
          uint64_t u;
          while (((u = w.ranks[me].ll[h][p * kLL + i].load(std::memory_order_acquire)) >> 32) != tag) {
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
              w.timeouts.fetch_add(1);
              return;
            }
            std::this_thread::yield();
          }
          if ((uint32_t)u != payload(p, (int)s, i)) w.failures.fetch_add(1);
        }
      }
    } else if (st.op == kBroadcastSwitch) {
      const int root = st.root;
      if (me == root)
        for (int p = 0; p < W; ++p)
          for (size_t i = 0; i < kSlot; ++i) w.ranks[p].half[h][i] = payload(root, (int)s, i);
      for (int p = 0; p < W; ++p)
        if (p != me) signal(w, me, p, 0, tag);
      for (int p = 0; p < W; ++p)
        if (p != me && !wait_flag(w, me, 0, p, tag)) return;
      if (me != root) {
        if (st.slow_rank == me) std::this_thread::sleep_for(std::chrono::milliseconds(30));
        for (size_t i = 0; i < kSlot; ++i)
          if (w.ranks[me].half[h][i] != payload(root, (int)s, i)) w.failures.fetch_add(1);
      }
    } else {  // broadcast
      const int root = st.root;
      if (me == root) {
        for (int p = 0; p < W; ++p)
          if (p != me)
            for (size_t i = 0; i < kSlot; ++i) w.ranks[p].half[h][i] = payload(root, (int)s, i);
        for (int p = 0; p < W; ++p)
          if (p != me) signal(w, me, p, 0, tag);
        for (int p = 0; p < W; ++p)
          if (p != me && !wait_flag(w, me, 1, p, tag)) return;
        if (w.release)
          for (int p = 0; p < W; ++p)
            if (p != me) signal(w, me, p, 2, tag);
      } else {
        if (!wait_flag(w, me, 0, root, tag)) return;
        if (st.slow_rank == me) std::this_thread::sleep_for(std::chrono::milliseconds(30));
        for (size_t i = 0; i < kSlot; ++i)
          if (w.ranks[me].half[h][i] != payload(root, (int)s, i)) w.failures.fetch_add(1);
        signal(w, me, root, 1, tag);
        if (w.release && !wait_flag(w, me, 2, root, tag)) return;
      }
    }
    epoch += 1;
  }
}

int run(int W, bool release, const std::vector<Step>& prog) {
  World w(W, release);
  std::vector<std::thread> ts;
  for (int r = 0; r < W; ++r) ts.emplace_back(rank_main, &w, r, &prog);
  for (auto& t : ts) t.join();
  if (w.timeouts.load()) return 2;
  return w.failures.load() ? 3 : 0;
}

}  // namespace

int main(int argc, char** argv) {
  const bool norelease = argc > 1 && !std::strcmp(argv[1], "norelease");
  if (norelease) {
    // the minimal sequence that needs the release step (see the header)
    std::vector<Step> prog = {{kAllGather, 0, 2}, {kBroadcast, 1, -1}, {kBroadcast, 0, -1}};
    const int rc = run(3, false, prog);
    std::printf("without the release step: %s\n", rc == 3 ? "corruption detected (expected)" : rc == 0 ? "no corruption seen" : "timeout");
    return rc;
  }
  int bad = 0;
  // the same sequence with the release step, then random programs with random slow ranks
  bad += run(3, true, {{kAllGather, 0, 2}, {kBroadcast, 1, -1}, {kBroadcast, 0, -1}}) != 0;
  // the switch broadcast has no release step and must not need one: slow readers between broadcasts of changing roots
  bad += run(3, true, {{kAllGather, 0, 2}, {kBroadcastSwitch, 1, 2}, {kBroadcastSwitch, 0, 1}, {kBroadcast, 2, 0}, {kBroadcastSwitch, 2, 0},
                       {kAllReduce, 0, 1}, {kBroadcastSwitch, 1, -1}}) != 0;
  // low-latency exchanges back to back (decode: two per layer) with slow readers, then mixed with the staged kernels
  bad += run(4, true, {{kLowLatency, 0, 1}, {kLowLatency, 0, 2}, {kLowLatency, 0, 1}, {kLowLatency, 0, 3}, {kAllGather, 0, 0},
                       {kLowLatency, 0, 2}, {kBroadcastSwitch, 3, 1}, {kLowLatency, 0, 0}, {kLowLatency, 0, 3}}) != 0;
  std::mt19937 rng(1234);
  for (int W : {2, 3, 5, 8}) {
    for (int trial = 0; trial < 6; ++trial) {
      std::vector<Step> prog;
      for (int s = 0; s < 40; ++s) prog.push_back({(Op)(rng() % kNumOps), (int)(rng() % W), (rng() % 5 == 0) ? (int)(rng() % W) : -1});
      const int rc = run(W, true, prog);
      if (rc) std::printf("world %d trial %d: rc %d\n", W, trial, rc);
      bad += rc != 0;
    }
  }
  std::printf("%s\n", bad == 0 ? "PASS" : "FAIL");
  return bad == 0 ? 0 : 1;
}
