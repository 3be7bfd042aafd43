// Shared-memory communicator for CPU tensors: one POSIX shm segment per process group, holding a
// sequence-number barrier, two staging slots per rank (used alternately so that a fast rank can
// start the next step while a slow one still reads the previous one) and one ring channel per
// ordered pair of ranks for send/recv.
//
// This is the host-side replacement of the oneCCL host transport behind the reference's
// VanillaCPU stub (src/cpu/cpu_ccl.cpp:66-92 creates a oneCCL communicator from a KVS address
// carried by the c10d Store). Here the Store carries the shm segment name; ranks must share a
// host. Every wait has a deadline; on expiry an abort flag is raised so that the other ranks
// fail fast instead of hanging.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

namespace ccl {
namespace cpu {

constexpr int kMaxCpuRanks = 64;

struct ShmStore {
  std::function<void(const std::string&, const std::vector<uint8_t>&)> set;
  std::function<std::vector<uint8_t>(const std::string&)> get;
  std::function<int64_t(const std::string&, int64_t)> add;
};

class ShmTimeout : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

class ShmComm {
 public:
  ShmComm(ShmStore store, int rank, int world, size_t slot_bytes, std::chrono::milliseconds init_timeout);
  ~ShmComm();
  ShmComm(const ShmComm&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }
  size_t slot_bytes() const { return slot_bytes_; }

  // Staging slot of rank r for the current step (parity advances with next_step()).
  char* slot(int r) const;
  uint64_t* scratch() const;  // world uint64 words of the current step, one per rank
  void next_step() { ++step_; }
  // All ranks arrive; throws ShmTimeout after `timeout` or when another rank aborted.
  void barrier(std::chrono::milliseconds timeout);
  void abort();
  bool aborted() const;

  // Blocking point-to-point transfers through the (src,dst) ring channel.
  void send(const void* buf, size_t bytes, int dst, std::chrono::milliseconds timeout);
  void recv(void* buf, size_t bytes, int src, std::chrono::milliseconds timeout);

 private:
  struct Header;
  struct Channel;
  Channel* channel(int src, int dst) const;

  int rank_, world_;
  size_t slot_bytes_;
  size_t chan_bytes_;
  size_t total_bytes_ = 0;
  char* base_ = nullptr;
  Header* hdr_ = nullptr;
  char* slots_ = nullptr;
  char* chans_ = nullptr;
  uint64_t seq_ = 0;
  uint64_t step_ = 0;
  std::string name_;
};

}  // namespace cpu
}  // namespace ccl
