// Observability of the backend: the verbose per-op tracer (same line format as the reference's
// DebugCCLStub, src/dispatch_stub.cpp:61-119), per-op statistics and a flight recorder ring of
// the most recent operations that is dumped when a collective times out. The reference has only
// the tracer (stdout); statistics and the flight recorder have no counterpart there.
#pragma once
#include <ATen/ATen.h>

#include <array>
#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace ccl {

// "(cpu, [3, 1000])" / "[(cuda:0, [4]), ...]" like the reference's format_tensors_size.
void format_tensors(std::ostream& os, const at::Tensor& t);
void format_tensors(std::ostream& os, const std::vector<at::Tensor>& v);
void format_tensors(std::ostream& os, const std::vector<std::vector<at::Tensor>>& v);

// RAII tracer of one op. Prints
//   oneccl_bindings_for_pytorch::<dev>::<op>: [rank/size#seq] [a->b] <tensors>
// at construction and the same line followed by " Time elapsed (ms): x" at destruction,
// when ONECCL_BINDINGS_FOR_PYTORCH_ENV_VERBOSE is non-zero.
class OpTrace {
 public:
  OpTrace(bool enabled, const char* dev, const char* op, int rank, int size, uint64_t seq,
          const std::string& flow, const std::string& tensors);
  ~OpTrace();

 private:
  bool enabled_;
  std::string line_;
  std::chrono::steady_clock::time_point t0_;
};

struct OpStat {
  uint64_t count = 0;
  uint64_t bytes = 0;
  double host_us_total = 0;
  std::array<uint64_t, 24> host_us_hist{};  // bucket i: [2^i, 2^(i+1)) microseconds
  std::map<std::string, uint64_t> algos;
};

struct FlightEntry {
  uint64_t seq = 0;
  const char* op = "";      // string literals: recording an op allocates nothing
  const char* device = "";
  uint64_t bytes = 0;
  char algo[16] = {0};
  double t_enqueue_us = 0;   // since process start
  double t_complete_us = -1;  // -1: not completed yet
};

class Telemetry {
 public:
  static Telemetry& get();
  // Returns the slot index of the flight-recorder entry.
  // `op` and `device` must be string literals (their addresses are kept).
  size_t record_start(uint64_t seq, const char* op, const char* device, uint64_t bytes, const char* algo);
  void record_host_time(const char* op, const char* device, uint64_t bytes, const char* algo, double host_us);
  void record_complete(size_t slot, uint64_t seq);
  std::map<std::string, OpStat> stats() const;
  std::vector<FlightEntry> flight() const;
  std::string dump_flight() const;
  void reset();
  static double now_us();

 private:
  static constexpr size_t kRing = 256;
  mutable std::mutex mu_;
  std::map<std::pair<const char*, const char*>, OpStat> stats_;  // keyed by literal addresses
  std::array<FlightEntry, kRing> ring_;
  size_t next_ = 0;
  size_t filled_ = 0;
};

}  // namespace ccl
