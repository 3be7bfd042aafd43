#include "pg/Telemetry.h"

#include <cmath>
#include <cstdio>
#include <iostream>

namespace ccl {

void format_tensors(std::ostream& os, const at::Tensor& t) {
  os << "(" << t.device() << ", " << t.sizes() << ")";
}
void format_tensors(std::ostream& os, const std::vector<at::Tensor>& v) {
  os << "[";
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) os << ", ";
    format_tensors(os, v[i]);
  }
  os << "]";
}
void format_tensors(std::ostream& os, const std::vector<std::vector<at::Tensor>>& v) {
  os << "[";
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) os << ", ";
    format_tensors(os, v[i]);
  }
  os << "]";
}

OpTrace::OpTrace(bool enabled, const char* dev, const char* op, int rank, int size, uint64_t seq,
                 const std::string& flow, const std::string& tensors)
    : enabled_(enabled) {
  if (!enabled_) return;
  std::stringstream os;
  os << "oneccl_bindings_for_pytorch::" << dev << "::" << op << ": [" << rank << "/" << size << "#" << seq << "]";
  if (!flow.empty()) os << " " << flow;
  os << " " << tensors;
  line_ = os.str();
  std::cout << line_ << std::endl;
  t0_ = std::chrono::steady_clock::now();
}

OpTrace::~OpTrace() {
  if (!enabled_) return;
  const auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0_);
  std::cout << line_ << " Time elapsed (ms): " << us.count() / 1000.0F << std::endl;
}

Telemetry& Telemetry::get() {
  static Telemetry* t = new Telemetry();  // intentionally leaked: used from worker threads at exit
  return *t;
}

double Telemetry::now_us() {
  static const auto t0 = std::chrono::steady_clock::now();
  return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
}

size_t Telemetry::record_start(uint64_t seq, const char* op, const char* device, uint64_t bytes,
                               const char* algo) {
  std::lock_guard<std::mutex> g(mu_);
  const size_t slot = next_;
  FlightEntry& e = ring_[slot];
  e.seq = seq;
  e.op = op;
  e.device = device;
  e.bytes = bytes;
  std::snprintf(e.algo, sizeof(e.algo), "%s", algo ? algo : "");
  e.t_enqueue_us = now_us();
  e.t_complete_us = -1;
  next_ = (next_ + 1) % kRing;
  if (filled_ < kRing) ++filled_;
  return slot;
}

void Telemetry::record_host_time(const char* op, const char* device, uint64_t bytes, const char* algo,
                                 double host_us) {
  std::lock_guard<std::mutex> g(mu_);
  OpStat& s = stats_[std::make_pair(device, op)];
  s.count++;
  s.bytes += bytes;
  s.host_us_total += host_us;
  int b = host_us < 1 ? 0 : (int)std::floor(std::log2(host_us));
  if (b > 23) b = 23;
  s.host_us_hist[b]++;
  if (algo && algo[0]) s.algos[algo]++;
}

void Telemetry::record_complete(size_t slot, uint64_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  if (slot < kRing && ring_[slot].seq == seq) ring_[slot].t_complete_us = now_us();
}

std::map<std::string, OpStat> Telemetry::stats() const {
  std::lock_guard<std::mutex> g(mu_);
  std::map<std::string, OpStat> out;
  for (const auto& kv : stats_) {
    OpStat& d = out[std::string(kv.first.first) + "::" + kv.first.second];
    d.count += kv.second.count;
    d.bytes += kv.second.bytes;
    d.host_us_total += kv.second.host_us_total;
    for (size_t i = 0; i < d.host_us_hist.size(); ++i) d.host_us_hist[i] += kv.second.host_us_hist[i];
    for (const auto& a : kv.second.algos) d.algos[a.first] += a.second;
  }
  return out;
}

std::vector<FlightEntry> Telemetry::flight() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<FlightEntry> out;
  const size_t start = (next_ + kRing - filled_) % kRing;
  for (size_t i = 0; i < filled_; ++i) out.push_back(ring_[(start + i) % kRing]);
  return out;
}

std::string Telemetry::dump_flight() const {
  std::stringstream os;
  os << "ccl flight recorder (oldest first):\n";
  for (const auto& e : flight()) {
    os << "  #" << e.seq << " " << e.device << "::" << e.op << " bytes=" << e.bytes;
    if (e.algo[0]) os << " algo=" << e.algo;
    os << " enqueued@" << (uint64_t)e.t_enqueue_us << "us";
    if (e.t_complete_us >= 0) os << " completed@" << (uint64_t)e.t_complete_us << "us";
    else os << " NOT COMPLETED";
    os << "\n";
  }
  return os.str();
}

void Telemetry::reset() {
  std::lock_guard<std::mutex> g(mu_);
  stats_.clear();
  filled_ = 0;
  next_ = 0;
}

}  // namespace ccl
