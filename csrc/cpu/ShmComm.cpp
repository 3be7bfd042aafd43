#include "cpu/ShmComm.h"

#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstddef>
#include <cstring>
#include <random>
#include <stdexcept>
#include <thread>

namespace ccl {
namespace cpu {

namespace {
constexpr size_t kCacheLine = 64;
constexpr size_t kChanSlots = 2;

struct alignas(kCacheLine) PaddedCounter {
  std::atomic<uint64_t> v;
  char pad[kCacheLine - sizeof(std::atomic<uint64_t>)];
};

inline void backoff(uint32_t& spins) {
  ++spins;
  if (spins < 200) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  } else if (spins < 2000) {
    sched_yield();
  } else {
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}
}  // namespace

struct ShmComm::Header {
  std::atomic<uint32_t> abort;
  char pad0[kCacheLine - sizeof(std::atomic<uint32_t>)];
  PaddedCounter arrive[kMaxCpuRanks];
  uint64_t scratch[2][kMaxCpuRanks];
};

struct ShmComm::Channel {
  alignas(kCacheLine) std::atomic<uint64_t> head;  // chunks published by the sender
  alignas(kCacheLine) std::atomic<uint64_t> tail;  // chunks consumed by the receiver
  alignas(kCacheLine) uint64_t len[kChanSlots];
  alignas(kCacheLine) char data[1];
};

ShmComm::ShmComm(ShmStore store, int rank, int world, size_t slot_bytes, std::chrono::milliseconds init_timeout)
    : rank_(rank), world_(world), slot_bytes_((slot_bytes + 4095) / 4096 * 4096) {
  if (world < 1 || world > kMaxCpuRanks) throw std::runtime_error("ccl: CPU communicators support up to 64 ranks");
  chan_bytes_ = 256 << 10;
  const size_t hdr_bytes = (sizeof(Header) + 4095) / 4096 * 4096;
  const size_t slots_bytes = 2 * slot_bytes_ * world_;
  const size_t chan_stride = (offsetof(Channel, data) + kChanSlots * chan_bytes_ + 4095) / 4096 * 4096;
  total_bytes_ = hdr_bytes + slots_bytes + chan_stride * world_ * world_;

  int fd = -1;
  if (rank_ == 0) {
    std::random_device rd;
    name_ = "/ccl-" + std::to_string(getpid()) + "-" + std::to_string(rd()) + std::to_string(rd());
    fd = shm_open(name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("ccl: shm_open(create) failed: " + std::string(strerror(errno)));
    if (ftruncate(fd, (off_t)total_bytes_) != 0) {
      close(fd);
      shm_unlink(name_.c_str());
      throw std::runtime_error("ccl: ftruncate(shm) failed: " + std::string(strerror(errno)));
    }
    store.set("shm/name", std::vector<uint8_t>(name_.begin(), name_.end()));
  } else {
    auto v = store.get("shm/name");
    name_ = std::string(v.begin(), v.end());
    fd = shm_open(name_.c_str(), O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("ccl: shm_open(" + name_ + ") failed: " + std::string(strerror(errno)) +
                                         " (CPU ranks must share a host)");
  }
  void* p = mmap(nullptr, total_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("ccl: mmap(shm) failed: " + std::string(strerror(errno)));
  base_ = static_cast<char*>(p);
  hdr_ = reinterpret_cast<Header*>(base_);  // a fresh segment is zero-filled: counters start at 0
  slots_ = base_ + hdr_bytes;
  chans_ = slots_ + slots_bytes;

  // everyone has mapped the segment -> the name can disappear (no stale segment after a crash)
  store.add("shm/mapped", 1);
  const auto t0 = std::chrono::steady_clock::now();
  int64_t mapped = 0;
  while ((mapped = store.add("shm/mapped", 0)) < world_) {
    if (std::chrono::steady_clock::now() - t0 > init_timeout) {
      if (rank_ == 0) shm_unlink(name_.c_str());
      munmap(base_, total_bytes_);  // the destructor does not run for an object whose constructor throws
      base_ = nullptr;
      throw ShmTimeout("ccl: communicator bring-up timed out after " + std::to_string(init_timeout.count()) + " ms on rank " +
                       std::to_string(rank_) + ": " + std::to_string(mapped) + " of " + std::to_string(world_) +
                       " ranks mapped the shared-memory segment (does every rank of the group run and reach its first CPU collective?)");
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  if (rank_ == 0) shm_unlink(name_.c_str());
}

ShmComm::~ShmComm() {
  if (base_) munmap(base_, total_bytes_);
}

char* ShmComm::slot(int r) const { return slots_ + ((size_t)(step_ & 1) * world_ + r) * slot_bytes_; }
uint64_t* ShmComm::scratch() const { return hdr_->scratch[step_ & 1]; }

void ShmComm::abort() { hdr_->abort.store(1, std::memory_order_release); }
bool ShmComm::aborted() const { return hdr_->abort.load(std::memory_order_acquire) != 0; }

void ShmComm::barrier(std::chrono::milliseconds timeout) {
  ++seq_;
  hdr_->arrive[rank_].v.store(seq_, std::memory_order_release);
  const auto t0 = std::chrono::steady_clock::now();
  for (int p = 0; p < world_; ++p) {
    uint32_t spins = 0;
    while (hdr_->arrive[p].v.load(std::memory_order_acquire) < seq_) {
      if (aborted()) throw ShmTimeout("ccl: communicator aborted by another rank");
      if ((spins & 255) == 255 && std::chrono::steady_clock::now() - t0 > timeout) {
        abort();
        throw ShmTimeout("Caught collective operation timeout: rank " + std::to_string(rank_) +
                         " waited for rank " + std::to_string(p) + " for " + std::to_string(timeout.count()) + " ms");
      }
      backoff(spins);
    }
  }
}

ShmComm::Channel* ShmComm::channel(int src, int dst) const {
  const size_t chan_stride = (offsetof(Channel, data) + kChanSlots * chan_bytes_ + 4095) / 4096 * 4096;
  return reinterpret_cast<Channel*>(chans_ + ((size_t)src * world_ + dst) * chan_stride);
}

void ShmComm::send(const void* buf, size_t bytes, int dst, std::chrono::milliseconds timeout) {
  Channel* ch = channel(rank_, dst);
  const char* p = static_cast<const char*>(buf);
  size_t left = bytes;
  const auto t0 = std::chrono::steady_clock::now();
  do {  // a zero-byte message still hands over one (empty) chunk
    const size_t n = left < chan_bytes_ ? left : chan_bytes_;
    const uint64_t h = ch->head.load(std::memory_order_relaxed);
    uint32_t spins = 0;
    while (h - ch->tail.load(std::memory_order_acquire) >= kChanSlots) {
      if (aborted()) throw ShmTimeout("ccl: communicator aborted by another rank");
      if ((spins & 255) == 255 && std::chrono::steady_clock::now() - t0 > timeout)
        throw ShmTimeout("Caught collective operation timeout: send to rank " + std::to_string(dst));
      backoff(spins);
    }
    std::memcpy(ch->data + (h % kChanSlots) * chan_bytes_, p, n);
    ch->len[h % kChanSlots] = n;
    ch->head.store(h + 1, std::memory_order_release);
    p += n;
    left -= n;
  } while (left > 0);
}

void ShmComm::recv(void* buf, size_t bytes, int src, std::chrono::milliseconds timeout) {
  Channel* ch = channel(src, rank_);
  char* p = static_cast<char*>(buf);
  size_t left = bytes;
  const auto t0 = std::chrono::steady_clock::now();
  do {
    const uint64_t t = ch->tail.load(std::memory_order_relaxed);
    uint32_t spins = 0;
    while (ch->head.load(std::memory_order_acquire) <= t) {
      if (aborted()) throw ShmTimeout("ccl: communicator aborted by another rank");
      if ((spins & 255) == 255 && std::chrono::steady_clock::now() - t0 > timeout)
        throw ShmTimeout("Caught collective operation timeout: recv from rank " + std::to_string(src));
      backoff(spins);
    }
    const size_t n = ch->len[t % kChanSlots];
    if (n > left) throw std::runtime_error("ccl: recv: message from rank " + std::to_string(src) + " is larger than the receive buffer");
    std::memcpy(p, ch->data + (t % kChanSlots) * chan_bytes_, n);
    ch->tail.store(t + 1, std::memory_order_release);
    p += n;
    left -= n;
    if (n < chan_bytes_ && left > 0)
      throw std::runtime_error("ccl: recv: message from rank " + std::to_string(src) + " is smaller than the receive buffer");
  } while (left > 0);
}

}  // namespace cpu
}  // namespace ccl
