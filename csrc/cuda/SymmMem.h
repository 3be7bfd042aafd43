// Symmetric memory: one device allocation per rank that every other rank of the node maps into
// its own address space, so that kernels can load, store and reduce over NVLink directly.
//
// Two transports for the memory handles:
//   * kIpc — `cudaIpcGetMemHandle` blobs published through the key-value store (default);
//   * kVmm — the allocation is a driver virtual-memory object (`cuMemCreate`), exported as a POSIX
//     file descriptor and handed to each peer over a UNIX-domain socket with SCM_RIGHTS. This is
//     the form an NVLink multicast object can later be bound to.
//
// Counterpart of the reference's `exchange_peer_ipc_mem` (src/gpu/allreduce.h:1208-1248), which
// turns a Level-Zero IPC handle into a file descriptor and all-gathers the descriptors with
// `un_allgather` over UNIX sockets (src/gpu/allreduce.h:216-390), synchronising with MPI_Barrier.
// Here the socket names travel through the c10d Store and no MPI is involved.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace ccl {

struct KvStore {
  std::function<void(const std::string&, const std::vector<uint8_t>&)> set;
  std::function<std::vector<uint8_t>(const std::string&)> get;  // blocks until the key exists
  std::function<int64_t(const std::string&, int64_t)> add;      // atomic counter
};

// Blocks until `world` ranks have arrived at `key` (no-op without a store).
void barrier_kv(KvStore& kv, const std::string& key, int world, uint64_t timeout_ms);

// All-gather of one file descriptor per rank between the processes of one node.
// Returns `world` descriptors; entry [rank] is a duplicate of `my_fd`. The caller closes them.
// Every rank listens on an abstract-namespace UNIX socket whose name it publishes under
// `<prefix>/fdsock/<rank>`, connects to every peer, sends {rank, fd} and then accepts world-1
// messages. Connections complete against the listen backlog, so no rank blocks another.
std::vector<int> exchange_fds(KvStore& kv, const std::string& prefix, int rank, int world, int my_fd,
                              uint64_t timeout_ms);

enum class SymmKind : int { kIpc = 0, kVmm = 1 };
SymmKind parse_symm_kind(const std::string& s);  // "ipc" | "vmm"

class SymmMem {
 public:
  // Collective over the `world` processes of `kv` (world == 1 allocates locally only).
  // The memory is zeroed before any peer can see it.
  // `multicast`: additionally bind all ranks' allocations to one NVLink multicast object (NVLS) and
  // map it, so that `multimem` instructions can reduce over / store to every rank's copy at once.
  // Needs kVmm and at least two ranks (the driver refuses a one-device object); silently left off
  // when the device does not report multicast support.
  SymmMem(SymmKind kind, int rank, int world, int device, size_t bytes, KvStore& kv, const std::string& prefix,
          bool multicast = false);
  ~SymmMem();
  SymmMem(const SymmMem&) = delete;
  SymmMem& operator=(const SymmMem&) = delete;

  void* local() const { return bases_[rank_]; }
  void* peer(int p) const { return bases_[p]; }
  const std::vector<void*>& bases() const { return bases_; }
  size_t bytes() const { return bytes_; }        // requested size
  size_t mapped_bytes() const { return mapped_; }  // rounded up to the allocation granularity
  SymmKind kind() const { return kind_; }
  // Multicast mapping of the allocation (same layout; nullptr when not enabled / not supported).
  void* multicast_base() const { return mc_base_; }
  static bool multicast_supported(int device);

 private:
  void init_ipc(KvStore& kv, const std::string& prefix);
  void init_vmm(KvStore& kv, const std::string& prefix, bool multicast);
  void init_multicast(KvStore& kv, const std::string& prefix, size_t gran);
  void init_multicast_impl(KvStore& kv, const std::string& prefix, size_t gran);
  void release_multicast();

  SymmKind kind_;
  int rank_, world_, device_;
  size_t bytes_ = 0, mapped_ = 0;
  std::vector<void*> bases_;
  std::vector<unsigned long long> handles_;  // kVmm: CUmemGenericAllocationHandle per rank
  unsigned long long mc_handle_ = 0;         // multicast object (0: none)
  void* mc_base_ = nullptr;
  bool mc_bound_ = false;
};

}  // namespace ccl
