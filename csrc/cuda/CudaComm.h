// Host side of one CUDA communicator: the peer-mapped arena of every rank ("symmetric memory"),
// the bootstrap that exchanges memory handles through a key-value store, algorithm selection
// and the launch wrappers of every collective kernel.
//
// Counterpart of the reference's IPC bring-up (`exchange_peer_ipc_mem`,
// src/gpu/allreduce.h:1208-1248, which all-gathers Level-Zero IPC handles over UNIX sockets and
// needs MPI_Barrier) and of its per-op branches in src/gpu/dpcpp_ccl.cpp:731-1656. Here the
// handles travel through the c10d Store (cudaIpc) or over UNIX sockets (driver virtual-memory
// objects), see SymmMem.h; no MPI is involved.
//
// A CudaComm is either *real* (one process per GPU; nctx() == 1) or *emulated* (all ranks'
// arenas on one GPU and one cooperative launch per collective; nctx() == world) — the latter
// exists so that every kernel can be tested on a single GPU.
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "cuda/SymmMem.h"
#include "cuda/kernels/collectives.h"
#include "cuda/kernels/collectives_multi.h"
#include "cuda/kernels/collectives_symm.h"
#include "cuda/kernels/decode_fused.h"
#include "cuda/kernels/gemm_collective.h"
#include "cuda/kernels/moe_a2a.h"

namespace ccl {

enum class Algo : int { kAuto = 0, kOneShot = 1, kTwoShot = 2, kNvls = 3 };

struct CommConfig {
  size_t half_bytes = 256ull << 20;   // one staging half per rank (arena = 2 halves + flags)
  uint64_t spin_timeout_ms = 30000;   // device-side wait budget
  size_t oneshot_max_bytes = 0;        // 0: pick from the world size (see default_oneshot_max)
  size_t ag_push_max_bytes = 0;        // per-piece size up to which all_gather pushes (0: built-in, 2 MB)
  int max_blocks = 256;               // CTAs for bandwidth-bound collectives
  int threads = 512;
  Algo algo = Algo::kAuto;
  int ablate = kAblateNone;
  SymmKind symm = SymmKind::kIpc;     // how the arenas are shared (CCL_SYMM_MEM = ipc | vmm)
  // NVLS: bind the arenas to an NVLink multicast object (needs symm = kVmm and device support) and
  // route SUM all_reduces of bf16 / f16 / f32 of at least nvls_min_bytes through the switch.
  bool nvls = false;                  // CCL_NVLS
  size_t nvls_min_bytes = (size_t)-1;  // -1: built-in (2 MB, measured at 8 ranks: the staged switch kernel wins from there, 28 vs 40 us; never for two ranks)
  // Symmetric heap: memory for user tensors that every rank maps (allocate through the backend's
  // allocateTensor / symm_empty). Collectives on such tensors run zero-copy: no staging through the
  // arena. Created at the first allocation; bound to a multicast object when `nvls` is set.
  size_t heap_bytes = 1ull << 30;     // CCL_SYMM_HEAP_MB
  // smaller symmetric messages still take the staged one-shot kernel. Measured at 8 ranks: zero-copy 16.9 us
  // against 18.7 us at 512 KB, 17.6 against 24.5 us at 1 MB, 36.6 against 48.4 us at 8 MB; below 512 KB a tie.
  // (2 ranks: the staged one-shot kernel stays ahead up to 16 MB; a tuning file can raise the threshold there.)
  // Caps on the bytes one staging round moves per rank (0: the arena half; -1: built-in, see apply_builtin_thresholds).
  // Setting round_bytes (CCL_ROUND_MB) also sets the two special cases that are left at -1.
  size_t round_bytes = (size_t)-1;          // peer-memory kernels (built-in 128 MB)
  size_t nvls_round_bytes = (size_t)-1;     // staged switch kernels (built-in 64 MB)
  size_t ag_pull_round_bytes = (size_t)-1;  // all_gather pull mode (built-in 32 MB)
  size_t ag_nvls_max_bytes = 128u << 20;    // all_gather outputs from this size use the pull mode even when the switch is enabled
  size_t symm_min_bytes = (size_t)-1;  // -1: built-in (512 KB; 16 MB for two ranks)
};

// One-shot all_reduce moves (W-1)*S bytes into every GPU, two-shot 2*S*(W-1)/W: with two ranks
// they move the same, with eight the measured crossover is 1 MB (see CudaComm.cpp).
size_t default_oneshot_max(int world);

struct AlgoChoice {
  Algo algo;
  int nblocks;
  int nthreads;
};

class CudaComm {
 public:
  // Real communicator: collective over all `world` processes (blocks on the store).
  CudaComm(int rank, int world, int device, const CommConfig& cfg, KvStore kv, const std::string& prefix);
  // Emulated communicator on one device.
  CudaComm(int world, int device, const CommConfig& cfg);
  ~CudaComm();
  CudaComm(const CudaComm&) = delete;
  CudaComm& operator=(const CudaComm&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }
  int nctx() const { return emulated_ ? world_ : 1; }
  int device() const { return device_; }
  bool emulated() const { return emulated_; }
  // True when the arenas are mapped through a multicast object (real communicators only).
  bool nvls_available() const { return symm_ && symm_->multicast_base() != nullptr; }
  const CommConfig& config() const { return cfg_; }
  CommConfig& mutable_config() { return cfg_; }
  const RankCtx& ctx(int i = 0) const { return host_ctx_[i]; }

  // Error record written by kernels whose bounded waits expired: {code, rank, peer, phase}.
  // Returns code (0 = healthy).
  int poll_status(int* rank = nullptr, int* peer = nullptr, int* phase = nullptr) const;
  void clear_status();
  // Own arena staging pointer (for zero-copy consumers) and its size.
  char* local_data(int i = 0) const { return host_ctx_[i].data[host_ctx_[i].rank]; }

  // ---- collectives. `args` has nctx() entries (one per emulated rank, or exactly one). ----
  // The wrappers fill chunk_vecs / rounds / mode, choose algorithm and grid, and launch on `stream`.
  cudaError_t allreduce(int dtype, std::vector<CollArgs> args, cudaStream_t stream, AlgoChoice* chosen = nullptr);
  cudaError_t reduce(int dtype, std::vector<CollArgs> args, cudaStream_t stream);  // args.root set
  cudaError_t reduce_scatter(int in_dtype, int out_dtype, std::vector<CollArgs> args, cudaStream_t stream);
  cudaError_t all_gather(std::vector<CollArgs> args, cudaStream_t stream);
  cudaError_t all_to_all(std::vector<CollArgs> args, bool uneven, cudaStream_t stream);
  cudaError_t rooted(std::vector<CollArgs> args, cudaStream_t stream);  // mode + root + count set
  cudaError_t barrier(cudaStream_t stream);
  // Failure-detection probe: plays ONLY rank `i` of the barrier, so its wait for the other
  // ranks' flags (which nothing sets) runs into the bounded-wait budget and reports a timeout.
  cudaError_t barrier_single_rank(int i, cudaStream_t stream);
  cudaError_t allreduce_residual_rmsnorm(int dtype, std::vector<FusedNormArgs> args, cudaStream_t stream);

  // A list of small tensors in ONE launch (see collectives_multi.h). `args` has nctx() entries with the same
  // n / mode / counts. Returns cudaErrorInvalidValue when the list does not fit the staging arena (or has more
  // than kMaxMulti tensors): the caller then issues the tensors one by one. multi_fits tells in advance.
  bool multi_fits(int dtype, const MultiArgs& a) const;
  cudaError_t multi(int dtype, std::vector<MultiArgs> args, cudaStream_t stream);

  // Decode step: row-parallel projection + all_reduce + residual + RMSNorm in one launch, and
  // arg-max + all-gather of the winners (see decode_fused.h). fits_gemm_ar_norm tells whether the
  // fused kernel takes the shape (else the caller runs GEMM and allreduce_residual_rmsnorm).
  bool fits_gemm_ar_norm(int rows, int hidden, int K) const;
  cudaError_t gemm_ar_norm(const std::vector<GemmArNormArgs>& args, cudaStream_t stream);
  cudaError_t sample_allgather(const std::vector<SampleArgs>& args, cudaStream_t stream);

  // ---- symmetric heap ----------------------------------------------------------------------
  // Allocation is COLLECTIVE IN ORDER: every rank must allocate (and release) the same sizes in the
  // same order, so that a tensor sits at the same heap offset on every rank; kernels then address
  // a peer's copy as that peer's heap base + the local offset, with no per-tensor handle exchange.
  // The first call creates the heap (collective over the communicator, blocks on the store).
  // Returns nullptr when the heap is exhausted.
  void* symm_alloc(size_t bytes);
  void symm_free(void* p);
  // Offset of [p, p + bytes) inside this rank's heap, or false if it is not (wholly) symmetric memory.
  bool symm_offset(const void* p, size_t bytes, size_t* off, int ctx_index = 0) const;
  bool heap_multicast() const { return heap_ && heap_->multicast_base() != nullptr; }
  // Base of rank context i's heap (emulation: one per played rank; real: this rank's own at i == 0).
  void* heap_base(int ctx_index = 0) const { return heap_bases_.empty() ? nullptr : heap_bases_[emulated_ ? ctx_index : rank_]; }
  size_t heap_in_use() const;
  // Zero-copy collectives on symmetric tensors (no staging through the arena). `in_off` / `out_off`
  // are heap offsets (symm_offset); buffers that are plain local memory are passed as pointers.
  // all_reduce: in and out symmetric (may be the same); SUM through the switch when the heap is
  // bound to a multicast object and `use_nvls`, else peer loads/stores. count * elem size % 16 == 0.
  cudaError_t allreduce_symm(int dtype, size_t in_off, size_t out_off, size_t count, int op, float scale, int has_scale,
                             bool use_nvls, cudaStream_t stream);
  // reduce_scatter: in symmetric [world * count], out[r] local [count] (out dtype may be fp32 for bf16/f16 input).
  cudaError_t reduce_scatter_symm(int in_dtype, int out_dtype, size_t in_off, std::vector<void*> outs, size_t count, int op,
                                  float scale, int has_scale, bool use_nvls, cudaStream_t stream);
  // all_gather: in[r] local [bytes], out symmetric [world * bytes].
  cudaError_t all_gather_symm(std::vector<const void*> ins, size_t out_off, size_t bytes, bool use_nvls, cudaStream_t stream);

  // Asks every kernel of this communicator that is (or will be) waiting for a peer to give up:
  // sets the host-mapped abort word that all bounded waits sample. The waits return within about a
  // millisecond with status kStatusAborted; the communicator stays failed until clear_abort().
  void abort();
  void clear_abort();
  bool aborted() const;

  // Fused tensor-parallel GEMMs (one entry per rank context, like the collectives).
  cudaError_t gemm_rs(const std::vector<GemmRsArgs>& args, cudaStream_t stream);
  cudaError_t ag_gemm(const std::vector<AgGemmArgs>& args, cudaStream_t stream);

  // Expert-parallel MoE token exchange. `cap` rows per (source, destination) pair is derived
  // from the arena size; moe_capacity() reports it.
  int moe_capacity(int hidden) const;
  cudaError_t moe_dispatch(std::vector<MoeArgs> args, cudaStream_t stream);
  cudaError_t moe_combine(std::vector<MoeArgs> args, cudaStream_t stream);

  // Capacity (bytes per rank) of the one-shot fused norm path.
  size_t fused_norm_capacity() const { return cfg_.half_bytes / world_; }

  uint64_t launches() const { return launches_; }
  // Whether the last reduce_scatter / all_gather went through the multicast object.
  void apply_builtin_thresholds();   // resolves the -1 knobs from the world size (measured tables)
  bool last_used_nvls() const { return last_algo_ == Algo::kNvls; }

 private:
  void init_tables();
  void enter_stream(cudaStream_t s);
  template <typename ArgsT>
  const ArgsT* upload(const std::vector<ArgsT>& args, cudaStream_t stream);
  LaunchCfg launch_cfg(int nblocks, int nthreads, cudaStream_t stream) const;
  int blocks_for(size_t vecs, int cap) const;

  int rank_ = 0, world_ = 1, device_ = 0;
  bool emulated_ = false;
  CommConfig cfg_;
  KvStore kv_;
  std::string prefix_;
  size_t arena_bytes_ = 0;
  std::unique_ptr<SymmMem> symm_;     // real communicators: owns the arena and the peer mappings
  std::vector<void*> local_arenas_;   // emulated communicators: one cudaMalloc per played rank
  std::vector<void*> peer_arenas_;    // real: mapped peer bases (own at [rank])
  std::vector<RankCtx> host_ctx_;     // nctx entries
  RankCtx* dev_ctx_table_ = nullptr;  // emulation only
  void* dev_args_table_ = nullptr;    // emulation only
  int* status_host_ = nullptr;        // pinned + mapped
  int* status_dev_ = nullptr;
  uint64_t launches_ = 0;
  void ensure_heap();
  std::unique_ptr<SymmMem> heap_;          // real communicators
  std::vector<void*> emu_heaps_;           // emulated communicators: one region per played rank
  std::vector<void*> heap_bases_;          // per rank (own at [rank] / all local in emulation)
  mutable std::mutex heap_mu_;
  std::vector<std::pair<size_t, size_t>> heap_free_;   // sorted (offset, size) holes
  std::vector<std::pair<size_t, size_t>> heap_used_;   // (offset, size) of live blocks
  std::mutex order_mu_;
  cudaEvent_t order_ev_ = nullptr;
  cudaStream_t last_stream_ = nullptr;
  bool has_last_stream_ = false;
  Algo last_algo_ = Algo::kAuto;
};

}  // namespace ccl
