#include "cuda/CudaComm.h"
#include "cuda/Tuner.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace ccl {

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("ccl: ") + what + " failed: " + cudaGetErrorString(e));
  }
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

// Built-in algorithm thresholds, from bench/tune.py on B200 / NVSwitch (device-timed, max over ranks;
// a CCL_TUNE_FILE measured on the machine at hand overrides them):
//   2 ranks: one-shot 9-10 us up to 512 KB, 25 us at 4 MB, 188 us at 64 MB against two-shot 16-20 / 40 / 185 us:
//            one-shot whenever the tensor fits its staging slot;
//   8 ranks: one-shot 12.5 us at 32 KB, 18.7 us at 512 KB, 24.5 us at 1 MB, 46.7 us at 2 MB; two-shot 31-38 us up
//            to 1 MB, 40 us at 2 MB, 50 us at 8 MB, 157 us at 32 MB; through the switch (staged, CCL_NVLS=1) 27 us
//            at 1 MB, 28 us at 2 MB, 49 us at 8 MB, 114 us at 32 MB: one-shot up to 1 MB, then the switch (from
//            2 MB) or two-shot.
size_t default_oneshot_max(int world) {
  if (world <= 2) return (size_t)1 << 40;
  return 1u << 20;
}

// all_gather: push (every rank writes its piece into all peers' arenas) against pull. 2 ranks: push wins up to
// 2 MB per piece (8 KB 7.8 vs 8.7 us, 1 MB 14.1 vs 16.6); 8 ranks: push wins or ties up to 2 MB per piece
// (8 KB 14.0 vs 21.5 us, 256 KB 17.5 vs 25.9, 2 MB 42.0 vs 41.5).
static size_t default_ag_push_max(int /*world*/) { return 2u << 20; }

namespace {

size_t arena_size(size_t half) { return 2 * half + kFlagBytes + kStateBytes + kLLBytes; }

void fill_ctx(RankCtx& c, int rank, int world, const std::vector<void*>& bases, size_t half,
              uint64_t spin_ms, int* status, void* multicast_base) {
  std::memset(&c, 0, sizeof(c));
  for (int p = 0; p < world; ++p) {
    c.data[p] = static_cast<char*>(bases[p]);
    c.flags[p] = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[p]) + 2 * half);
    c.ll[p] = static_cast<char*>(bases[p]) + 2 * half + kFlagBytes + kStateBytes;
  }
  c.state = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[rank]) + 2 * half + kFlagBytes);
  c.status = status;
  c.abort_flag = status ? status + 8 : nullptr;  // word 8 of the host-mapped status block
  c.half_bytes = half;
  c.spin_ns = spin_ms * 1000000ull;
  c.mc_data = static_cast<char*>(multicast_base);
  c.rank = rank;
  c.world = world;
}

}  // namespace

void CudaComm::apply_builtin_thresholds() { resolve_builtin_thresholds(world_, &cfg_); }

CudaComm::CudaComm(int rank, int world, int device, const CommConfig& cfg, KvStore kv,
                   const std::string& prefix)
    : rank_(rank), world_(world), device_(device), emulated_(false), cfg_(cfg), kv_(std::move(kv)),
      prefix_(prefix) {
  if (world < 1 || world > kMaxRanks) throw std::runtime_error("ccl: CUDA communicators support 1..8 ranks");
  DeviceGuard g(device_);
  cfg_.half_bytes = round_up(cfg_.half_bytes, 1 << 20);
  if (cfg_.oneshot_max_bytes == 0) cfg_.oneshot_max_bytes = default_oneshot_max(world_);
  if (cfg_.ag_push_max_bytes == 0) cfg_.ag_push_max_bytes = default_ag_push_max(world_);
  apply_builtin_thresholds();
  arena_bytes_ = arena_size(cfg_.half_bytes);
  check(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped | cudaHostAllocPortable),
        "cudaHostAlloc(status)");
  std::memset(status_host_, 0, 64);
  check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_), status_host_, 0), "cudaHostGetDevicePointer");
  // allocates and zeroes this rank's arena, maps every peer's, and returns once all ranks have
  symm_ = std::make_unique<SymmMem>(cfg_.symm, rank_, world_, device_, arena_bytes_, kv_, prefix_,
                                    cfg_.nvls && cfg_.symm == SymmKind::kVmm);
  peer_arenas_ = symm_->bases();
  check(cudaEventCreateWithFlags(&order_ev_, cudaEventDisableTiming), "cudaEventCreate(order)");
  init_tables();
}

CudaComm::CudaComm(int world, int device, const CommConfig& cfg)
    : rank_(0), world_(world), device_(device), emulated_(true), cfg_(cfg) {
  if (world < 1 || world > kMaxRanks) throw std::runtime_error("ccl: CUDA communicators support 1..8 ranks");
  DeviceGuard g(device_);
  cfg_.half_bytes = round_up(cfg_.half_bytes, 1 << 20);
  if (cfg_.oneshot_max_bytes == 0) cfg_.oneshot_max_bytes = default_oneshot_max(world_);
  if (cfg_.ag_push_max_bytes == 0) cfg_.ag_push_max_bytes = default_ag_push_max(world_);
  apply_builtin_thresholds();
  arena_bytes_ = arena_size(cfg_.half_bytes);
  for (int r = 0; r < world_; ++r) {
    void* base = nullptr;
    check(cudaMalloc(&base, arena_bytes_), "cudaMalloc(arena)");
    check(cudaMemset(base, 0, arena_bytes_), "cudaMemset(arena)");
    local_arenas_.push_back(base);
  }
  peer_arenas_ = local_arenas_;
  check(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped | cudaHostAllocPortable),
        "cudaHostAlloc(status)");
  std::memset(status_host_, 0, 64);
  check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_), status_host_, 0), "cudaHostGetDevicePointer");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  check(cudaEventCreateWithFlags(&order_ev_, cudaEventDisableTiming), "cudaEventCreate(order)");
  init_tables();
}

void CudaComm::init_tables() {
  const int n = nctx();
  host_ctx_.resize(n);
  for (int i = 0; i < n; ++i) {
    const int r = emulated_ ? i : rank_;
    fill_ctx(host_ctx_[i], r, world_, peer_arenas_, cfg_.half_bytes, cfg_.spin_timeout_ms, status_dev_,
             symm_ ? symm_->multicast_base() : nullptr);
  }
  if (emulated_) {
    check(cudaMalloc(reinterpret_cast<void**>(&dev_ctx_table_), sizeof(RankCtx) * n), "cudaMalloc(ctx table)");
    check(cudaMemcpy(dev_ctx_table_, host_ctx_.data(), sizeof(RankCtx) * n, cudaMemcpyHostToDevice), "cudaMemcpy(ctx table)");
    check(cudaMalloc(&dev_args_table_, 64 << 10), "cudaMalloc(args table)");
  }
}

CudaComm::~CudaComm() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (!emulated_ && world_ > 1) {
    // peers may still be reading this arena: wait for them (best effort) before unmapping
    try {
      barrier_kv(kv_, prefix_ + "/bye", world_, 5000);
    } catch (...) {
    }
  }
  heap_.reset();
  for (void* h : emu_heaps_) cudaFree(h);
  symm_.reset();
  for (void* a : local_arenas_) cudaFree(a);
  if (dev_ctx_table_) cudaFree(dev_ctx_table_);
  if (dev_args_table_) cudaFree(dev_args_table_);
  if (status_host_) cudaFreeHost(status_host_);
  if (order_ev_) cudaEventDestroy(order_ev_);
}

int CudaComm::poll_status(int* rank, int* peer, int* phase) const {
  volatile int* s = status_host_;
  const int code = s[0];
  if (code) {
    if (rank) *rank = s[1];
    if (peer) *peer = s[2];
    if (phase) *phase = s[3];
  }
  return code;
}
void CudaComm::clear_status() {
  volatile int* s = status_host_;
  s[1] = s[2] = s[3] = 0;
  s[0] = 0;
}

// One launch in flight per communicator: the kernels of a communicator share its epoch, ticket and
// staging halves, so two of them must never run concurrently. Launches on one stream are ordered
// by the stream; when the caller moves to another stream (c10d ops run on the backend's
// communication stream, the fused ops on the caller's current stream) the new stream is made to
// wait for everything enqueued on the previous one. Costs nothing while the stream stays the
// same. Streams that are being captured are left alone: inside a CUDA graph the capture's own
// dependencies order the launches.
void CudaComm::enter_stream(cudaStream_t s) {
  std::lock_guard<std::mutex> g(order_mu_);
  if (has_last_stream_ && last_stream_ != s) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone, cl = cudaStreamCaptureStatusNone;
    const bool q = cudaStreamIsCapturing(s, &cs) == cudaSuccess && cudaStreamIsCapturing(last_stream_, &cl) == cudaSuccess;
    if (q && cs == cudaStreamCaptureStatusNone && cl == cudaStreamCaptureStatusNone &&
        cudaEventRecord(order_ev_, last_stream_) == cudaSuccess) {
      cudaStreamWaitEvent(s, order_ev_, 0);
    } else {
      (void)cudaGetLastError();
    }
  }
  last_stream_ = s;
  has_last_stream_ = true;
}

template <typename ArgsT>
const ArgsT* CudaComm::upload(const std::vector<ArgsT>& args, cudaStream_t stream) {
  if (!emulated_) return args.data();
  if (sizeof(ArgsT) * args.size() > (64u << 10)) throw std::runtime_error("ccl: args table too large");
  // emulation is a test vehicle: a synchronous copy keeps lifetimes trivial
  check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  check(cudaMemcpy(dev_args_table_, args.data(), sizeof(ArgsT) * args.size(), cudaMemcpyHostToDevice), "cudaMemcpy(args)");
  return static_cast<const ArgsT*>(dev_args_table_);
}

LaunchCfg CudaComm::launch_cfg(int nblocks, int nthreads, cudaStream_t stream) const {
  LaunchCfg c;
  c.nblocks = std::max(1, std::min(nblocks, kMaxBlocks));
  c.nthreads = nthreads;
  c.nctx = nctx();
  c.cooperative = emulated_;
  c.stream = stream;
  if (emulated_) c.nblocks = std::min(c.nblocks, std::max(1, 128 / world_));  // keep every CTA co-resident
  return c;
}

// Small messages get small CTAs (cheaper to launch and to synchronise).
static int threads_for(size_t vecs, int nblocks, int max_threads) {
  size_t per = (vecs + (size_t)nblocks - 1) / (size_t)std::max(1, nblocks);
  size_t t = (per + 31) / 32 * 32;
  if (t < 128) t = 128;
  if (t > (size_t)max_threads) t = max_threads;
  return (int)t;
}

int CudaComm::blocks_for(size_t vecs, int cap) const {
  // one 16-byte vector per thread and peer up to the CTA cap, more beyond it
  const size_t per_block = (size_t)cfg_.threads;
  size_t b = (vecs + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > (size_t)cap) b = cap;
  return (int)b;
}

// Staging slots are packed back to back when the whole message fits in one round: a slot stride
// derived from the arena capacity would spread a small message over pages tens of MB apart in
// every peer's arena, and the address translations for those scattered peer pages cost far
// more than the transfer (measured: ~80 us floor for a 1 MB all_reduce at 8 GPUs).
static size_t compact_stride(size_t capacity_stride, size_t needed_vecs) {
  size_t want = (needed_vecs + 7) / 8 * 8;
  if (want < 8) want = 8;
  return want < capacity_stride ? want : capacity_stride;
}

// Optional cap on a staging round (CCL_ROUND_MB): `slots` slots of `stride` vectors make one round.
// Smaller rounds keep what one phase stages in L2 for the next phase and let the CTAs of a kernel
// drift into different phases (local copies overlap NVLink transfers); every extra round costs
// its flag exchanges (about 10 us each at 2 GPUs).
static size_t cap_stride(size_t stride, size_t slots, size_t round_bytes) {
  if (round_bytes == 0) return stride;
  size_t cap = round_bytes / 16 / std::max<size_t>(slots, 1) / 8 * 8;
  if (cap < 8) cap = 8;
  return std::min(stride, cap);
}

#define CCL_CHECK_ARGS(v)                                                             \
  if ((int)(v).size() != nctx()) return cudaErrorInvalidValue;

cudaError_t CudaComm::allreduce(int dtype, std::vector<CollArgs> args, cudaStream_t stream, AlgoChoice* chosen) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const size_t esz = dtype_size(dtype);
  const size_t count = args[0].count;
  const size_t bytes = count * esz;
  const size_t nvec = (bytes + 15) / 16;
  Algo algo = cfg_.algo;
  // symmetric tensors (allocated from the communicator's heap) skip the staging arena altogether
  if (world_ > 1 && !heap_bases_.empty() && cfg_.ablate == kAblateNone && bytes >= cfg_.symm_min_bytes && bytes % 16 == 0 &&
      (algo == Algo::kAuto || algo == Algo::kNvls)) {
    size_t in_off = 0, out_off = 0;
    bool symm = true;
    for (int i = 0; i < nctx() && symm; ++i) {
      size_t io = 0, oo = 0;
      symm = symm_offset(args[i].in, bytes, &io, i) && symm_offset(args[i].out, bytes, &oo, i) && (i == 0 || (io == in_off && oo == out_off));
      in_off = io;
      out_off = oo;
    }
    if (symm && in_off % 16 == 0 && out_off % 16 == 0) {
      cudaError_t es = allreduce_symm(dtype, in_off, out_off, count, args[0].op, args[0].scale, args[0].has_scale, true, stream);
      if (chosen) *chosen = AlgoChoice{last_algo_, 0, 0};
      return es;
    }
  }
  const size_t slot = round_up(nvec * 16, 128);
  const bool fits_oneshot = slot * world_ <= cfg_.half_bytes;
  // the switch reduces SUMs of bf16 / f16 / f32 only; the emulation plays it in software when forced
  const bool nvls_ok = (emulated_ || nvls_available()) && args[0].op == kSum && (dtype == kBF16 || dtype == kF16 || dtype == kF32) &&
                       world_ > (emulated_ ? 1 : 0);
  if (algo == Algo::kNvls && !nvls_ok) algo = Algo::kAuto;
  if (algo == Algo::kAuto && !emulated_ && cfg_.nvls && nvls_ok && bytes >= cfg_.nvls_min_bytes) algo = Algo::kNvls;
  if (algo == Algo::kAuto)
    algo = (bytes <= cfg_.oneshot_max_bytes && fits_oneshot) ? Algo::kOneShot : Algo::kTwoShot;
  if (algo == Algo::kOneShot && !fits_oneshot) algo = Algo::kTwoShot;
  for (auto& a : args) {
    a.ablate = cfg_.ablate;
    a.root = -1;
  }
  cudaError_t e;
  LaunchCfg lc;
  if (algo == Algo::kOneShot) {
    lc = launch_cfg(blocks_for(nvec, cfg_.max_blocks), threads_for(nvec, blocks_for(nvec, cfg_.max_blocks), cfg_.threads), stream);
    e = launch_allreduce_oneshot(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  } else if (algo == Algo::kNvls) {
    size_t stride = cap_stride(cfg_.half_bytes / (16 * (size_t)world_), world_, cfg_.nvls_round_bytes);
    stride = compact_stride(stride / 8 * 8, (nvec + world_ - 1) / world_);
    for (auto& a : args) a.chunk_vecs = stride;
    const size_t per_shard = (nvec + world_ - 1) / world_;
    lc = launch_cfg(blocks_for(per_shard, cfg_.max_blocks), threads_for(per_shard, blocks_for(per_shard, cfg_.max_blocks), cfg_.threads), stream);
    e = launch_allreduce_nvls(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  } else {
    size_t stride = cap_stride(cfg_.half_bytes / (16 * (size_t)(world_ + 1)), world_, cfg_.round_bytes);
    stride = compact_stride(stride / 8 * 8, (nvec + world_ - 1) / world_);
    for (auto& a : args) a.chunk_vecs = stride;
    lc = launch_cfg(blocks_for((nvec + world_ - 1) / world_, cfg_.max_blocks), threads_for((nvec + world_ - 1) / world_, blocks_for((nvec + world_ - 1) / world_, cfg_.max_blocks), cfg_.threads), stream);
    e = launch_allreduce_twoshot(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  }
  if (chosen) *chosen = AlgoChoice{algo, lc.nblocks, lc.nthreads};
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::reduce(int dtype, std::vector<CollArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const size_t nvec = (args[0].count * dtype_size(dtype) + 15) / 16;
  size_t stride = cfg_.half_bytes / (16 * (size_t)(world_ + 1));
  stride = compact_stride(stride / 8 * 8, (nvec + world_ - 1) / world_);
  for (auto& a : args) {
    a.chunk_vecs = stride;
    a.ablate = cfg_.ablate;
  }
  LaunchCfg lc = launch_cfg(blocks_for((nvec + world_ - 1) / world_, cfg_.max_blocks), threads_for((nvec + world_ - 1) / world_, blocks_for((nvec + world_ - 1) / world_, cfg_.max_blocks), cfg_.threads), stream);
  cudaError_t e = launch_allreduce_twoshot(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::reduce_scatter(int in_dtype, int out_dtype, std::vector<CollArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const size_t esz = dtype_size(in_dtype);
  // flat symmetric input (equal pieces, back to back, inside the heap): reduce straight out of the peers' buffers
  if (world_ > 1 && !heap_bases_.empty() && cfg_.ablate == kAblateNone && (cfg_.algo == Algo::kAuto || cfg_.algo == Algo::kNvls)) {
    const size_t cnt = args[0].in_cnt[0];
    const size_t pb = cnt * esz;
    bool symm = pb >= cfg_.symm_min_bytes / world_ && pb % 16 == 0;
    size_t in_off = 0;
    std::vector<void*> outs;
    for (int i = 0; i < nctx() && symm; ++i) {
      const char* base = static_cast<const char*>(args[i].in_piece[0]);
      for (int p = 0; p < world_ && symm; ++p) symm = args[i].in_cnt[p] == cnt && args[i].in_piece[p] == base + (size_t)p * pb;
      size_t io = 0;
      symm = symm && symm_offset(base, pb * world_, &io, i) && (i == 0 || io == in_off) && io % 16 == 0 &&
             (reinterpret_cast<uintptr_t>(args[i].out) & 15) == 0;
      in_off = io;
      outs.push_back(args[i].out);
    }
    if (symm) return reduce_scatter_symm(in_dtype, out_dtype, in_off, outs, cnt, args[0].op, args[0].scale, args[0].has_scale, true, stream);
  }
  const size_t per_vec = 16 / esz;
  size_t maxv = 0;
  for (auto& a : args)
    for (int p = 0; p < world_; ++p) maxv = std::max(maxv, ((size_t)a.in_cnt[p] + per_vec - 1) / per_vec);
  // in-switch reduction: SUM of bf16 / f16 / f32 into the same dtype (the switch returns the sum rounded to the
  // input type, so the widened bf16 -> fp32 gradient path stays on the peer-load kernel, which keeps fp32)
  const bool nvls_ok = (emulated_ ? world_ > 1 : nvls_available()) && args[0].op == kSum && in_dtype == out_dtype &&
                       (in_dtype == kBF16 || in_dtype == kF16 || in_dtype == kF32);
  const bool use_nvls = nvls_ok && (cfg_.algo == Algo::kNvls || (!emulated_ && cfg_.nvls && cfg_.algo == Algo::kAuto &&
                                                                  maxv * 16 * world_ >= cfg_.nvls_min_bytes));
  size_t stride = cap_stride(cfg_.half_bytes / (16 * (size_t)world_), world_, use_nvls ? cfg_.nvls_round_bytes : cfg_.round_bytes);
  stride = compact_stride(stride / 8 * 8, maxv);
  const int rounds = (int)((maxv + stride - 1) / stride);
  for (auto& a : args) {
    a.chunk_vecs = stride;
    a.rounds = rounds;
    a.ablate = cfg_.ablate;
  }
  LaunchCfg lc = launch_cfg(blocks_for(std::min(maxv, stride), cfg_.max_blocks), threads_for(std::min(maxv, stride), blocks_for(std::min(maxv, stride), cfg_.max_blocks), cfg_.threads), stream);
  last_algo_ = use_nvls ? Algo::kNvls : Algo::kTwoShot;
  if (use_nvls) {
    cudaError_t en = launch_reduce_scatter_nvls(in_dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
    if (en == cudaSuccess) ++launches_;
    return en;
  }
  cudaError_t e = launch_reduce_scatter(in_dtype, out_dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::all_gather(std::vector<CollArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  // flat symmetric output (equal pieces, back to back, inside the heap): write straight into the peers' buffers
  if (world_ > 1 && !heap_bases_.empty() && cfg_.ablate == kAblateNone && (cfg_.algo == Algo::kAuto || cfg_.algo == Algo::kNvls)) {
    const size_t pb = args[0].out_cnt[0];
    bool symm = pb >= cfg_.symm_min_bytes / world_ && pb % 16 == 0;
    size_t out_off = 0;
    std::vector<const void*> ins;
    for (int i = 0; i < nctx() && symm; ++i) {
      const char* base = static_cast<const char*>(args[i].out_piece[0]);
      for (int p = 0; p < world_ && symm; ++p) symm = args[i].out_cnt[p] == pb && args[i].out_piece[p] == base + (size_t)p * pb;
      size_t oo = 0;
      symm = symm && symm_offset(base, pb * world_, &oo, i) && (i == 0 || oo == out_off) && oo % 16 == 0 &&
             (reinterpret_cast<uintptr_t>(args[i].in) & 15) == 0;
      out_off = oo;
      ins.push_back(args[i].in);
    }
    if (symm) return all_gather_symm(ins, out_off, pb, true, stream);
  }
  size_t maxb = 0;
  for (auto& a : args)
    for (int p = 0; p < world_; ++p) maxb = std::max(maxb, (size_t)a.out_cnt[p]);
  const size_t maxv = (maxb + 15) / 16;
  const bool nvls_ok = emulated_ ? world_ > 1 : nvls_available();
  // The switch variant (one multimem.st per vector, then a local copy-out of everything) wins in the middle range; for
  // large outputs the pull mode, whose reads land straight in the user tensor, is faster (4 ranks, 512 MB: 671 vs 878 us).
  const bool use_nvls = nvls_ok && (cfg_.algo == Algo::kNvls || (!emulated_ && cfg_.nvls && cfg_.algo == Algo::kAuto &&
                                                                  maxb * world_ >= cfg_.nvls_min_bytes &&
                                                                  maxb * world_ < cfg_.ag_nvls_max_bytes));
  last_algo_ = use_nvls ? Algo::kNvls : Algo::kTwoShot;
  const int mode = (use_nvls || maxb <= cfg_.ag_push_max_bytes) ? 1 : 0;  // NVLS uses the push layout: one slot per source
  size_t stride = mode == 1 ? cfg_.half_bytes / (16 * (size_t)world_) : cfg_.half_bytes / 16;
  // Pull mode stages the own piece locally and lets the peers read it: rounds of at most 32 MB keep the staged
  // round in L2 for the readers and let the CTAs drift apart, so that one CTA's staging overlaps another's reads
  // (2 GPUs, 2 x 256 MB: 653 us with 256 MB rounds, 530 us with 64 MB, 553 us with 16 MB; NCCL 627 us).
  if (mode == 0) stride = cap_stride(stride, 1, cfg_.ag_pull_round_bytes);
  else stride = cap_stride(stride, world_, use_nvls ? cfg_.nvls_round_bytes : cfg_.round_bytes);
  stride = compact_stride(stride / 8 * 8, maxv);
  const int rounds = (int)((maxv + stride - 1) / stride);
  for (auto& a : args) {
    a.chunk_vecs = stride;
    a.rounds = rounds;
    a.mode = mode;
    a.ablate = cfg_.ablate;
  }
  LaunchCfg lc = launch_cfg(blocks_for(std::min(maxv, stride), cfg_.max_blocks), threads_for(std::min(maxv, stride), blocks_for(std::min(maxv, stride), cfg_.max_blocks), cfg_.threads), stream);
  cudaError_t e = use_nvls ? launch_all_gather_nvls(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc)
                           : launch_all_gather(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::all_to_all(std::vector<CollArgs> args, bool uneven, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  // the round cap pays for up to four ranks (512 MB: 680 -> 643 us at 2, 819 -> 798 at 4); at eight it does not (920 -> 948)
  size_t stride = cap_stride(cfg_.half_bytes / (16 * (size_t)world_), world_, (uneven || world_ > 4) ? 0 : cfg_.round_bytes);
  stride = stride / 8 * 8;
  size_t maxb = 0;
  for (auto& a : args)
    for (int p = 0; p < world_; ++p) maxb = std::max(maxb, std::max((size_t)a.in_cnt[p], (size_t)a.out_cnt[p]));
  const size_t maxv = (maxb + 15) / 16;
  // With uneven splits the number of rounds is agreed on the device (rounds = 0); the emulated
  // communicator sees every rank's sizes, the real one only its own.
  if (!uneven) stride = compact_stride(stride, maxv);  // uneven: sizes differ per rank, keep the common capacity stride
  const int rounds = uneven ? 0 : (int)((maxv + stride - 1) / stride);
  for (auto& a : args) {
    a.chunk_vecs = stride;
    a.rounds = rounds;
    a.ablate = cfg_.ablate;
  }
  LaunchCfg lc = launch_cfg(blocks_for(std::min(std::max(maxv, (size_t)1), stride), cfg_.max_blocks), threads_for(std::min(std::max(maxv, (size_t)1), stride), blocks_for(std::min(std::max(maxv, (size_t)1), stride), cfg_.max_blocks), cfg_.threads), stream);
  if (uneven) lc.nblocks = std::max(1, std::min(cfg_.max_blocks, emulated_ ? std::max(1, 128 / world_) : cfg_.max_blocks) / 2);
  cudaError_t e = launch_all_to_all(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::rooted(std::vector<CollArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  int mode = args[0].mode;
  if (mode == kBroadcast && world_ > 1 && cfg_.ablate == kAblateNone) {
    // Large broadcasts leave the root once and are replicated by the switch.
    const bool nvls_ok = emulated_ ? true : nvls_available();
    const bool use_nvls = nvls_ok && (cfg_.algo == Algo::kNvls || (!emulated_ && cfg_.nvls && cfg_.algo == Algo::kAuto &&
                                                                    (size_t)args[0].count >= cfg_.nvls_min_bytes));
    last_algo_ = use_nvls ? Algo::kNvls : Algo::kTwoShot;
    if (use_nvls) {
      mode = kBroadcastSwitch;
      for (auto& a : args) a.mode = kBroadcastSwitch;
    }
  }
  size_t stride = (mode == kGather) ? cfg_.half_bytes / (16 * (size_t)world_) : cfg_.half_bytes / 16;
  stride = stride / 8 * 8;
  const size_t maxv = ((size_t)args[0].count + 15) / 16;
  stride = compact_stride(stride, maxv);
  const int rounds = (int)((maxv + stride - 1) / stride);
  for (auto& a : args) {
    a.chunk_vecs = stride;
    a.rounds = rounds;
    a.ablate = cfg_.ablate;
  }
  LaunchCfg lc = launch_cfg(blocks_for(std::min(maxv, stride), cfg_.max_blocks), threads_for(std::min(maxv, stride), blocks_for(std::min(maxv, stride), cfg_.max_blocks), cfg_.threads), stream);
  cudaError_t e = launch_rooted(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

bool CudaComm::multi_fits(int dtype, const MultiArgs& a) const {
  return world_ > 1 && a.n >= 1 && a.n <= kMaxMulti && cfg_.ablate == kAblateNone &&
         multi_slot_bytes(dtype, a) * (size_t)world_ <= cfg_.half_bytes;
}

cudaError_t CudaComm::multi(int dtype, std::vector<MultiArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  if (!multi_fits(dtype, args[0])) return cudaErrorInvalidValue;
  const size_t slot = multi_slot_bytes(dtype, args[0]);
  for (auto& a : args) a.slot_bytes = slot;
  const size_t vecs = slot / 16;
  LaunchCfg lc = launch_cfg(blocks_for(vecs, std::min(cfg_.max_blocks, 64)), threads_for(vecs, blocks_for(vecs, std::min(cfg_.max_blocks, 64)), cfg_.threads), stream);
  cudaError_t e = launch_multi(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::barrier(cudaStream_t stream) {
  DeviceGuard g(device_);
  enter_stream(stream);
  std::vector<CollArgs> args(nctx());
  for (auto& a : args) a.ablate = kAblateNone;
  LaunchCfg lc = launch_cfg(1, 32, stream);
  cudaError_t e = launch_barrier(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::gemm_rs(const std::vector<GemmRsArgs>& args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  // every rank's GEMM only pushes and signals; the reduce kernels wait. Played one rank after
  // the other in emulation, which is safe because the pushes never wait.
  for (int i = 0; i < nctx(); ++i) {
    cudaError_t e = launch_gemm_rs(host_ctx_[i], args[i], stream);
    if (e != cudaSuccess) return e;
    ++launches_;
  }
  for (int i = 0; i < nctx(); ++i) {
    const size_t nvec = (size_t)(args[i].M / world_) * args[i].N * 2 / 16;
    cudaError_t e = launch_gemm_rs_reduce(host_ctx_[i], args[i], blocks_for(nvec, 64), stream);
    if (e != cudaSuccess) return e;
    ++launches_;
  }
  return cudaSuccess;
}

cudaError_t CudaComm::ag_gemm(const std::vector<AgGemmArgs>& args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const int ncomm = 8;
  if (!emulated_) {
    cudaError_t e = launch_ag_gemm(host_ctx_[0], args[0], 0, ncomm, stream);
    if (e == cudaSuccess) ++launches_;
    return e;
  }
  for (int mode = 1; mode <= 2; ++mode) {
    for (int i = 0; i < nctx(); ++i) {
      cudaError_t e = launch_ag_gemm(host_ctx_[i], args[i], mode, ncomm, stream);
      if (e != cudaSuccess) return e;
      ++launches_;
    }
  }
  return cudaSuccess;
}

int CudaComm::moe_capacity(int hidden) const {
  const size_t per_src = cfg_.half_bytes / world_;
  const size_t fixed = (size_t)kMaxBlocks * 4 + 256;
  if (per_src <= fixed) return 0;
  return (int)((per_src - fixed) / ((size_t)hidden * 2 + 8));
}

cudaError_t CudaComm::moe_dispatch(std::vector<MoeArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const int cap = moe_capacity(args[0].hidden);
  if (cap <= 0 || args[0].hidden % 8 != 0) return cudaErrorInvalidValue;
  for (auto& a : args) {
    a.cap = cap;
    a.slot_bytes = moe_dispatch_slot_bytes(cap, a.hidden);
    if (a.slot_bytes * world_ > cfg_.half_bytes) {
      a.cap = cap - 64;
      a.slot_bytes = moe_dispatch_slot_bytes(a.cap, a.hidden);
    }
  }
  LaunchCfg lc = launch_cfg(std::min(64, cfg_.max_blocks), 512, stream);
  cudaError_t e = launch_moe_dispatch(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::moe_combine(std::vector<MoeArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  if ((size_t)args[0].tokens * args[0].topk * args[0].hidden * 2 > cfg_.half_bytes) return cudaErrorInvalidValue;
  LaunchCfg lc = launch_cfg(std::min(64, cfg_.max_blocks), 512, stream);
  cudaError_t e = launch_moe_combine(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::barrier_single_rank(int i, cudaStream_t stream) {
  DeviceGuard g(device_);
  enter_stream(stream);
  if (i < 0 || i >= nctx()) return cudaErrorInvalidValue;
  CollArgs a;
  LaunchCfg lc;
  lc.nblocks = 1;
  lc.nthreads = 32;
  lc.nctx = 1;
  lc.stream = stream;
  return launch_barrier(&host_ctx_[i], &a, lc);
}

// ------------------------------------------------------------------------------------------
// symmetric heap
// ------------------------------------------------------------------------------------------
void CudaComm::ensure_heap() {
  if (!heap_bases_.empty()) return;
  DeviceGuard g(device_);
  const size_t bytes = round_up(cfg_.heap_bytes, 2u << 20);
  if (emulated_) {
    for (int r = 0; r < world_; ++r) {
      void* base = nullptr;
      check(cudaMalloc(&base, bytes), "cudaMalloc(symmetric heap)");
      emu_heaps_.push_back(base);
    }
    heap_bases_ = emu_heaps_;
  } else {
    // collective over the communicator: every rank reaches its first symmetric allocation together
    const bool mc = cfg_.nvls && world_ > 1;
    heap_ = std::make_unique<SymmMem>(mc ? SymmKind::kVmm : cfg_.symm, rank_, world_, device_, bytes, kv_, prefix_ + "/heap", mc);
    heap_bases_ = heap_->bases();
  }
  cfg_.heap_bytes = bytes;
  heap_free_.assign(1, {0, bytes});
  for (int i = 0; i < nctx(); ++i) {
    for (int p = 0; p < world_; ++p) host_ctx_[i].heap[p] = static_cast<char*>(heap_bases_[p]);
    host_ctx_[i].mc_heap = heap_ ? static_cast<char*>(heap_->multicast_base()) : nullptr;
  }
  if (emulated_)
    check(cudaMemcpy(dev_ctx_table_, host_ctx_.data(), sizeof(RankCtx) * nctx(), cudaMemcpyHostToDevice), "cudaMemcpy(ctx table)");
}

void* CudaComm::symm_alloc(size_t bytes) {
  std::lock_guard<std::mutex> g(heap_mu_);
  ensure_heap();
  const size_t need = round_up(std::max<size_t>(bytes, 1), 1024);
  // first fit in address order: the same sequence of calls gives the same offsets on every rank
  for (size_t i = 0; i < heap_free_.size(); ++i) {
    if (heap_free_[i].second < need) continue;
    const size_t off = heap_free_[i].first;
    if (heap_free_[i].second == need) heap_free_.erase(heap_free_.begin() + i);
    else heap_free_[i] = {off + need, heap_free_[i].second - need};
    heap_used_.push_back({off, need});
    return static_cast<char*>(heap_bases_[emulated_ ? 0 : rank_]) + off;
  }
  return nullptr;
}

void CudaComm::symm_free(void* p) {
  std::lock_guard<std::mutex> g(heap_mu_);
  if (heap_bases_.empty() || !p) return;
  const size_t off = static_cast<char*>(p) - static_cast<char*>(heap_bases_[emulated_ ? 0 : rank_]);
  for (size_t i = 0; i < heap_used_.size(); ++i) {
    if (heap_used_[i].first != off) continue;
    std::pair<size_t, size_t> blk = heap_used_[i];
    heap_used_.erase(heap_used_.begin() + i);
    // insert in address order and merge with the neighbours
    size_t k = 0;
    while (k < heap_free_.size() && heap_free_[k].first < blk.first) ++k;
    heap_free_.insert(heap_free_.begin() + k, blk);
    if (k + 1 < heap_free_.size() && heap_free_[k].first + heap_free_[k].second == heap_free_[k + 1].first) {
      heap_free_[k].second += heap_free_[k + 1].second;
      heap_free_.erase(heap_free_.begin() + k + 1);
    }
    if (k > 0 && heap_free_[k - 1].first + heap_free_[k - 1].second == heap_free_[k].first) {
      heap_free_[k - 1].second += heap_free_[k].second;
      heap_free_.erase(heap_free_.begin() + k);
    }
    return;
  }
}

size_t CudaComm::heap_in_use() const {
  std::lock_guard<std::mutex> g(heap_mu_);
  size_t n = 0;
  for (auto& b : heap_used_) n += b.second;
  return n;
}

bool CudaComm::symm_offset(const void* p, size_t bytes, size_t* off, int ctx_index) const {
  if (heap_bases_.empty() || !p) return false;
  const char* base = static_cast<const char*>(heap_bases_[emulated_ ? ctx_index : rank_]);
  const char* c = static_cast<const char*>(p);
  if (c < base || c + bytes > base + cfg_.heap_bytes) return false;
  if (off) *off = (size_t)(c - base);
  return true;
}

static bool switch_dtype(int dt) { return dt == kBF16 || dt == kF16 || dt == kF32; }

cudaError_t CudaComm::allreduce_symm(int dtype, size_t in_off, size_t out_off, size_t count, int op, float scale, int has_scale,
                                     bool use_nvls, cudaStream_t stream) {
  DeviceGuard g(device_);
  enter_stream(stream);
  const size_t bytes = count * dtype_size(dtype);
  if (bytes % 16 || in_off % 16 || out_off % 16 || heap_bases_.empty()) return cudaErrorInvalidValue;
  std::vector<SymmArgs> args(nctx());
  for (auto& a : args) {
    a.in_off = in_off;
    a.out_off = out_off;
    a.count = count;
    a.op = op;
    a.scale = scale;
    a.has_scale = has_scale;
    a.use_mc = (use_nvls && op == kSum && switch_dtype(dtype) && (emulated_ || heap_multicast())) ? 1 : 0;
  }
  const size_t share = ceil_div(bytes / 16, (size_t)world_);
  LaunchCfg lc = launch_cfg(blocks_for(share, cfg_.max_blocks), threads_for(share, blocks_for(share, cfg_.max_blocks), cfg_.threads), stream);
  last_algo_ = args[0].use_mc ? Algo::kNvls : Algo::kTwoShot;
  cudaError_t e = launch_allreduce_symm(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::reduce_scatter_symm(int in_dtype, int out_dtype, size_t in_off, std::vector<void*> outs, size_t count, int op,
                                          float scale, int has_scale, bool use_nvls, cudaStream_t stream) {
  CCL_CHECK_ARGS(outs)
  DeviceGuard g(device_);
  enter_stream(stream);
  const size_t bytes = count * dtype_size(in_dtype);
  if (bytes % 16 || in_off % 16 || heap_bases_.empty()) return cudaErrorInvalidValue;
  std::vector<SymmArgs> args(nctx());
  for (int i = 0; i < nctx(); ++i) {
    SymmArgs& a = args[i];
    a.in_off = in_off;
    a.out = outs[i];
    a.count = count;
    a.op = op;
    a.scale = scale;
    a.has_scale = has_scale;
    a.use_mc = (use_nvls && op == kSum && switch_dtype(in_dtype) && (emulated_ || heap_multicast())) ? 1 : 0;
  }
  const size_t pv = bytes / 16;
  LaunchCfg lc = launch_cfg(blocks_for(pv, cfg_.max_blocks), threads_for(pv, blocks_for(pv, cfg_.max_blocks), cfg_.threads), stream);
  last_algo_ = args[0].use_mc ? Algo::kNvls : Algo::kTwoShot;
  cudaError_t e = launch_reduce_scatter_symm(in_dtype, out_dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::all_gather_symm(std::vector<const void*> ins, size_t out_off, size_t bytes, bool use_nvls, cudaStream_t stream) {
  CCL_CHECK_ARGS(ins)
  DeviceGuard g(device_);
  enter_stream(stream);
  if (bytes % 16 || out_off % 16 || heap_bases_.empty()) return cudaErrorInvalidValue;
  std::vector<SymmArgs> args(nctx());
  for (int i = 0; i < nctx(); ++i) {
    if (reinterpret_cast<uintptr_t>(ins[i]) & 15) return cudaErrorInvalidValue;
    SymmArgs& a = args[i];
    a.in = ins[i];
    a.out_off = out_off;
    a.count = bytes;
    a.use_mc = (use_nvls && (emulated_ || heap_multicast())) ? 1 : 0;
  }
  const size_t pv = bytes / 16;
  LaunchCfg lc = launch_cfg(blocks_for(pv, cfg_.max_blocks), threads_for(pv, blocks_for(pv, cfg_.max_blocks), cfg_.threads), stream);
  last_algo_ = args[0].use_mc ? Algo::kNvls : Algo::kTwoShot;
  cudaError_t e = launch_all_gather_symm(emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

void CudaComm::abort() {
  volatile int* s = status_host_;
  s[8] = 1;
}
void CudaComm::clear_abort() {
  volatile int* s = status_host_;
  s[8] = 0;
}
bool CudaComm::aborted() const {
  volatile int* s = status_host_;
  return s[8] != 0;
}

bool CudaComm::fits_gemm_ar_norm(int rows, int hidden, int K) const {
  return rows > 0 && rows <= gemm_ar_norm_max_rows(hidden) && hidden % 128 == 0 && hidden / 8 <= 192 * 6 && K > 0 && K % 8 == 0 &&
         cfg_.ablate == kAblateNone;
}

cudaError_t CudaComm::gemm_ar_norm(const std::vector<GemmArNormArgs>& args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  cudaError_t e = launch_gemm_ar_norm(host_ctx_.data(), dev_ctx_table_, args.data(), nctx(), stream);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::sample_allgather(const std::vector<SampleArgs>& args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  cudaError_t e = launch_sample_allgather(host_ctx_.data(), dev_ctx_table_, args.data(), nctx(), stream);
  if (e == cudaSuccess) ++launches_;
  return e;
}

cudaError_t CudaComm::allreduce_residual_rmsnorm(int dtype, std::vector<FusedNormArgs> args, cudaStream_t stream) {
  CCL_CHECK_ARGS(args)
  DeviceGuard g(device_);
  enter_stream(stream);
  const FusedNormArgs& a0 = args[0];
  if (a0.hidden % 8 != 0 || a0.rows <= 0) return cudaErrorInvalidValue;
  int threads = std::min(512, std::max(32, ((a0.hidden / 8 + 31) / 32) * 32));  // kernel is compiled for <= 512 threads
  if (a0.hidden / 8 > threads * 4) return cudaErrorInvalidValue;
  if ((size_t)a0.rows * a0.hidden * 2 > fused_norm_capacity() && world_ > 1) return cudaErrorInvalidValue;
  for (auto& a : args) {
    a.ablate = cfg_.ablate;
    // small decode-sized inputs take the low-latency protocol (payload and epoch in one store)
    a.use_ll = (world_ > 1 && cfg_.ablate == kAblateNone && (size_t)a0.rows * a0.hidden * 4 <= kLLSlotBytes) ? 1 : 0;
  }
  LaunchCfg lc = launch_cfg(std::min(a0.rows, kMaxBlocks), threads, stream);
  cudaError_t e = launch_allreduce_residual_rmsnorm(dtype, emulated_ ? dev_ctx_table_ : host_ctx_.data(), upload(args, stream), lc);
  if (e == cudaSuccess) ++launches_;
  return e;
}

}  // namespace ccl
