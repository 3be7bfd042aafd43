#include "cuda/CudaBackend.h"
#include "cuda/Tuner.h"

#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <dlfcn.h>
#include <nccl.h>
#include <nvtx3/nvToolsExt.h>

#include <iostream>

#include "bindings/common.h"
#include "pg/Env.h"
#include "pg/Telemetry.h"
#include "pg/TensorChecks.h"

namespace ccl {

using c10d::ProcessGroupCCL;
using AsyncWork = ProcessGroupCCL::AsyncWorkCCL;

namespace {
struct EventPool {
  std::mutex mu;
  std::vector<cudaEvent_t> free_plain[16], free_timing[16];
};
EventPool& event_pool() {
  static EventPool* p = new EventPool();  // leaked: events may be returned during static destruction
  return *p;
}
}  // namespace

PooledEvent::~PooledEvent() {
  if (!ev) return;
  EventPool& p = event_pool();
  std::lock_guard<std::mutex> g(p.mu);
  (timing ? p.free_timing : p.free_plain)[device & 15].push_back(ev);
}

std::shared_ptr<PooledEvent> acquire_event(int device, bool timing) {
  auto e = std::make_shared<PooledEvent>();
  e->timing = timing;
  e->device = device;
  {
    EventPool& p = event_pool();
    std::lock_guard<std::mutex> g(p.mu);
    auto& v = (timing ? p.free_timing : p.free_plain)[device & 15];
    if (!v.empty()) {
      e->ev = v.back();
      v.pop_back();
    }
  }
  if (!e->ev) C10_CUDA_CHECK(cudaEventCreateWithFlags(&e->ev, timing ? cudaEventDefault : cudaEventDisableTiming));
  return e;
}

namespace {

[[noreturn]] void throw_dist_error(const std::string& msg) {
  throw c10::DistBackendError(c10::SourceLocation{"ccl", __FILE__, __LINE__}, msg);
}

std::string status_message(CudaComm& c) {
  int r = -1, p = -1, ph = -1;
  const int code = c.poll_status(&r, &p, &ph);
  if (code == 0) return "";
  if (code == kStatusAborted)
    return "ccl: collective aborted: rank " + std::to_string(r) + " gave up waiting for rank " + std::to_string(p) +
           " because the communicator was aborted (abort() on the process group, or its watchdog after the group's timeout)";
  return "ccl: device-side wait expired (code " + std::to_string(code) + "): rank " + std::to_string(r) +
         " waited for rank " + std::to_string(p) + " in phase " + std::to_string(ph) +
         "; the communicator is unusable, destroy the process group";
}

// Work of one CUDA collective.
class CudaWork : public AsyncWork {
 public:
  CudaWork(int rank, c10d::OpType op, const char* title, uint64_t seq, at::Device device)
      : AsyncWork(rank, op, title, seq), device_(device) {}

  bool isCompleted() override {
    if (Work::isCompleted()) return true;
    return end_ && end_->query();
  }

  bool wait(std::chrono::milliseconds timeout) override {
    if (blocking_ || host_blocking_) {
      const auto budget = (timeout == kNoTimeout || timeout.count() <= 0) ? timeout_ : timeout;
      const auto t0 = std::chrono::steady_clock::now();
      while (!end_->query()) {
        if (std::chrono::steady_clock::now() - t0 > budget) {
          std::cerr << "[ccl] rank " << rank_ << " collective #" << seq_ << " timed out after " << budget.count()
                    << " ms\n" << Telemetry::get().dump_flight();
          throw_dist_error("Caught collective operation timeout: Work ran for more than " +
                           std::to_string(budget.count()) + " milliseconds");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(10));
      }
      if (comm_) {
        const std::string m = status_message(*comm_);
        if (!m.empty()) throw_dist_error(m);
      }
    } else if (!same_stream_) {
      C10_CUDA_CHECK(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream(device_.index()).stream(), end_->ev, 0));
    }
    std::exception_ptr e;
    {
      std::lock_guard<std::mutex> g(mutex_);
      e = exception_;
    }
    if (e) std::rethrow_exception(e);
    return true;
  }

  void synchronize() override {
    if (!same_stream_ && end_) C10_CUDA_CHECK(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream(device_.index()).stream(), end_->ev, 0));
  }

  int cudaDevice() const override { return device_.index(); }

  float getDuration() const override {
    if (!start_ || !end_ || !timed_) return -1.f;
    if (!end_->query()) return -1.f;
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, start_->ev, end_->ev) != cudaSuccess) return -1.f;
    return ms;
  }

  // The future of CUDA work is completed in stream order: consumers of the future synchronise
  // with the stream the collective ran on.
  void completeFutureNow() override {
    if (stream_) {
      c10::cuda::CUDAStreamGuard g(*stream_);
      AsyncWork::completeFutureNow();
    } else {
      AsyncWork::completeFutureNow();
    }
  }

  std::shared_ptr<PooledEvent> start_, end_;
  std::optional<c10::cuda::CUDAStream> stream_;
  std::shared_ptr<CudaComm> comm_;
  bool blocking_ = false, same_stream_ = false, host_blocking_ = false, timed_ = false;
  std::chrono::milliseconds timeout_{10000};
  at::Device device_;
};

}  // namespace

// ------------------------------------------------------------------------------------------
// watchdog
// ------------------------------------------------------------------------------------------
Watchdog& Watchdog::get() {
  static Watchdog* w = new Watchdog();  // leaked on purpose: outlives static destruction order
  return *w;
}

Watchdog::Watchdog() : th_([this] { loop(); }) {}

void Watchdog::enqueue(Item item) {
  {
    std::lock_guard<std::mutex> g(mu_);
    q_.push_back(std::move(item));
  }
  cv_.notify_all();
}

void Watchdog::drain() {
  std::unique_lock<std::mutex> l(mu_);
  cv_.wait(l, [this] { return q_.empty() && !busy_; });
}

void Watchdog::stop() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (th_.joinable()) th_.join();
}

void Watchdog::loop() {
  std::unique_lock<std::mutex> l(mu_);
  while (true) {
    cv_.wait(l, [this] { return stop_ || !q_.empty(); });
    if (stop_ && q_.empty()) return;
    Item it = std::move(q_.front());
    q_.pop_front();
    busy_ = true;
    l.unlock();
    try {
      // works complete in stream order, so waiting on the oldest one first is enough
      // a coarse poll: waiters use the event directly, the watchdog only retires work.
      // Deadline: every device wait of the library is bounded (spin budget <= the group's timeout), so a work
      // normally ends or fails by itself. The deadline is the backstop for a spin budget configured longer than
      // the timeout: kGrace after the timeout the watchdog raises the communicator's abort word (every bounded
      // wait samples it and returns within about a millisecond, status "aborted"); if the event has not fired
      // kGiveUp later either, the work is failed without it and its tensors are leaked rather than freed under
      // a kernel that may still run.
      constexpr auto kGrace = std::chrono::seconds(2), kGiveUp = std::chrono::seconds(10);
      const auto t0 = std::chrono::steady_clock::now();
      bool raised = false, gave_up = false;
      while (!it.end->query()) {
        if (it.timeout.count() > 0) {
          const auto waited = std::chrono::steady_clock::now() - t0;
          if (!raised && waited > it.timeout + kGrace) {
            raised = true;
            std::cerr << "[ccl] watchdog: work " << it.seq << " is past its timeout of " << it.timeout.count()
                      << " ms; aborting the communicator\n" << Telemetry::get().dump_flight();
            if (it.comm) it.comm->abort();
          }
          if (raised && waited > it.timeout + kGrace + kGiveUp) {
            gave_up = true;
            break;
          }
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
      }
      Telemetry::get().record_complete(it.work->flight_slot, it.seq);
      if (gave_up) {
        static std::vector<std::vector<at::Tensor>>* leaked = new std::vector<std::vector<at::Tensor>>();
        leaked->push_back(std::move(it.keep));
        it.work->finishError(std::make_exception_ptr(c10::DistBackendError(
            c10::SourceLocation{"ccl", __FILE__, __LINE__},
            "ccl: watchdog gave up on work " + std::to_string(it.seq) + " after its timeout of " +
                std::to_string(it.timeout.count()) + " ms (the kernel did not end after the abort)")));
      } else {
        std::string m = it.comm ? status_message(*it.comm) : std::string();
        if (m.empty()) {
          it.work->finishOk();
        } else {
          std::cerr << "[ccl] " << m << "\n" << Telemetry::get().dump_flight();
          it.work->finishError(std::make_exception_ptr(
              c10::DistBackendError(c10::SourceLocation{"ccl", __FILE__, __LINE__}, m)));
        }
      }
    } catch (...) {
      it.work->finishError(std::current_exception());
    }
    it = Item{};
    l.lock();
    busy_ = false;
    cv_.notify_all();
  }
}

// ------------------------------------------------------------------------------------------
// NCCL point-to-point side channel (the only NCCL use of the backend)
// ------------------------------------------------------------------------------------------
class NcclP2P {
 public:
  NcclP2P(c10::intrusive_ptr<c10d::Store> store, int rank, int size) : store_(std::move(store)), rank_(rank), size_(size) {
    load();
  }
  ~NcclP2P() {
    for (auto& kv : comms_)
      if (kv.second) fn_destroy_(kv.second);
  }

  // 2-rank communicator per unordered pair (keyed "lo:hi", created by whichever side arrives,
  // the low rank publishes the id) or the group-wide communicator for batched transfers —
  // the same keying as the reference (src/utils.h:733-750; src/ccl_comm_collector.cpp:15-28).
  ncclComm_t get(const std::string& key, int nranks, int myrank, int device) {
    auto it = comms_.find(key);
    if (it != comms_.end()) return it->second;
    ncclUniqueId id;
    const std::string skey = "ccl/nccl/" + key;
    if (myrank == 0) {
      check(fn_get_id_(&id), "ncclGetUniqueId");
      store_->set(skey, std::vector<uint8_t>(reinterpret_cast<uint8_t*>(&id), reinterpret_cast<uint8_t*>(&id) + sizeof(id)));
    } else {
      auto v = store_->get(skey);
      TORCH_CHECK(v.size() == sizeof(id), "ccl: malformed NCCL id in store");
      std::memcpy(&id, v.data(), sizeof(id));
    }
    c10::cuda::CUDAGuard g((c10::DeviceIndex)device);
    ncclComm_t comm = nullptr;
    check(fn_init_(&comm, nranks, id, myrank), "ncclCommInitRank");
    comms_[key] = comm;
    return comm;
  }

  void send(const void* buf, size_t bytes, int peer, ncclComm_t comm, cudaStream_t s) {
    check(fn_send_(buf, bytes, ncclInt8, peer, comm, s), "ncclSend");
  }
  void recv(void* buf, size_t bytes, int peer, ncclComm_t comm, cudaStream_t s) {
    check(fn_recv_(buf, bytes, ncclInt8, peer, comm, s), "ncclRecv");
  }
  void group_start() { check(fn_gstart_(), "ncclGroupStart"); }
  void group_end() { check(fn_gend_(), "ncclGroupEnd"); }

 private:
  template <typename F>
  void sym(F& f, const char* name) {
    void* p = dlsym(RTLD_DEFAULT, name);
    if (!p && handle_) p = dlsym(handle_, name);
    TORCH_CHECK(p != nullptr, "ccl: NCCL symbol ", name, " not found (send/recv on CUDA tensors need NCCL)");
    f = reinterpret_cast<F>(p);
  }
  void load() {
    if (!dlsym(RTLD_DEFAULT, "ncclSend")) handle_ = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    sym(fn_get_id_, "ncclGetUniqueId");
    sym(fn_init_, "ncclCommInitRank");
    sym(fn_destroy_, "ncclCommDestroy");
    sym(fn_send_, "ncclSend");
    sym(fn_recv_, "ncclRecv");
    sym(fn_gstart_, "ncclGroupStart");
    sym(fn_gend_, "ncclGroupEnd");
    sym(fn_errstr_, "ncclGetErrorString");
  }
  void check(ncclResult_t r, const char* what) {
    TORCH_CHECK(r == ncclSuccess, "ccl: ", what, " failed: ", fn_errstr_(r));
  }

  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, size_;
  void* handle_ = nullptr;
  std::unordered_map<std::string, ncclComm_t> comms_;
  ncclResult_t (*fn_get_id_)(ncclUniqueId*) = nullptr;
  ncclResult_t (*fn_init_)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*fn_destroy_)(ncclComm_t) = nullptr;
  ncclResult_t (*fn_send_)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*fn_recv_)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*fn_gstart_)() = nullptr;
  ncclResult_t (*fn_gend_)() = nullptr;
  const char* (*fn_errstr_)(ncclResult_t) = nullptr;
};

// ------------------------------------------------------------------------------------------
// CudaBackendImpl
// ------------------------------------------------------------------------------------------
CudaBackendImpl::CudaBackendImpl(ProcessGroupCCL* pg, c10::intrusive_ptr<c10d::Store> store, int rank, int size)
    : pg_(pg), store_(std::move(store)), rank_(rank), size_(size) {}

CudaBackendImpl::~CudaBackendImpl() { shutdown(); }

CudaComm& CudaBackendImpl::comm(const at::Device& device) {
  std::lock_guard<std::mutex> g(mu_);
  if (!comm_) {
    const Env& env = Env::get();
    int dev = device.has_index() ? device.index() : (int)c10::cuda::current_device();
    CommConfig cfg;
    cfg.half_bytes = (size_t)env.arena_mb << 20;
    const int64_t pg_ms = pg_->timeout().count();
    cfg.spin_timeout_ms = env.spin_timeout_ms > 0 ? (uint64_t)env.spin_timeout_ms
                                                  : (uint64_t)std::max<int64_t>(1000, std::min<int64_t>(pg_ms, 30000));
    // measured thresholds for this machine first, explicit environment variables on top
    if (!env.tune_file.empty()) apply_tuning(parse_tune_file(env.tune_file), size_, &cfg);
    if (env.oneshot_max_bytes >= 0) cfg.oneshot_max_bytes = (size_t)env.oneshot_max_bytes;
    if (env.max_blocks > 0) cfg.max_blocks = std::min(env.max_blocks, (int)kMaxBlocks);
    if (env.threads > 0) cfg.threads = std::max(32, std::min(512, env.threads / 32 * 32));
    if (env.symm_heap_mb > 0) cfg.heap_bytes = (size_t)env.symm_heap_mb << 20;
    if (env.symm_min_bytes >= 0) cfg.symm_min_bytes = (size_t)env.symm_min_bytes;
    if (env.nvls_min_bytes >= 0) cfg.nvls_min_bytes = (size_t)env.nvls_min_bytes;
    if (env.round_mb >= 0) cfg.round_bytes = (size_t)env.round_mb << 20;
    cfg.symm = parse_symm_kind(env.symm_mem);
    if (env.nvls || env.algo == "nvls") {
      // the multicast object binds driver virtual-memory allocations only
      cfg.nvls = true;
      cfg.symm = SymmKind::kVmm;
    }
    if (env.algo == "oneshot") cfg.algo = Algo::kOneShot;
    else if (env.algo == "twoshot") cfg.algo = Algo::kTwoShot;
    else if (env.algo == "nvls") cfg.algo = Algo::kNvls;
    if (env.work_only) cfg.ablate = kAblateWorkOnly;
    if (env.sync_only) cfg.ablate = kAblateSyncOnly;
    comm_ = std::make_shared<CudaComm>(rank_, size_, dev, cfg, ccl_py::make_kv(store_), "ccl/cuda/" + device_key(at::Device(at::kCUDA, 0)));
    if (env.llm_allreduce_debug || env.log_level > 0)
      std::cout << "Allreduce goes to the peer-memory kernel path (arena " << env.arena_mb << " MB per half)." << std::endl;
  }
  return *comm_;
}

std::shared_ptr<CudaComm> CudaBackendImpl::comm_ptr(const at::Device& device) {
  (void)comm(device);
  std::lock_guard<std::mutex> g(mu_);
  return comm_;
}

namespace {
struct SymmBlock {
  std::shared_ptr<CudaComm> comm;  // keeps the heap mapped while the tensor lives
  void* ptr;
};
void release_symm_block(void* ctx) {
  auto* b = static_cast<SymmBlock*>(ctx);
  b->comm->symm_free(b->ptr);
  delete b;
}
}  // namespace

c10::DataPtr CudaBackendImpl::symm_allocate(size_t bytes, const at::Device& device) {
  std::shared_ptr<CudaComm> c = comm_ptr(device);
  void* p = c->symm_alloc(bytes);
  TORCH_CHECK(p != nullptr, "ccl: symmetric heap exhausted (", c->heap_in_use() >> 20, " MB of ", c->config().heap_bytes >> 20,
              " MB in use, ", bytes >> 20, " MB requested); raise CCL_SYMM_HEAP_MB");
  auto* blk = new SymmBlock{c, p};
  return c10::DataPtr(p, blk, &release_symm_block, at::Device(at::kCUDA, (c10::DeviceIndex)c->device()));
}

at::Tensor CudaBackendImpl::symm_empty(int64_t numel, at::TensorOptions options) {
  const at::Device dev = options.has_device() && options.device().is_cuda() && options.device().has_index()
                             ? options.device() : at::Device(at::kCUDA, c10::cuda::current_device());
  const auto dtype = options.has_dtype() ? c10::typeMetaToScalarType(options.dtype()) : at::kFloat;
  const size_t bytes = (size_t)numel * c10::elementSize(dtype);
  c10::DataPtr dp = symm_allocate(bytes, dev);
  auto storage = c10::make_intrusive<c10::StorageImpl>(c10::StorageImpl::use_byte_size_t(), bytes, std::move(dp), /*allocator=*/nullptr,
                                                        /*resizable=*/false);
  at::Tensor t = at::detail::make_tensor<at::TensorImpl>(std::move(storage), c10::DispatchKeySet(c10::DispatchKey::CUDA),
                                                         c10::scalarTypeToTypeMeta(dtype));
  t.unsafeGetTensorImpl()->set_sizes_contiguous({numel});
  return t;
}

c10::cuda::CUDAStream CudaBackendImpl::comm_stream(const at::Device& device) {
  std::lock_guard<std::mutex> g(mu_);
  if (!stream_) {
    const int dev = device.has_index() ? device.index() : (int)c10::cuda::current_device();
    stream_ = std::make_unique<c10::cuda::CUDAStream>(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, (c10::DeviceIndex)dev));
  }
  return *stream_;
}

c10::intrusive_ptr<c10d::Work> CudaBackendImpl::run(c10d::OpType type, const char* title, const at::Device& device,
                                                    const LaunchFn& fn, const std::vector<at::Tensor>& keep,
                                                    std::vector<at::Tensor> outs, std::vector<std::vector<at::Tensor>> nested,
                                                    bool use_nested, uint64_t bytes, bool host_blocking) {
  CudaComm& c = comm(device);
  if (c.poll_status() != 0) throw_dist_error(status_message(c));
  const int dev = c.device();
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)dev);
  const bool same = pg_->sameStream();
  const uint64_t seq = pg_->getSequenceNumberForGroup();
  auto work = c10::make_intrusive<CudaWork>(rank_, type, title, seq, at::Device(at::kCUDA, (c10::DeviceIndex)dev));
  if (use_nested) work->setOutputs(std::move(nested));
  else work->setOutputs(std::move(outs));
  work->blocking_ = pg_->blockingWait();
  work->same_stream_ = same;
  work->host_blocking_ = host_blocking;
  work->timeout_ = pg_->timeout();
  work->comm_ = comm_;
  work->timed_ = pg_->timingEnabled();

  c10::cuda::CUDAStream cur = c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)dev);
  c10::cuda::CUDAStream stream = same ? cur : comm_stream(device);
  work->stream_ = stream;
  if (!same) {
    // fork: the communication stream waits for what the caller has enqueued so far. One event
    // per backend is enough: a wait captures the record that precedes it.
    if (!fork_event_) fork_event_ = acquire_event(dev, false);
    C10_CUDA_CHECK(cudaEventRecord(fork_event_->ev, cur.stream()));
    C10_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), fork_event_->ev, 0));
  }
  if (work->timed_) {
    work->start_ = acquire_event(dev, true);
    C10_CUDA_CHECK(cudaEventRecord(work->start_->ev, stream.stream()));
  }
  std::string algo;
  {
    RECORD_FUNCTION(title, std::vector<c10::IValue>{});
    // NVTX range around the launches (a no-op unless a tool has injected the NVTX library)
    nvtxRangePushA(title);
    struct Pop {
      ~Pop() { nvtxRangePop(); }
    } pop;
    algo = fn(c, stream.stream());
  }
  work->end_ = acquire_event(dev, work->timed_);
  C10_CUDA_CHECK(cudaEventRecord(work->end_->ev, stream.stream()));
  work->flight_slot = Telemetry::get().record_start(seq, title, "cuda", bytes, algo.c_str());

  Watchdog::Item item;
  item.work = work;
  item.end = work->end_;
  item.comm = comm_;
  item.keep = keep;  // keeps the tensors alive until the kernels have run (instead of record_stream)
  item.seq = seq;
  item.timeout = pg_->timeout();
  Watchdog::get().enqueue(std::move(item));
  return work;
}

// ---- p2p ------------------------------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> CudaBackendImpl::p2p(bool is_send, at::Tensor& tensor, int peer, bool batched) {
  const int dev = tensor.device().index();
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)dev);
  if (!nccl_) nccl_ = std::make_unique<NcclP2P>(store_, rank_, size_);
  const size_t bytes = (size_t)tensor.numel() * tensor.element_size();
  const uint64_t seq = pg_->getSequenceNumberForGroup();
  auto make_work = [&](c10d::OpType t) {
    auto w = c10::make_intrusive<CudaWork>(rank_, t, is_send ? "oneccl_bindings_for_pytorch::cuda::send" : "oneccl_bindings_for_pytorch::cuda::recv", seq, tensor.device());
    w->setOutputs(std::vector<at::Tensor>{tensor});
    w->blocking_ = true;  // point-to-point waits poll on the host with a timeout, like the reference
    w->same_stream_ = pg_->sameStream();
    w->timeout_ = pg_->timeout();
    return w;
  };
  c10::cuda::CUDAStream cur = c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)dev);
  c10::cuda::CUDAStream stream = pg_->sameStream() ? cur : comm_stream(tensor.device());
  if (batched) {
    // inside start/endCoalescing: queue into one NCCL group on the group-wide communicator
    ncclComm_t comm = nccl_->get("world", size_, rank_, dev);
    if (!p2p_in_group_) {
      if (!pg_->sameStream()) {
        if (!fork_event_) fork_event_ = acquire_event(dev, false);
        C10_CUDA_CHECK(cudaEventRecord(fork_event_->ev, cur.stream()));
        C10_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), fork_event_->ev, 0));
      }
      nccl_->group_start();
      p2p_in_group_ = true;
      p2p_device_ = tensor.device();
    }
    if (is_send) nccl_->send(tensor.data_ptr(), bytes, peer, comm, stream.stream());
    else nccl_->recv(tensor.data_ptr(), bytes, peer, comm, stream.stream());
    ++p2p_batch_ops_;
    p2p_batch_tensors_.push_back(tensor);
    auto w = make_work(is_send ? c10d::OpType::SEND : c10d::OpType::RECV);
    w->end_ = acquire_event(dev, false);  // recorded before the group runs: completion is the Work of endCoalescing
    C10_CUDA_CHECK(cudaEventRecord(w->end_->ev, cur.stream()));
    w->finishOk();
    return w;
  }
  auto w = make_work(is_send ? c10d::OpType::SEND : c10d::OpType::RECV);
  if (!pg_->sameStream()) {
    if (!fork_event_) fork_event_ = acquire_event(dev, false);
    C10_CUDA_CHECK(cudaEventRecord(fork_event_->ev, cur.stream()));
    C10_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), fork_event_->ev, 0));
  }
  if (peer == rank_) {
    // self send/recv: a FIFO of pending sends matched by the next self-recv
    static thread_local std::deque<at::Tensor> self_q;
    if (is_send) {
      self_q.push_back(tensor.clone());
    } else {
      TORCH_CHECK(!self_q.empty(), "ccl: recv from self without a matching send");
      c10::cuda::CUDAStreamGuard sg(stream);
      tensor.copy_(self_q.front(), /*non_blocking=*/true);
      self_q.pop_front();
    }
  } else {
    const int lo = std::min(rank_, peer);
    ncclComm_t comm = nccl_->get(p2p_key(rank_, peer), 2, rank_ == lo ? 0 : 1, dev);
    const int target = rank_ == lo ? 1 : 0;
    if (is_send) nccl_->send(tensor.data_ptr(), bytes, target, comm, stream.stream());
    else nccl_->recv(tensor.data_ptr(), bytes, target, comm, stream.stream());
  }
  w->stream_ = stream;
  w->end_ = acquire_event(dev, false);
  C10_CUDA_CHECK(cudaEventRecord(w->end_->ev, stream.stream()));
  Watchdog::Item item;
  item.work = w;
  item.end = w->end_;
  item.keep = {tensor};
  item.seq = seq;
  item.timeout = pg_->timeout();
  Watchdog::get().enqueue(std::move(item));
  return w;
}

void CudaBackendImpl::p2p_group_start() {}

c10::intrusive_ptr<c10d::Work> CudaBackendImpl::p2p_group_end() {
  TORCH_CHECK(p2p_in_group_, "ccl: no batched point-to-point operations to close");
  const int dev = p2p_device_.index();
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)dev);
  nccl_->group_end();
  p2p_in_group_ = false;
  p2p_batch_ops_ = 0;
  c10::cuda::CUDAStream stream = pg_->sameStream() ? c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)dev) : comm_stream(p2p_device_);
  const uint64_t seq = pg_->getSequenceNumberForGroup();
  auto w = c10::make_intrusive<CudaWork>(rank_, c10d::OpType::COALESCED, "oneccl_bindings_for_pytorch::cuda::end_coalescing", seq, p2p_device_);
  w->setOutputs(std::vector<at::Tensor>{});
  w->blocking_ = pg_->blockingWait();
  w->same_stream_ = pg_->sameStream();
  w->timeout_ = pg_->timeout();
  w->stream_ = stream;
  w->end_ = acquire_event(dev, false);
  C10_CUDA_CHECK(cudaEventRecord(w->end_->ev, stream.stream()));
  Watchdog::Item item;
  item.work = w;
  item.end = w->end_;
  item.keep = std::move(p2p_batch_tensors_);
  p2p_batch_tensors_.clear();
  item.seq = seq;
  item.timeout = pg_->timeout();
  Watchdog::get().enqueue(std::move(item));
  return w;
}

void CudaBackendImpl::shutdown() {
  if (comm_ || nccl_) Watchdog::get().drain();
  nccl_.reset();
  comm_.reset();
  stream_.reset();
}

// Raises the communicator's abort word: every kernel that is (or will be) spinning on a peer
// returns within about a millisecond instead of after the spin budget, its Work fails with the
// "aborted" status, and further collectives on this group are refused.
void CudaBackendImpl::abort() {
  std::lock_guard<std::mutex> g(mu_);
  if (comm_) comm_->abort();
}

}  // namespace ccl
