#include "pg/ProcessGroupCCL.hpp"

#include <future>
#include <ATen/record_function.h>
#include <c10/util/Exception.h>
#include <torch/csrc/distributed/c10d/Utils.hpp>
#include <unistd.h>

#include <iostream>

#include "bindings/common.h"
#include "cpu/CpuCollectives.h"
#include "cpu/ShmComm.h"
#include "cuda/CudaBackend.h"
#include "pg/Env.h"
#include "pg/TaskThread.h"
#include "pg/Telemetry.h"
#include "pg/TensorChecks.h"

namespace c10d {

using ccl::Env;
using ccl::Telemetry;

namespace {

std::string tensors_str(const std::vector<at::Tensor>& v) {
  std::stringstream os;
  ccl::format_tensors(os, v);
  return os.str();
}
std::string tensors_str(const at::Tensor& t) {
  std::stringstream os;
  ccl::format_tensors(os, t);
  return os.str();
}
std::string tensors_str2(const std::vector<std::vector<at::Tensor>>& o, const std::vector<at::Tensor>& i) {
  std::stringstream os;
  os << "input ";
  ccl::format_tensors(os, i);
  os << " output ";
  ccl::format_tensors(os, o);
  return os.str();
}

std::vector<c10::IValue> to_ivalues(const std::vector<at::Tensor>& v) {
  std::vector<c10::IValue> r;
  r.reserve(v.size());
  for (const auto& t : v) r.emplace_back(t);
  return r;
}

uint64_t nbytes(const std::vector<at::Tensor>& v) {
  uint64_t b = 0;
  for (const auto& t : v) b += (uint64_t)t.numel() * t.element_size();
  return b;
}

ccl::cpu::ReduceDesc cpu_reduce_desc(const ReduceOp& op, at::ScalarType st, int world) {
  const ccl::ReduceSpec s = ccl::make_reduce_spec(op, st, world);
  ccl::cpu::ReduceDesc d;
  d.dtype = ccl_py::to_ccl_dtype(st);
  d.kind = s.kind;
  d.has_scale = s.has_scale;
  d.is_avg = s.is_avg;
  d.scale = s.scale;
  return d;
}

// Sends `n` tensors through CudaComm::multi in chunks of kMaxMulti (one launch per chunk). `head` carries mode / op /
// scale, `entry(m, i)` writes tensor i into slot m.n of a chunk. Returns false without launching anything when a chunk
// does not fit the staging arena; the caller then issues the tensors one by one.
template <typename Entry>
bool run_multi(ccl::CudaComm& c, int dtype, size_t n, const ccl::MultiArgs& head, cudaStream_t s, Entry entry) {
  std::vector<ccl::MultiArgs> chunks;
  for (size_t i = 0; i < n;) {
    ccl::MultiArgs m = head;
    m.n = 0;
    for (; i < n && m.n < ccl::kMaxMulti; ++i) {
      entry(m, i);
      if (m.count[m.n] != 0) ++m.n;   // empty tensors take no slot
    }
    if (m.n == 0) continue;
    if (!c.multi_fits(dtype, m)) return false;
    chunks.push_back(m);
  }
  for (auto& m : chunks) C10_CUDA_CHECK(c.multi(dtype, {m}, s));
  return true;
}

void fill_reduce(ccl::CollArgs& a, const ccl::ReduceSpec& s, at::ScalarType st) {
  a.op = s.kind;
  if (s.has_scale) {
    a.has_scale = (s.is_avg && !at::isFloatingType(st)) ? 2 : 1;
    a.scale = (float)s.scale;
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Work
// ------------------------------------------------------------------------------------------
ProcessGroupCCL::AsyncWorkCCL::AsyncWorkCCL(int rank, OpType op, const char* title, uint64_t seq)
    : Work(rank, op, title), seq_(seq) {}

ProcessGroupCCL::AsyncWorkCCL::~AsyncWorkCCL() = default;

void ProcessGroupCCL::AsyncWorkCCL::makeFuture(bool nested, const std::vector<c10::Device>& devices) {
  auto list_t = c10::ListType::create(c10::TensorType::get());
  future_ = c10::make_intrusive<c10::ivalue::Future>(nested ? c10::ListType::create(list_t) : list_t, devices);
}

void ProcessGroupCCL::AsyncWorkCCL::setOutputs(std::vector<at::Tensor> outs) {
  outputs_ = std::move(outs);
  nested_ = false;
}

void ProcessGroupCCL::AsyncWorkCCL::setOutputs(std::vector<std::vector<at::Tensor>> outs) {
  nested_outputs_ = std::move(outs);
  nested_ = true;
}

void ProcessGroupCCL::AsyncWorkCCL::completeFutureNow() {
  if (nested_) future_->markCompleted(c10::IValue(nested_outputs_));
  else future_->markCompleted(c10::IValue(outputs_));
}

c10::intrusive_ptr<c10::ivalue::Future> ProcessGroupCCL::AsyncWorkCCL::getFuture() {
  std::lock_guard<std::mutex> g(fut_mu_);
  if (!future_) {
    std::vector<c10::Device> devs;
    if (!nested_ && !outputs_.empty() && outputs_[0].is_cuda()) devs.push_back(outputs_[0].device());
    if (nested_ && !nested_outputs_.empty() && !nested_outputs_[0].empty() && nested_outputs_[0][0].is_cuda())
      devs.push_back(nested_outputs_[0][0].device());
    makeFuture(nested_, devs);
    if (done_err_) future_->setError(done_err_);
    else if (done_ok_ || !devs.empty()) completeFutureNow();  // CUDA work: stream-ordered completion
  }
  return future_;
}

std::vector<at::Tensor> ProcessGroupCCL::AsyncWorkCCL::result() {
  TORCH_CHECK(isCompleted(), "Work needs to be completed before calling result(). "
                             "Should call wait() before result().");
  TORCH_CHECK(!nested_ || nested_outputs_.size() <= 1,
              "work result does not support list of lists, use .getFuture() and value()");
  return nested_ ? (nested_outputs_.empty() ? std::vector<at::Tensor>{} : nested_outputs_[0]) : outputs_;
}

void ProcessGroupCCL::AsyncWorkCCL::finishOk() {
  {
    std::lock_guard<std::mutex> g(fut_mu_);
    done_ok_ = true;
    if (future_ && !future_->completed()) completeFutureNow();
  }
  finish();
  finished_.store(true, std::memory_order_release);
}

bool ProcessGroupCCL::AsyncWorkCCL::wait(std::chrono::milliseconds timeout) {
  const auto t0 = std::chrono::steady_clock::now();
  while (!finished_.load(std::memory_order_acquire) && std::chrono::steady_clock::now() - t0 < std::chrono::microseconds(60)) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  return Work::wait(timeout);
}

void ProcessGroupCCL::AsyncWorkCCL::finishError(std::exception_ptr e) {
  {
    std::lock_guard<std::mutex> g(fut_mu_);
    done_err_ = e;
    if (future_ && !future_->completed()) future_->setError(e);
  }
  finish(e);
  finished_.store(true, std::memory_order_release);
}

void ProcessGroupCCL::AsyncWorkCCL::abort() { aborted_.store(true); }

// ------------------------------------------------------------------------------------------
// construction
// ------------------------------------------------------------------------------------------
void ProcessGroupCCL::cclInitOnce() {
  static std::once_flag once;
  std::call_once(once, [] { (void)Env::get(); });
}

c10::intrusive_ptr<Backend> ProcessGroupCCL::createProcessGroupCCL(const c10::intrusive_ptr<Store>& store,
                                                                   int rank, int size,
                                                                   std::chrono::milliseconds timeout) {
  return c10::make_intrusive<ProcessGroupCCL>(store, rank, size, timeout);
}

ProcessGroupCCL::ProcessGroupCCL(const c10::intrusive_ptr<Store>& store, int rank, int size,
                                 std::chrono::milliseconds timeout)
    : Backend(rank, size), store_(store), timeout_(timeout) {
  const Env& env = Env::get();
  blocking_wait_ = env.blocking_wait;
  same_stream_ = env.same_stream;
  if (env.wait_gdb != 0) {
#ifdef NDEBUG
    TORCH_CHECK(false, "ONECCL_BINDINGS_FOR_PYTORCH_ENV_WAIT_GDB needs a debug build (DEBUG=1 python setup.py build_ext)");
#else
    volatile int released = 0;
    std::cout << "ccl: rank " << rank << " pid " << getpid() << " waiting for a debugger; set `released` to continue" << std::endl;
    while (!released) sleep(1);
#endif
  }
  init();
}

ProcessGroupCCL::~ProcessGroupCCL() {
  try {
    shutdown();
  } catch (...) {
  }
}

c10::intrusive_ptr<Backend::Options> ProcessGroupCCL::getBackendOptions() {
  return c10::static_intrusive_pointer_cast<Backend::Options>(c10::make_intrusive<Options>(timeout_));
}

std::chrono::milliseconds ProcessGroupCCL::opTimeout(std::chrono::milliseconds op_timeout) const {
  return (op_timeout == kUnsetTimeout || op_timeout.count() <= 0) ? timeout_ : op_timeout;
}

ccl::cpu::ShmComm& ProcessGroupCCL::shm() {
  std::lock_guard<std::mutex> g(init_mu_);
  if (!shm_) {
    ccl::cpu::ShmStore s;
    auto store = store_;
    s.set = [store](const std::string& k, const std::vector<uint8_t>& v) { store->set("ccl/" + k, v); };
    s.get = [store](const std::string& k) { return store->get("ccl/" + k); };
    s.add = [store](const std::string& k, int64_t v) { return store->add("ccl/" + k, v); };
    // ranks reach their first CPU collective at different times (imports, data loading): never less than 30 s
    try {
      const int64_t init_ms = Env::get().init_timeout_ms;
      shm_ = std::make_unique<ccl::cpu::ShmComm>(s, rank_, size_, (size_t)Env::get().shm_slot_mb << 20,
                                                 init_ms >= 0 ? std::chrono::milliseconds(init_ms)
                                                              : std::max(timeout_, std::chrono::milliseconds(30000)));
    } catch (const ccl::cpu::ShmTimeout& e) {
      C10_THROW_ERROR(DistBackendError, e.what());
    }
    cpu_worker_ = std::make_unique<ccl::TaskThread>();
  }
  return *shm_;
}

ccl::CudaBackendImpl& ProcessGroupCCL::cudaImpl(const at::Device& device) {
  std::lock_guard<std::mutex> g(init_mu_);
  if (!cuda_) cuda_ = std::make_unique<ccl::CudaBackendImpl>(this, store_, rank_, size_);
  return *cuda_;
}

void ProcessGroupCCL::eagerConnectSingleDevice(at::Device device) {
  if (device.is_cuda()) (void)cudaImpl(device).comm(device);
}

void ProcessGroupCCL::waitForPendingWorks() {
  // The host workers are FIFO: a marker task that has run means everything posted before it has run.
  std::vector<ccl::TaskThread*> workers;
  {
    std::lock_guard<std::mutex> g(init_mu_);
    if (cpu_worker_) workers.push_back(cpu_worker_.get());
    for (auto& kv : p2p_send_workers_) workers.push_back(kv.second.get());
    for (auto& kv : p2p_recv_workers_) workers.push_back(kv.second.get());
  }
  std::vector<std::future<void>> done;
  for (ccl::TaskThread* w : workers) {
    auto marker = std::make_shared<std::promise<void>>();
    done.push_back(marker->get_future());
    w->post([marker] { marker->set_value(); });
  }
  for (auto& f : done) f.wait();
  // CUDA works are retired by the process-wide watchdog, in issue order
  if (cuda_) ccl::Watchdog::get().drain();
}

void ProcessGroupCCL::abort() {
  aborted_.store(true);
  if (shm_) shm_->abort();
  if (cuda_) cuda_->abort();
}

void ProcessGroupCCL::shutdown() {
  if (cpu_worker_) cpu_worker_->drain_and_stop();
  for (auto& kv : p2p_send_workers_) kv.second->drain_and_stop();
  for (auto& kv : p2p_recv_workers_) kv.second->drain_and_stop();
  cpu_worker_.reset();
  p2p_send_workers_.clear();
  p2p_recv_workers_.clear();
  if (cuda_) {
    cuda_->shutdown();
    cuda_.reset();
  }
  shm_.reset();
}

ErrorType ProcessGroupCCL::getError() {
  if (cuda_ && cuda_->status_code() != 0) return ErrorType::TIMEOUT;
  if (aborted_.load() || (shm_ && shm_->aborted())) return ErrorType::COMM_ERROR;
  return ErrorType::SUCCESS;
}

// ------------------------------------------------------------------------------------------
// CPU execution engine: one FIFO worker for collectives, one per (peer, direction) for p2p so
// that a send never queues behind the matching recv of the other side.
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::enqueueCpu(OpType type, const char* title,
                                                     std::function<void(ccl::cpu::ShmComm&)> fn,
                                                     std::vector<at::Tensor> outs,
                                                     std::vector<std::vector<at::Tensor>> nested, bool use_nested,
                                                     uint64_t seq, size_t flight_slot) {
  TORCH_CHECK(!aborted_.load(), "ccl: process group was aborted");
  auto work = c10::make_intrusive<AsyncWorkCCL>(rank_, type, title, seq);
  if (use_nested) work->setOutputs(std::move(nested));
  else work->setOutputs(std::move(outs));
  work->flight_slot = flight_slot;
  ccl::cpu::ShmComm* comm = &shm();
  cpu_worker_->post([work, fn = std::move(fn), comm, seq]() {
    try {
      if (work->isAborted()) throw std::runtime_error("ccl: work aborted");
      fn(*comm);
      Telemetry::get().record_complete(work->flight_slot, seq);
      work->finishOk();
    } catch (const ccl::cpu::ShmTimeout& e) {
      std::cerr << "[ccl] " << e.what() << "\n" << Telemetry::get().dump_flight();
      work->finishError(std::make_exception_ptr(c10::DistBackendError(c10::SourceLocation{"ccl", __FILE__, __LINE__}, e.what())));
    } catch (...) {
      work->finishError(std::current_exception());
    }
  });
  return work;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::enqueueCpuP2P(OpType type, const char* title, int peer, bool is_send,
                                                        std::function<void(ccl::cpu::ShmComm&)> fn,
                                                        std::vector<at::Tensor> outs, uint64_t seq,
                                                        size_t flight_slot) {
  TORCH_CHECK(!aborted_.load(), "ccl: process group was aborted");
  auto work = c10::make_intrusive<AsyncWorkCCL>(rank_, type, title, seq);
  work->setOutputs(std::move(outs));
  work->flight_slot = flight_slot;
  ccl::cpu::ShmComm* comm = &shm();
  ccl::TaskThread* th;
  {
    std::lock_guard<std::mutex> g(init_mu_);
    auto& map = is_send ? p2p_send_workers_ : p2p_recv_workers_;
    auto& slot = map[peer];
    if (!slot) slot = std::make_unique<ccl::TaskThread>();
    th = slot.get();
  }
  th->post([work, fn = std::move(fn), comm, seq]() {
    try {
      fn(*comm);
      Telemetry::get().record_complete(work->flight_slot, seq);
      work->finishOk();
    } catch (const ccl::cpu::ShmTimeout& e) {
      work->finishError(std::make_exception_ptr(c10::DistBackendError(c10::SourceLocation{"ccl", __FILE__, __LINE__}, e.what())));
    } catch (...) {
      work->finishError(std::current_exception());
    }
  });
  return work;
}

// ------------------------------------------------------------------------------------------
// helpers shared by the op bodies
// ------------------------------------------------------------------------------------------
#define CCL_OP_PROLOGUE(OPNAME, FIRST_TENSOR, FLOW, TENSORS_STR, BYTES)                                  \
  const uint64_t seq = nextSeq();                                                                        \
  const bool on_cuda = (FIRST_TENSOR).is_cuda();                                                         \
  const char* devname = on_cuda ? "cuda" : "cpu";                                                        \
  const bool verbose__ = Env::get().verbose != 0;                                                        \
  ccl::OpTrace trace__(verbose__, devname, OPNAME, rank_, size_, seq, verbose__ ? std::string(FLOW) : std::string(), \
                       verbose__ ? (TENSORS_STR) : std::string());                                       \
  const uint64_t bytes__ = (BYTES);                                                                      \
  /* CUDA ops are entered into the flight recorder by the launcher, with the algorithm chosen */         \
  const size_t flight__ = on_cuda ? 0 : Telemetry::get().record_start(seq, OPNAME, devname, bytes__, ""); \
  struct HostTimer__ {                                                                                   \
    const char* op; const char* dev; uint64_t bytes; double t0;                                          \
    ~HostTimer__() { Telemetry::get().record_host_time(op, dev, bytes, "", Telemetry::now_us() - t0); }  \
  } host_timer__{OPNAME, devname, bytes__, Telemetry::now_us()};                                         \
  (void)flight__;                                                                                        \
  if (Env::get().debug_checks) debugConsistencyCheck(OPNAME, (FIRST_TENSOR).scalar_type(), bytes__);

// Debug mode (CCL_DEBUG_CHECKS=1): before a collective is enqueued, every rank publishes
// {op, dtype, bytes} under the group's own collective counter and compares with every peer, so that
// ranks that call different collectives (or the same one with different sizes) get an exception
// naming both sides instead of a timeout or silently wrong data. The reference has no such check
// (a mismatch there hangs inside oneCCL until the timeout, src/utils.h:295-319).
void ProcessGroupCCL::debugConsistencyCheck(const char* op, at::ScalarType dtype, uint64_t bytes) {
  const std::string name(op);
  if (size_ == 1 || name == "send" || name == "recv") return;
  // sizes may legitimately differ between ranks for the list / uneven forms
  const bool sized = name == "allreduce" || name == "allreduce_coalesced" || name == "broadcast" || name == "reduce" ||
                     name == "_allgather_base" || name == "_reduce_scatter_base" || name == "barrier";
  const uint64_t n = check_seq_++;
  const std::string mine = name + " " + c10::toString(dtype) + (sized ? " " + std::to_string(bytes) + " bytes" : "");
  const std::string base = "ccl/chk/";
  store_->set(base + std::to_string(n) + "/" + std::to_string(rank_), std::vector<uint8_t>(mine.begin(), mine.end()));
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) continue;
    const std::string key = base + std::to_string(n) + "/" + std::to_string(p);
    try {
      store_->wait({key}, timeout_);
    } catch (const std::exception&) {
      C10_THROW_ERROR(DistBackendError, "ccl: collective #" + std::to_string(n) + " (" + mine + ") on rank " + std::to_string(rank_) +
                                            ": rank " + std::to_string(p) + " did not enter a collective within the timeout");
    }
    const std::vector<uint8_t> v = store_->get(key);
    const std::string theirs(v.begin(), v.end());
    if (theirs != mine)
      C10_THROW_ERROR(DistBackendError, "ccl: collective mismatch at collective #" + std::to_string(n) + ": rank " + std::to_string(rank_) +
                                            " called [" + mine + "] but rank " + std::to_string(p) + " called [" + theirs + "]");
  }
  // everyone has passed collective n-1 only after reading this rank's key of n-2: safe to drop it
  if (n >= 2) store_->deleteKey(base + std::to_string(n - 2) + "/" + std::to_string(rank_));
}

static std::string flow_str(int from, int to) {
  return "[" + std::to_string(from) + "->" + std::to_string(to) + "]";
}

// ------------------------------------------------------------------------------------------
// symmetric tensors
// ------------------------------------------------------------------------------------------
at::Tensor ProcessGroupCCL::allocateTensor(long size, at::TensorOptions options) {
  TORCH_CHECK(size >= 0, "allocateTensor: negative size");
  const at::Device dev = options.has_device() && options.device().is_cuda() && options.device().has_index()
                             ? options.device() : at::Device(at::kCUDA, c10::cuda::current_device());
  at::Tensor t = cudaImpl(dev).symm_empty(size, options);
  // Symmetric allocation is collective in order: a rank that allocates in another order would address other memory
  // of its peers than they do. With CCL_DEBUG_CHECKS=1 the ranks compare {heap offset, bytes} of every allocation.
  if (Env::get().debug_checks && size_ > 1) {
    size_t off = 0;
    cudaImpl(dev).comm_ptr(dev)->symm_offset(t.data_ptr(), t.nbytes(), &off);
    const std::string what = "symm_alloc[heap offset " + std::to_string(off) + ", " + std::to_string(t.nbytes()) + " bytes]";
    debugConsistencyCheck(what.c_str(), t.scalar_type(), 0);
  }
  return t;
}

namespace {
// c10::Allocator over the symmetric heap, for torch.cuda.MemPool-style users.
class SymmAllocator : public c10::Allocator {
 public:
  explicit SymmAllocator(ProcessGroupCCL* pg) : pg_(pg) {}
  c10::DataPtr allocate(size_t n) override {
    const at::Device dev(at::kCUDA, c10::cuda::current_device());
    return pg_->cudaImpl(dev).symm_allocate(n, dev);
  }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    C10_CUDA_CHECK(cudaMemcpy(dest, src, count, cudaMemcpyDeviceToDevice));
  }

 private:
  ProcessGroupCCL* pg_;
};
}  // namespace

std::shared_ptr<c10::Allocator> ProcessGroupCCL::getMemAllocator() {
  return std::make_shared<SymmAllocator>(this);
}

// ------------------------------------------------------------------------------------------
// coalescing
// ------------------------------------------------------------------------------------------
void ProcessGroupCCL::startCoalescing() {
  ++coalescing_depth_;
  if (coalescing_depth_ == 1) coalesced_works_.clear();
}

c10::intrusive_ptr<Work> ProcessGroupCCL::endCoalescing() {
  TORCH_CHECK(coalescing_depth_ > 0, "endCoalescing called without startCoalescing");
  --coalescing_depth_;
  if (coalescing_depth_ > 0) return nullptr;
  // batched point-to-point ops on CUDA were queued into one NCCL group: close it
  if (cuda_ && cuda_->p2p_batch_active()) {
    coalesced_works_.clear();
    return cuda_->p2p_group_end();
  }
  auto works = std::move(coalesced_works_);
  coalesced_works_.clear();
  int cuda_dev = -1;
  std::vector<c10::intrusive_ptr<Work>> host_works;
  for (auto& w : works) {
    auto* aw = dynamic_cast<AsyncWorkCCL*>(w.get());
    const int d = aw ? aw->cudaDevice() : -1;
    if (d >= 0) cuda_dev = d;
    else host_works.push_back(w);
  }
  if (cuda_dev >= 0) {
    // CUDA collectives were issued in the window: the returned Work must order the CALLER's
    // stream after them. A marker launch on the communication stream does exactly that: its end
    // event is recorded after the last inner op, wait() / synchronize() make the current stream
    // wait for it, and the watchdog retires it. Host-side work of a mixed window is finished first.
    for (auto& w : host_works) w->wait();
    const at::Device dev(at::kCUDA, (c10::DeviceIndex)cuda_dev);
    return cudaImpl(dev).run(OpType::COALESCED, "oneccl_bindings_for_pytorch::end_coalescing", dev,
                             [](ccl::CudaComm&, cudaStream_t) { return std::string("marker"); }, {}, {}, {}, false, 0);
  }
  const uint64_t seq = nextSeq();
  auto work = c10::make_intrusive<AsyncWorkCCL>(rank_, OpType::COALESCED, "oneccl_bindings_for_pytorch::end_coalescing", seq);
  work->setOutputs(std::vector<at::Tensor>{});
  if (works.empty()) {
    work->finishOk();
    return work;
  }
  // Host-side work only: the window's Work completes when the last inner work does, from the
  // thread that completes it (a callback on each inner future) - no helper thread per call.
  struct Pending {
    std::atomic<int> left;
    std::mutex mu;
    std::exception_ptr err;
  };
  auto pending = std::make_shared<Pending>();
  pending->left.store((int)works.size());
  for (auto& w : works) {
    w->getFuture()->addCallback([work, pending](c10::ivalue::Future& f) {
      if (f.hasError()) {
        std::lock_guard<std::mutex> g(pending->mu);
        if (!pending->err) pending->err = f.exception_ptr();
      }
      if (pending->left.fetch_sub(1) == 1) {
        std::exception_ptr e;
        {
          std::lock_guard<std::mutex> g(pending->mu);
          e = pending->err;
        }
        if (e) work->finishError(e);
        else work->finishOk();
      }
    });
  }
  return work;
}

#define CCL_TRACK_COALESCED(W)                         \
  do {                                                 \
    if (coalescing_depth_ > 0) coalesced_works_.push_back(W); \
  } while (0)

// ------------------------------------------------------------------------------------------
// broadcast
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::broadcast(std::vector<at::Tensor>& tensors, const BroadcastOptions& opts) {
  ccl::check_rank(opts.rootRank, size_);
  ccl::check_single_tensor(tensors);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::broadcast", to_ivalues(tensors));
  CCL_OP_PROLOGUE("broadcast", tensors[0], flow_str((int)opts.rootRank, rank_), tensors_str(tensors), nbytes(tensors))
  at::Tensor t = tensors[0];
  const int root = (int)opts.rootRank;
  const auto tmo = opTimeout(opts.timeout);
  c10::intrusive_ptr<Work> w;
  if (on_cuda) {
    w = cudaImpl(t.device()).run(OpType::BROADCAST, "oneccl_bindings_for_pytorch::cuda::broadcast", t.device(),
        [t, root](ccl::CudaComm& c, cudaStream_t s) {
          if (c.world() == 1 || t.numel() == 0) return std::string("noop");
          ccl::CollArgs a;
          a.out = t.data_ptr();
          a.count = (uint64_t)t.numel() * t.element_size();
          a.root = root;
          a.mode = ccl::kBroadcast;
          C10_CUDA_CHECK(c.rooted({a}, s));
          return std::string("rooted");
        }, {t}, {t}, {}, false, bytes__);
  } else {
    w = enqueueCpu(OpType::BROADCAST, "oneccl_bindings_for_pytorch::cpu::broadcast",
        [t, root, tmo](ccl::cpu::ShmComm& c) {
          ccl::cpu::broadcast(c, t.data_ptr(), (size_t)t.numel() * t.element_size(), root, tmo);
        }, {t}, {}, false, seq, flight__);
  }
  CCL_TRACK_COALESCED(w);
  return w;
}

// ------------------------------------------------------------------------------------------
// allreduce / allreduce_coalesced
// ------------------------------------------------------------------------------------------
static c10::intrusive_ptr<Work> allreduce_impl(ProcessGroupCCL& pg, std::vector<at::Tensor> ts, const ReduceOp& rop,
                                               std::chrono::milliseconds tmo, OpType type, bool on_cuda,
                                               uint64_t seq, size_t flight, uint64_t bytes,
                                               const std::function<c10::intrusive_ptr<Work>(std::function<void(ccl::cpu::ShmComm&)>, std::vector<at::Tensor>)>& cpu_enqueue) {
  const int W = pg.getSize();
  if (on_cuda) {
    std::vector<ccl::ReduceSpec> specs;
    for (auto& t : ts) specs.push_back(ccl::make_reduce_spec(rop, t.scalar_type(), W));
    const bool disabled = Env::get().disable_allreduce;
    return pg.cudaImpl(ts[0].device()).run(type, "oneccl_bindings_for_pytorch::cuda::allreduce", ts[0].device(),
        [ts, specs, disabled](ccl::CudaComm& c, cudaStream_t s) {
          std::string tag = "noop";
          // a list of small tensors (DDP buckets, coalesced calls): one launch over a pointer table
          if (ts.size() > 1 && c.world() > 1 && !disabled) {
            bool uniform = true;
            for (size_t i = 1; i < ts.size(); ++i)
              uniform = uniform && specs[i].kind == specs[0].kind && specs[i].has_scale == specs[0].has_scale &&
                        specs[i].is_avg == specs[0].is_avg && specs[i].scale == specs[0].scale;
            ccl::CollArgs proto;
            fill_reduce(proto, specs[0], ts[0].scalar_type());
            ccl::MultiArgs head;
            head.mode = ccl::kMultiAllReduce;
            head.op = proto.op;
            head.has_scale = proto.has_scale;
            head.scale = proto.scale;
            if (uniform && run_multi(c, ccl_py::to_ccl_dtype(ts[0].scalar_type()), ts.size(), head, s, [&](ccl::MultiArgs& m, size_t i) {
                  m.in[m.n] = ts[i].data_ptr();
                  m.out[m.n] = ts[i].data_ptr();
                  m.count[m.n] = (uint64_t)ts[i].numel();
                }))
              return std::string("multi");
          }
          for (size_t i = 0; i < ts.size(); ++i) {
            const at::Tensor& t = ts[i];
            if (t.numel() == 0 || disabled) continue;
            if (c.world() == 1) {
              // one rank: only PREMUL_SUM changes the data
              if (specs[i].has_scale && !specs[i].is_avg) {
                c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(s, t.device().index()));
                const_cast<at::Tensor&>(t).mul_(specs[i].scale);
              }
              continue;
            }
            ccl::CollArgs a;
            a.in = t.data_ptr();
            a.out = t.data_ptr();
            a.count = t.numel();
            fill_reduce(a, specs[i], t.scalar_type());
            ccl::AlgoChoice ch{};
            C10_CUDA_CHECK(c.allreduce(ccl_py::to_ccl_dtype(t.scalar_type()), {a}, s, &ch));
            tag = ch.algo == ccl::Algo::kOneShot ? "oneshot" : (ch.algo == ccl::Algo::kNvls ? "nvls" : "twoshot");
          }
          return tag;
        }, ts, ts, {}, false, bytes);
  }
  std::vector<ccl::cpu::ReduceDesc> descs;
  for (auto& t : ts) descs.push_back(cpu_reduce_desc(rop, t.scalar_type(), W));
  return cpu_enqueue(
      [ts, descs, tmo](ccl::cpu::ShmComm& c) {
        for (size_t i = 0; i < ts.size(); ++i)
          ccl::cpu::allreduce(c, ts[i].data_ptr(), (size_t)ts[i].numel(), descs[i], tmo);
      }, ts);
}

c10::intrusive_ptr<Work> ProcessGroupCCL::allreduce(std::vector<at::Tensor>& tensors, const AllreduceOptions& opts) {
  ccl::check_single_tensor(tensors);
  TORCH_CHECK(!opts.sparseIndices.has_value(), "ccl: sparse allreduce is not supported");
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::allreduce", to_ivalues(tensors));
  CCL_OP_PROLOGUE("allreduce", tensors[0], "", tensors_str(tensors), nbytes(tensors))
  auto w = allreduce_impl(*this, tensors, opts.reduceOp, opTimeout(opts.timeout), OpType::ALLREDUCE, on_cuda, seq, flight__, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn, std::vector<at::Tensor> outs) {
        return enqueueCpu(OpType::ALLREDUCE, "oneccl_bindings_for_pytorch::cpu::allreduce", std::move(fn), std::move(outs), {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::allreduce_coalesced(std::vector<at::Tensor>& tensors, const AllreduceCoalescedOptions& opts) {
  TORCH_CHECK(!tensors.empty(), "allreduce_coalesced: empty tensor list");
  ccl::check_same_type(tensors[0], tensors);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::allreduce_coalesced", to_ivalues(tensors));
  CCL_OP_PROLOGUE("allreduce_coalesced", tensors[0], "", tensors_str(tensors), nbytes(tensors))
  auto w = allreduce_impl(*this, tensors, opts.reduceOp, opTimeout(opts.timeout), OpType::ALLREDUCE_COALESCED, on_cuda, seq, flight__, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn, std::vector<at::Tensor> outs) {
        return enqueueCpu(OpType::ALLREDUCE_COALESCED, "oneccl_bindings_for_pytorch::cpu::allreduce_coalesced", std::move(fn), std::move(outs), {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

// ------------------------------------------------------------------------------------------
// reduce
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::reduce(std::vector<at::Tensor>& tensors, const ReduceOptions& opts) {
  ccl::check_rank(opts.rootRank, size_);
  ccl::check_single_tensor(tensors);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::reduce", to_ivalues(tensors));
  CCL_OP_PROLOGUE("reduce", tensors[0], flow_str(rank_, (int)opts.rootRank), tensors_str(tensors), nbytes(tensors))
  at::Tensor t = tensors[0];
  const int root = (int)opts.rootRank;
  const auto tmo = opTimeout(opts.timeout);
  c10::intrusive_ptr<Work> w;
  if (on_cuda) {
    const ccl::ReduceSpec spec = ccl::make_reduce_spec(opts.reduceOp, t.scalar_type(), size_);
    w = cudaImpl(t.device()).run(OpType::REDUCE, "oneccl_bindings_for_pytorch::cuda::reduce", t.device(),
        [t, root, spec](ccl::CudaComm& c, cudaStream_t s) {
          if (c.world() == 1 || t.numel() == 0) return std::string("noop");
          ccl::CollArgs a;
          a.in = t.data_ptr();
          a.out = t.data_ptr();
          a.count = t.numel();
          a.root = root;
          fill_reduce(a, spec, t.scalar_type());
          C10_CUDA_CHECK(c.reduce(ccl_py::to_ccl_dtype(t.scalar_type()), {a}, s));
          return std::string("twoshot");
        }, {t}, {t}, {}, false, bytes__);
  } else {
    const auto desc = cpu_reduce_desc(opts.reduceOp, t.scalar_type(), size_);
    w = enqueueCpu(OpType::REDUCE, "oneccl_bindings_for_pytorch::cpu::reduce",
        [t, root, desc, tmo](ccl::cpu::ShmComm& c) { ccl::cpu::reduce(c, t.data_ptr(), (size_t)t.numel(), desc, root, tmo); },
        {t}, {}, false, seq, flight__);
  }
  CCL_TRACK_COALESCED(w);
  return w;
}

// ------------------------------------------------------------------------------------------
// allgather family
// ------------------------------------------------------------------------------------------
static c10::intrusive_ptr<Work> allgather_pieces(ProcessGroupCCL& pg, OpType type, const char* title_cuda, const char* title_cpu,
    std::vector<at::Tensor> ins, std::vector<std::vector<at::Tensor>> outs, bool nested_result,
    std::vector<at::Tensor> flat_result, std::chrono::milliseconds tmo, bool on_cuda, uint64_t seq, size_t flight, uint64_t bytes,
    const std::function<c10::intrusive_ptr<Work>(std::function<void(ccl::cpu::ShmComm&)>)>& cpu_enqueue) {
  if (on_cuda) {
    std::vector<at::Tensor> keep = ins;
    for (auto& l : outs) keep.insert(keep.end(), l.begin(), l.end());
    return pg.cudaImpl(ins[0].device()).run(type, title_cuda, ins[0].device(),
        [ins, outs](ccl::CudaComm& c, cudaStream_t s) {
          // several flat gathers (FSDP2 parameter groups, coalesced calls): one launch over a pointer table
          if (ins.size() > 1 && c.world() > 1) {
            bool flat = true;
            for (size_t i = 0; i < ins.size() && flat; ++i) {
              const size_t pb = (size_t)ins[i].numel() * ins[i].element_size();
              for (int p = 0; p < c.world() && flat; ++p)
                flat = (size_t)outs[i][p].numel() * outs[i][p].element_size() == pb &&
                       outs[i][p].data_ptr() == static_cast<char*>(outs[i][0].data_ptr()) + (size_t)p * pb;
            }
            ccl::MultiArgs head;
            head.mode = ccl::kMultiAllGather;
            if (flat && run_multi(c, ccl::kU8, ins.size(), head, s, [&](ccl::MultiArgs& m, size_t i) {
                  m.in[m.n] = ins[i].data_ptr();
                  m.out[m.n] = outs[i][0].data_ptr();
                  m.count[m.n] = (uint64_t)ins[i].numel() * ins[i].element_size();
                }))
              return std::string("multi");
          }
          for (size_t i = 0; i < ins.size(); ++i) {
            ccl::CollArgs a;
            a.in = ins[i].data_ptr();
            bool any = false;
            for (int p = 0; p < c.world(); ++p) {
              a.out_piece[p] = outs[i][p].data_ptr();
              a.out_cnt[p] = (uint64_t)outs[i][p].numel() * outs[i][p].element_size();
              any |= a.out_cnt[p] != 0;
            }
            if (!any) continue;
            if (c.world() == 1) {
              if (a.out_piece[0] != a.in) C10_CUDA_CHECK(cudaMemcpyAsync(a.out_piece[0], a.in, a.out_cnt[0], cudaMemcpyDeviceToDevice, s));
              continue;
            }
            C10_CUDA_CHECK(c.all_gather({a}, s));
          }
          return std::string("all_gather");
        }, keep, nested_result ? std::vector<at::Tensor>{} : flat_result, nested_result ? outs : std::vector<std::vector<at::Tensor>>{}, nested_result, bytes);
  }
  return cpu_enqueue([ins, outs, tmo](ccl::cpu::ShmComm& c) {
    for (size_t i = 0; i < ins.size(); ++i) {
      std::vector<void*> o(c.world());
      std::vector<size_t> b(c.world());
      for (int p = 0; p < c.world(); ++p) {
        o[p] = outs[i][p].data_ptr();
        b[p] = (size_t)outs[i][p].numel() * outs[i][p].element_size();
      }
      ccl::cpu::allgatherv(c, ins[i].data_ptr(), o, b, tmo);
    }
  });
}

c10::intrusive_ptr<Work> ProcessGroupCCL::allgather(std::vector<std::vector<at::Tensor>>& outputTensors,
                                                    std::vector<at::Tensor>& inputTensors, const AllgatherOptions& opts) {
  ccl::check_single_tensor(inputTensors);
  TORCH_CHECK(outputTensors.size() == 1, "allgather: multi-GPU collective is not supported");
  TORCH_CHECK((int)outputTensors[0].size() == size_, "allgather: number of output tensors should equal to the world size");
  ccl::check_same_type(inputTensors[0], outputTensors);
  TORCH_CHECK(outputTensors[0][rank_].numel() == inputTensors[0].numel(), "allgather: send and recv count doesn't match");
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::allgather", to_ivalues(inputTensors));
  CCL_OP_PROLOGUE("allgather", inputTensors[0], "", tensors_str2(outputTensors, inputTensors), nbytes(outputTensors[0]))
  auto outs = outputTensors;
  auto w = allgather_pieces(*this, OpType::ALLGATHER, "oneccl_bindings_for_pytorch::cuda::allgather", "oneccl_bindings_for_pytorch::cpu::allgather",
      inputTensors, outs, true, {}, opTimeout(opts.timeout), on_cuda, seq, flight__, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::ALLGATHER, "oneccl_bindings_for_pytorch::cpu::allgather", std::move(fn), {}, outs, true, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

static std::vector<at::Tensor> split_flat(const at::Tensor& flat, int world) {
  std::vector<at::Tensor> v;
  const int64_t n = flat.numel() / world;
  at::Tensor f = flat.view({-1});
  for (int p = 0; p < world; ++p) v.push_back(f.narrow(0, p * n, n));
  return v;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::_allgather_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer, const AllgatherOptions& opts) {
  ccl::check_tensor(inputBuffer);
  ccl::check_tensor(outputBuffer);
  TORCH_CHECK(inputBuffer.scalar_type() == outputBuffer.scalar_type(), "output tensor must have the same type as input tensor");
  TORCH_CHECK(inputBuffer.numel() * size_ == outputBuffer.numel(), "output tensor size must be equal to world_size times input tensor size");
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::_allgather_base", std::vector<c10::IValue>({inputBuffer}));
  CCL_OP_PROLOGUE("_allgather_base", inputBuffer, "", tensors_str(inputBuffer), (uint64_t)outputBuffer.numel() * outputBuffer.element_size())
  if (on_cuda) {
    // flat buffers: piece p of the output is at p * bytes, no per-piece tensors are needed
    at::Tensor in = inputBuffer, ob = outputBuffer;
    auto w = cudaImpl(in.device()).run(OpType::_ALLGATHER_BASE, "oneccl_bindings_for_pytorch::cuda::_allgather_base", in.device(),
        [in, ob](ccl::CudaComm& c, cudaStream_t s) {
          const size_t bytes = (size_t)in.numel() * in.element_size();
          if (bytes == 0) return std::string("noop");
          char* o = static_cast<char*>(ob.data_ptr());
          if (c.world() == 1) {
            if (o != in.data_ptr()) C10_CUDA_CHECK(cudaMemcpyAsync(o, in.data_ptr(), bytes, cudaMemcpyDeviceToDevice, s));
            return std::string("copy");
          }
          ccl::CollArgs a;
          a.in = in.data_ptr();
          for (int p = 0; p < c.world(); ++p) {
            a.out_piece[p] = o + (size_t)p * bytes;
            a.out_cnt[p] = bytes;
          }
          C10_CUDA_CHECK(c.all_gather({a}, s));
          return std::string("all_gather");
        }, {in, ob}, {ob}, {}, false, bytes__);
    CCL_TRACK_COALESCED(w);
    return w;
  }
  std::vector<at::Tensor> ins{inputBuffer};
  std::vector<std::vector<at::Tensor>> outs{split_flat(outputBuffer, size_)};
  at::Tensor ob = outputBuffer;
  auto w = allgather_pieces(*this, OpType::_ALLGATHER_BASE, "oneccl_bindings_for_pytorch::cuda::_allgather_base", "oneccl_bindings_for_pytorch::cpu::_allgather_base",
      ins, outs, false, {ob}, opTimeout(opts.timeout), on_cuda, seq, flight__, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::_ALLGATHER_BASE, "oneccl_bindings_for_pytorch::cpu::_allgather_base", std::move(fn), {ob}, {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::allgather_coalesced(std::vector<std::vector<at::Tensor>>&, std::vector<at::Tensor>&, const AllgatherOptions&) {
  TORCH_CHECK(false, "ProcessGroupCCL does not support allgather_coalesced");
}

c10::intrusive_ptr<Work> ProcessGroupCCL::allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const AllgatherOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size() && !inputs.empty(), "allgather_into_tensor_coalesced: input and output lists must have the same non-zero length");
  for (size_t i = 0; i < inputs.size(); ++i) {
    ccl::check_tensor(inputs[i]);
    ccl::check_tensor(outputs[i]);
    TORCH_CHECK(inputs[i].scalar_type() == outputs[i].scalar_type(), "output tensor must have the same type as input tensor");
    TORCH_CHECK(inputs[i].numel() * size_ == outputs[i].numel(), "output tensor size must be equal to world_size times input tensor size");
  }
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::allgather_into_tensor_coalesced", to_ivalues(inputs));
  CCL_OP_PROLOGUE("allgather_into_tensor_coalesced", inputs[0], "", tensors_str(inputs), nbytes(outputs))
  std::vector<std::vector<at::Tensor>> outs;
  for (auto& o : outputs) outs.push_back(split_flat(o, size_));
  auto flat = outputs;
  auto w = allgather_pieces(*this, OpType::COALESCED, "oneccl_bindings_for_pytorch::cuda::allgather_into_tensor_coalesced", "",
      inputs, outs, false, flat, opTimeout(opts.timeout), on_cuda, seq, flight__, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::COALESCED, "oneccl_bindings_for_pytorch::cpu::allgather_into_tensor_coalesced", std::move(fn), flat, {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

// ------------------------------------------------------------------------------------------
// gather / scatter
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::gather(std::vector<std::vector<at::Tensor>>& outputTensors, std::vector<at::Tensor>& inputTensors, const GatherOptions& opts) {
  ccl::check_rank(opts.rootRank, size_);
  ccl::check_single_tensor(inputTensors);
  const int root = (int)opts.rootRank;
  if (rank_ != root) {
    TORCH_CHECK(outputTensors.empty(), "gather: number of output tensors should be 0 for non-root");
  } else {
    TORCH_CHECK(outputTensors.size() == 1, "gather: multi-GPU collective is not supported");
    TORCH_CHECK((int)outputTensors[0].size() == size_, "gather: number of output tensors should equal to the world size");
    ccl::check_same_type(inputTensors[0], outputTensors);
    for (auto& t : outputTensors[0])
      TORCH_CHECK(t.numel() == inputTensors[0].numel(), "All tensor operands to scatter/gather must have the same number of elements");
  }
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::gather", to_ivalues(inputTensors));
  CCL_OP_PROLOGUE("gather", inputTensors[0], flow_str(rank_, root), tensors_str(inputTensors), nbytes(inputTensors))
  at::Tensor in = inputTensors[0];
  std::vector<at::Tensor> outs = rank_ == root ? outputTensors[0] : std::vector<at::Tensor>{};
  const auto tmo = opTimeout(opts.timeout);
  std::vector<std::vector<at::Tensor>> nested = outputTensors;
  if (on_cuda) {
    std::vector<at::Tensor> keep = outs;
    keep.push_back(in);
    const int me = rank_;
    return cudaImpl(in.device()).run(OpType::GATHER, "oneccl_bindings_for_pytorch::cuda::gather", in.device(),
        [in, outs, root, me](ccl::CudaComm& c, cudaStream_t s) {
          const size_t bytes = (size_t)in.numel() * in.element_size();
          if (bytes == 0) return std::string("noop");
          if (c.world() == 1) {
            if (outs[0].data_ptr() != in.data_ptr()) C10_CUDA_CHECK(cudaMemcpyAsync(outs[0].data_ptr(), in.data_ptr(), bytes, cudaMemcpyDeviceToDevice, s));
            return std::string("copy");
          }
          ccl::CollArgs a;
          a.in = in.data_ptr();
          a.count = bytes;
          a.root = root;
          a.mode = ccl::kGather;
          if (me == root) for (int p = 0; p < c.world(); ++p) a.out_piece[p] = outs[p].data_ptr();
          C10_CUDA_CHECK(c.rooted({a}, s));
          return std::string("rooted");
        }, keep, {}, nested, true, bytes__);
  }
  return enqueueCpu(OpType::GATHER, "oneccl_bindings_for_pytorch::cpu::gather",
      [in, outs, root, tmo](ccl::cpu::ShmComm& c) {
        std::vector<void*> o;
        for (auto& t : outs) o.push_back(t.data_ptr());
        ccl::cpu::gather(c, in.data_ptr(), o, (size_t)in.numel() * in.element_size(), root, tmo);
      }, {}, nested, true, seq, flight__);
}

c10::intrusive_ptr<Work> ProcessGroupCCL::scatter(std::vector<at::Tensor>& outputTensors, std::vector<std::vector<at::Tensor>>& inputTensors, const ScatterOptions& opts) {
  ccl::check_rank(opts.rootRank, size_);
  ccl::check_single_tensor(outputTensors);
  const int root = (int)opts.rootRank;
  if (rank_ != root) {
    TORCH_CHECK(inputTensors.empty(), "scatter: number of input tensors should be 0 for non-root");
  } else {
    TORCH_CHECK(inputTensors.size() == 1, "scatter: multi-GPU collective is not supported");
    TORCH_CHECK((int)inputTensors[0].size() == size_, "scatter: number of input tensors should equal to the world size");
    ccl::check_same_type(outputTensors[0], inputTensors);
    for (auto& t : inputTensors[0])
      TORCH_CHECK(t.numel() == outputTensors[0].numel(), "All tensor operands to scatter/gather must have the same number of elements");
  }
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::scatter", to_ivalues(outputTensors));
  CCL_OP_PROLOGUE("scatter", outputTensors[0], flow_str(root, rank_), tensors_str(outputTensors), nbytes(outputTensors))
  at::Tensor out = outputTensors[0];
  std::vector<at::Tensor> ins = rank_ == root ? inputTensors[0] : std::vector<at::Tensor>{};
  const auto tmo = opTimeout(opts.timeout);
  if (on_cuda) {
    std::vector<at::Tensor> keep = ins;
    keep.push_back(out);
    const int me = rank_;
    return cudaImpl(out.device()).run(OpType::SCATTER, "oneccl_bindings_for_pytorch::cuda::scatter", out.device(),
        [out, ins, root, me](ccl::CudaComm& c, cudaStream_t s) {
          const size_t bytes = (size_t)out.numel() * out.element_size();
          if (bytes == 0) return std::string("noop");
          if (c.world() == 1) {
            if (ins[0].data_ptr() != out.data_ptr()) C10_CUDA_CHECK(cudaMemcpyAsync(out.data_ptr(), ins[0].data_ptr(), bytes, cudaMemcpyDeviceToDevice, s));
            return std::string("copy");
          }
          ccl::CollArgs a;
          a.out = out.data_ptr();
          a.count = bytes;
          a.root = root;
          a.mode = ccl::kScatter;
          if (me == root) for (int p = 0; p < c.world(); ++p) a.in_piece[p] = ins[p].data_ptr();
          C10_CUDA_CHECK(c.rooted({a}, s));
          return std::string("rooted");
        }, keep, {out}, {}, false, bytes__);
  }
  return enqueueCpu(OpType::SCATTER, "oneccl_bindings_for_pytorch::cpu::scatter",
      [out, ins, root, tmo](ccl::cpu::ShmComm& c) {
        std::vector<const void*> i;
        for (auto& t : ins) i.push_back(t.data_ptr());
        ccl::cpu::scatter(c, i, out.data_ptr(), (size_t)out.numel() * out.element_size(), root, tmo);
      }, {out}, {}, false, seq, flight__);
}

// ------------------------------------------------------------------------------------------
// reduce_scatter family
// ------------------------------------------------------------------------------------------
static c10::intrusive_ptr<Work> reduce_scatter_pieces(ProcessGroupCCL& pg, OpType type, const char* title_cuda,
    std::vector<std::vector<at::Tensor>> ins, std::vector<at::Tensor> outs, const ReduceOp& rop, std::chrono::milliseconds tmo,
    bool on_cuda, uint64_t bytes, const std::function<c10::intrusive_ptr<Work>(std::function<void(ccl::cpu::ShmComm&)>)>& cpu_enqueue) {
  const int W = pg.getSize();
  if (on_cuda) {
    std::vector<at::Tensor> keep = outs;
    for (auto& l : ins) keep.insert(keep.end(), l.begin(), l.end());
    std::vector<ccl::ReduceSpec> specs;
    for (auto& o : outs) specs.push_back(ccl::make_reduce_spec(rop, o.scalar_type(), W));
    return pg.cudaImpl(outs[0].device()).run(type, title_cuda, outs[0].device(),
        [ins, outs, specs](ccl::CudaComm& c, cudaStream_t s) {
          // several flat reduce_scatters of one dtype (FSDP2 gradient groups, coalesced calls): one launch over a pointer table
          if (outs.size() > 1 && c.world() > 1) {
            bool flat = true;
            for (size_t i = 0; i < outs.size() && flat; ++i) {
              const size_t pb = (size_t)outs[i].numel() * outs[i].element_size();
              flat = outs[i].scalar_type() == outs[0].scalar_type() && specs[i].kind == specs[0].kind && specs[i].has_scale == specs[0].has_scale &&
                     specs[i].is_avg == specs[0].is_avg && specs[i].scale == specs[0].scale;
              for (int p = 0; p < c.world() && flat; ++p)
                flat = ins[i][p].numel() == outs[i].numel() && ins[i][p].scalar_type() == outs[i].scalar_type() &&
                       ins[i][p].data_ptr() == static_cast<char*>(ins[i][0].data_ptr()) + (size_t)p * pb;
            }
            ccl::CollArgs proto;
            fill_reduce(proto, specs[0], outs[0].scalar_type());
            ccl::MultiArgs head;
            head.mode = ccl::kMultiReduceScatter;
            head.op = proto.op;
            head.has_scale = proto.has_scale;
            head.scale = proto.scale;
            if (flat && run_multi(c, ccl_py::to_ccl_dtype(outs[0].scalar_type()), outs.size(), head, s, [&](ccl::MultiArgs& m, size_t i) {
                  m.in[m.n] = ins[i][0].data_ptr();
                  m.out[m.n] = outs[i].data_ptr();
                  m.count[m.n] = (uint64_t)outs[i].numel();
                }))
              return std::string("multi");
          }
          for (size_t i = 0; i < outs.size(); ++i) {
            ccl::CollArgs a;
            bool any = false;
            for (int p = 0; p < c.world(); ++p) {
              a.in_piece[p] = ins[i][p].data_ptr();
              a.in_cnt[p] = ins[i][p].numel();
              any |= a.in_cnt[p] != 0;
            }
            if (!any) continue;
            a.out = outs[i].data_ptr();
            if (c.world() == 1) {
              if (a.out != a.in_piece[0]) C10_CUDA_CHECK(cudaMemcpyAsync(a.out, a.in_piece[0], a.in_cnt[0] * outs[i].element_size(), cudaMemcpyDeviceToDevice, s));
              if (specs[i].has_scale && !specs[i].is_avg) {
                c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(s, outs[i].device().index()));
                const_cast<at::Tensor&>(outs[i]).mul_(specs[i].scale);
              }
              continue;
            }
            fill_reduce(a, specs[i], outs[i].scalar_type());
            const int dt = ccl_py::to_ccl_dtype(outs[i].scalar_type());
            C10_CUDA_CHECK(c.reduce_scatter(dt, dt, {a}, s));
          }
          return std::string("reduce_scatter");
        }, keep, outs, {}, false, bytes);
  }
  std::vector<ccl::cpu::ReduceDesc> descs;
  for (auto& o : outs) descs.push_back(cpu_reduce_desc(rop, o.scalar_type(), W));
  return cpu_enqueue([ins, outs, descs, tmo](ccl::cpu::ShmComm& c) {
    for (size_t i = 0; i < outs.size(); ++i) {
      std::vector<const void*> in(c.world());
      std::vector<size_t> cnt(c.world());
      for (int p = 0; p < c.world(); ++p) {
        in[p] = ins[i][p].data_ptr();
        cnt[p] = ins[i][p].numel();
      }
      ccl::cpu::reduce_scatterv(c, in, outs[i].data_ptr(), cnt, descs[i], tmo);
    }
  });
}

c10::intrusive_ptr<Work> ProcessGroupCCL::reduce_scatter(std::vector<at::Tensor>& outputTensors, std::vector<std::vector<at::Tensor>>& inputTensors, const ReduceScatterOptions& opts) {
  ccl::check_single_tensor(outputTensors);
  TORCH_CHECK(inputTensors.size() == 1, "reduce_scatter: multi-GPU collective is not supported");
  TORCH_CHECK((int)inputTensors[0].size() == size_, "reduce_scatter: number of input tensors should equal to the world size");
  ccl::check_same_type(outputTensors[0], inputTensors);
  TORCH_CHECK(inputTensors[0][rank_].numel() == outputTensors[0].numel(), "reduce_scatter: input piece of this rank and output size don't match");
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::reduce_scatter", to_ivalues(outputTensors));
  CCL_OP_PROLOGUE("reduce_scatter", outputTensors[0], "", tensors_str(outputTensors), nbytes(inputTensors[0]))
  auto outs = outputTensors;
  auto w = reduce_scatter_pieces(*this, OpType::REDUCE_SCATTER, "oneccl_bindings_for_pytorch::cuda::reduce_scatter", inputTensors, outs, opts.reduceOp,
      opTimeout(opts.timeout), on_cuda, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::REDUCE_SCATTER, "oneccl_bindings_for_pytorch::cpu::reduce_scatter", std::move(fn), outs, {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::_reduce_scatter_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer, const ReduceScatterOptions& opts) {
  ccl::check_tensor(inputBuffer);
  ccl::check_tensor(outputBuffer);
  TORCH_CHECK(inputBuffer.scalar_type() == outputBuffer.scalar_type(), "output tensor must have the same type as input tensor");
  TORCH_CHECK(outputBuffer.numel() * size_ == inputBuffer.numel(), "input tensor size must be equal to world_size times output tensor size");
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::_reduce_scatter_base", std::vector<c10::IValue>({inputBuffer}));
  CCL_OP_PROLOGUE("_reduce_scatter_base", inputBuffer, "", tensors_str(inputBuffer), (uint64_t)inputBuffer.numel() * inputBuffer.element_size())
  if (on_cuda) {
    at::Tensor in = inputBuffer, ob = outputBuffer;
    const ccl::ReduceSpec spec = ccl::make_reduce_spec(opts.reduceOp, ob.scalar_type(), size_);
    auto w = cudaImpl(in.device()).run(OpType::_REDUCE_SCATTER_BASE, "oneccl_bindings_for_pytorch::cuda::_reduce_scatter_base", in.device(),
        [in, ob, spec](ccl::CudaComm& c, cudaStream_t s) {
          const size_t n = ob.numel();
          if (n == 0) return std::string("noop");
          if (c.world() == 1) {
            if (ob.data_ptr() != in.data_ptr()) C10_CUDA_CHECK(cudaMemcpyAsync(ob.data_ptr(), in.data_ptr(), n * ob.element_size(), cudaMemcpyDeviceToDevice, s));
            if (spec.has_scale && !spec.is_avg) {
              c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(s, ob.device().index()));
              const_cast<at::Tensor&>(ob).mul_(spec.scale);
            }
            return std::string("copy");
          }
          ccl::CollArgs a;
          const char* i = static_cast<const char*>(in.data_ptr());
          for (int p = 0; p < c.world(); ++p) {
            a.in_piece[p] = i + (size_t)p * n * in.element_size();
            a.in_cnt[p] = n;
          }
          a.out = ob.data_ptr();
          fill_reduce(a, spec, ob.scalar_type());
          const int dt = ccl_py::to_ccl_dtype(ob.scalar_type());
          C10_CUDA_CHECK(c.reduce_scatter(dt, dt, {a}, s));
          return std::string("reduce_scatter");
        }, {in, ob}, {ob}, {}, false, bytes__);
    CCL_TRACK_COALESCED(w);
    return w;
  }
  std::vector<std::vector<at::Tensor>> ins{split_flat(inputBuffer, size_)};
  std::vector<at::Tensor> outs{outputBuffer};
  auto w = reduce_scatter_pieces(*this, OpType::_REDUCE_SCATTER_BASE, "oneccl_bindings_for_pytorch::cuda::_reduce_scatter_base", ins, outs, opts.reduceOp,
      opTimeout(opts.timeout), on_cuda, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::_REDUCE_SCATTER_BASE, "oneccl_bindings_for_pytorch::cpu::_reduce_scatter_base", std::move(fn), outs, {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size() && !inputs.empty(), "reduce_scatter_tensor_coalesced: input and output lists must have the same non-zero length");
  std::vector<std::vector<at::Tensor>> ins;
  for (size_t i = 0; i < inputs.size(); ++i) {
    ccl::check_tensor(inputs[i]);
    ccl::check_tensor(outputs[i]);
    TORCH_CHECK(inputs[i].scalar_type() == outputs[i].scalar_type(), "output tensor must have the same type as input tensor");
    TORCH_CHECK(outputs[i].numel() * size_ == inputs[i].numel(), "input tensor size must be equal to world_size times output tensor size");
    ins.push_back(split_flat(inputs[i], size_));
  }
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::reduce_scatter_tensor_coalesced", to_ivalues(inputs));
  CCL_OP_PROLOGUE("reduce_scatter_tensor_coalesced", inputs[0], "", tensors_str(inputs), nbytes(inputs))
  auto outs = outputs;
  auto w = reduce_scatter_pieces(*this, OpType::COALESCED, "oneccl_bindings_for_pytorch::cuda::reduce_scatter_tensor_coalesced", ins, outs, opts.reduceOp,
      opTimeout(opts.timeout), on_cuda, bytes__,
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::COALESCED, "oneccl_bindings_for_pytorch::cpu::reduce_scatter_tensor_coalesced", std::move(fn), outs, {}, false, seq, flight__);
      });
  CCL_TRACK_COALESCED(w);
  return w;
}

// ------------------------------------------------------------------------------------------
// alltoall family
// ------------------------------------------------------------------------------------------
static c10::intrusive_ptr<Work> alltoall_pieces(ProcessGroupCCL& pg, OpType type, const char* title_cuda,
    std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, bool uneven, std::vector<at::Tensor> result,
    std::chrono::milliseconds tmo, bool on_cuda, uint64_t bytes, const at::Device& dev,
    const std::function<c10::intrusive_ptr<Work>(std::function<void(ccl::cpu::ShmComm&)>)>& cpu_enqueue) {
  if (on_cuda) {
    std::vector<at::Tensor> keep = ins;
    keep.insert(keep.end(), outs.begin(), outs.end());
    return pg.cudaImpl(dev).run(type, title_cuda, dev,
        [ins, outs, uneven](ccl::CudaComm& c, cudaStream_t s) {
          ccl::CollArgs a;
          for (int p = 0; p < c.world(); ++p) {
            a.in_piece[p] = ins[p].data_ptr();
            a.in_cnt[p] = (uint64_t)ins[p].numel() * ins[p].element_size();
            a.out_piece[p] = outs[p].data_ptr();
            a.out_cnt[p] = (uint64_t)outs[p].numel() * outs[p].element_size();
          }
          if (c.world() == 1) {
            if (a.in_cnt[0] && a.in_piece[0] != a.out_piece[0])
              C10_CUDA_CHECK(cudaMemcpyAsync(a.out_piece[0], a.in_piece[0], a.in_cnt[0], cudaMemcpyDeviceToDevice, s));
            return std::string("copy");
          }
          C10_CUDA_CHECK(c.all_to_all({a}, uneven, s));
          return std::string(uneven ? "all_to_allv" : "all_to_all");
        }, keep, result, {}, false, bytes);
  }
  return cpu_enqueue([ins, outs, tmo](ccl::cpu::ShmComm& c) {
    std::vector<const void*> i(c.world());
    std::vector<void*> o(c.world());
    std::vector<size_t> sb(c.world()), rb(c.world());
    for (int p = 0; p < c.world(); ++p) {
      i[p] = ins[p].data_ptr();
      sb[p] = (size_t)ins[p].numel() * ins[p].element_size();
      o[p] = outs[p].data_ptr();
      rb[p] = (size_t)outs[p].numel() * outs[p].element_size();
    }
    ccl::cpu::alltoallv(c, i, sb, o, rb, tmo);
  });
}

static std::vector<at::Tensor> split_rows(const at::Tensor& t, const std::vector<int64_t>& splits, int world) {
  std::vector<at::Tensor> v;
  if (splits.empty()) {
    const int64_t n = t.size(0) / world;
    for (int p = 0; p < world; ++p) v.push_back(t.narrow(0, p * n, n));
  } else {
    int64_t off = 0;
    for (int p = 0; p < world; ++p) {
      v.push_back(t.narrow(0, off, splits[p]));
      off += splits[p];
    }
  }
  return v;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::alltoall_base(at::Tensor& outputTensor, at::Tensor& inputTensor, std::vector<int64_t>& outputSplitSizes,
                                                        std::vector<int64_t>& inputSplitSizes, const AllToAllOptions& opts) {
  ccl::check_tensor(inputTensor);
  ccl::check_tensor(outputTensor);
  TORCH_CHECK(inputTensor.scalar_type() == outputTensor.scalar_type(), "alltoall_base: tensors are not equal in size or data type");
  TORCH_CHECK(inputTensor.dim() > 0 && outputTensor.dim() > 0, "alltoall_base: tensors need at least one dimension");
  const bool uneven = !(outputSplitSizes.empty() && inputSplitSizes.empty());
  if (!uneven) {
    TORCH_CHECK(inputTensor.numel() == outputTensor.numel(), "alltoall_base: tensors are not equal in size or data type");
  }
  ccl::check_split_sizes(inputSplitSizes, inputTensor, size_);
  ccl::check_split_sizes(outputSplitSizes, outputTensor, size_);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::alltoall_base", std::vector<c10::IValue>({inputTensor}));
  CCL_OP_PROLOGUE("alltoall_base", inputTensor, "", tensors_str(inputTensor), (uint64_t)inputTensor.numel() * inputTensor.element_size())
  // On CUDA the form of the call selects the device protocol: without split lists the fixed-size exchange, with
  // them the one that first agrees on sizes. The choice is made from this rank's arguments alone, so either every
  // rank of the group passes split lists or none does; CCL_DEBUG_CHECKS=1 compares the form across ranks and
  // names the rank that differs instead of letting the mismatch end in a device-side timeout.
  if (on_cuda && Env::get().debug_checks)
    debugConsistencyCheck(uneven ? "alltoall_base[with split lists]" : "alltoall_base[without split lists]", inputTensor.scalar_type(), 0);
  if (on_cuda && !uneven) {
    at::Tensor in = inputTensor, ot2 = outputTensor;
    return cudaImpl(in.device()).run(OpType::ALLTOALL_BASE, "oneccl_bindings_for_pytorch::cuda::alltoall_base", in.device(),
        [in, ot2](ccl::CudaComm& c, cudaStream_t s) {
          const size_t total = (size_t)in.numel() * in.element_size();
          if (total == 0) return std::string("noop");
          if (c.world() == 1) {
            if (ot2.data_ptr() != in.data_ptr()) C10_CUDA_CHECK(cudaMemcpyAsync(ot2.data_ptr(), in.data_ptr(), total, cudaMemcpyDeviceToDevice, s));
            return std::string("copy");
          }
          const size_t piece = total / c.world();
          ccl::CollArgs a;
          for (int p = 0; p < c.world(); ++p) {
            a.in_piece[p] = static_cast<const char*>(in.data_ptr()) + (size_t)p * piece;
            a.out_piece[p] = static_cast<char*>(ot2.data_ptr()) + (size_t)p * piece;
            a.in_cnt[p] = piece;
            a.out_cnt[p] = piece;
          }
          C10_CUDA_CHECK(c.all_to_all({a}, false, s));
          return std::string("all_to_all");
        }, {in, ot2}, {ot2}, {}, false, bytes__);
  }
  auto ins = split_rows(inputTensor, inputSplitSizes, size_);
  auto outs = split_rows(outputTensor, outputSplitSizes, size_);
  at::Tensor ot = outputTensor;
  return alltoall_pieces(*this, OpType::ALLTOALL_BASE, "oneccl_bindings_for_pytorch::cuda::alltoall_base", ins, outs, uneven, {ot},
      opTimeout(opts.timeout), on_cuda, bytes__, inputTensor.device(),
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::ALLTOALL_BASE, "oneccl_bindings_for_pytorch::cpu::alltoall_base", std::move(fn), {ot}, {}, false, seq, flight__);
      });
}

c10::intrusive_ptr<Work> ProcessGroupCCL::alltoall(std::vector<at::Tensor>& outputTensors, std::vector<at::Tensor>& inputTensors, const AllToAllOptions& opts) {
  TORCH_CHECK((int)inputTensors.size() == size_, "alltoall: number of input tensors are not equal to group size");
  TORCH_CHECK((int)outputTensors.size() == size_, "alltoall: number of output tensors are not equal to group size");
  ccl::check_same_type(inputTensors[0], inputTensors);
  ccl::check_same_type(inputTensors[0], outputTensors);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::alltoall", to_ivalues(inputTensors));
  CCL_OP_PROLOGUE("alltoall", inputTensors[0], "", tensors_str(inputTensors), nbytes(inputTensors))
  auto outs = outputTensors;
  return alltoall_pieces(*this, OpType::ALLTOALL, "oneccl_bindings_for_pytorch::cuda::alltoall", inputTensors, outs, true, outs,
      opTimeout(opts.timeout), on_cuda, bytes__, inputTensors[0].device(),
      [&](std::function<void(ccl::cpu::ShmComm&)> fn) {
        return enqueueCpu(OpType::ALLTOALL, "oneccl_bindings_for_pytorch::cpu::alltoall", std::move(fn), outs, {}, false, seq, flight__);
      });
}

// ------------------------------------------------------------------------------------------
// point to point
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::send(std::vector<at::Tensor>& tensors, int dstRank, int /*tag*/) {
  ccl::check_single_tensor(tensors);
  ccl::check_rank(dstRank, size_);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::send", to_ivalues(tensors));
  CCL_OP_PROLOGUE("send", tensors[0], flow_str(rank_, dstRank), tensors_str(tensors), nbytes(tensors))
  at::Tensor t = tensors[0];
  if (on_cuda) return cudaImpl(t.device()).p2p(true, t, dstRank, coalescing_depth_ > 0);
  const auto tmo = opTimeout(kUnsetTimeout);
  auto w = enqueueCpuP2P(OpType::SEND, "oneccl_bindings_for_pytorch::cpu::send", dstRank, true,
      [t, dstRank, tmo](ccl::cpu::ShmComm& c) { c.send(t.data_ptr(), (size_t)t.numel() * t.element_size(), dstRank, tmo); },
      {t}, seq, flight__);
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::recv(std::vector<at::Tensor>& tensors, int srcRank, int /*tag*/) {
  ccl::check_single_tensor(tensors);
  ccl::check_rank(srcRank, size_);
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::recv", to_ivalues(tensors));
  CCL_OP_PROLOGUE("recv", tensors[0], flow_str(srcRank, rank_), tensors_str(tensors), nbytes(tensors))
  at::Tensor t = tensors[0];
  if (on_cuda) return cudaImpl(t.device()).p2p(false, t, srcRank, coalescing_depth_ > 0);
  const auto tmo = opTimeout(kUnsetTimeout);
  auto w = enqueueCpuP2P(OpType::RECV, "oneccl_bindings_for_pytorch::cpu::recv", srcRank, false,
      [t, srcRank, tmo](ccl::cpu::ShmComm& c) { c.recv(t.data_ptr(), (size_t)t.numel() * t.element_size(), srcRank, tmo); },
      {t}, seq, flight__);
  CCL_TRACK_COALESCED(w);
  return w;
}

c10::intrusive_ptr<Work> ProcessGroupCCL::recvAnysource(std::vector<at::Tensor>&, int) {
  TORCH_CHECK(false, "ProcessGroupCCL does not support recvAnysource");
}

// ------------------------------------------------------------------------------------------
// barrier
// ------------------------------------------------------------------------------------------
c10::intrusive_ptr<Work> ProcessGroupCCL::barrier(const BarrierOptions& opts) {
  RECORD_FUNCTION("oneccl_bindings_for_pytorch::barrier", std::vector<c10::IValue>{});
  // The device is chosen like torch does for its own backends: an explicit device / device_ids
  // wins; otherwise a group that has already used CUDA synchronises on the device.
  bool use_cuda = false;
  at::Device dev(at::kCPU);
  if (opts.device.has_value() && opts.device->is_cuda()) {
    use_cuda = true;
    dev = *opts.device;
  } else if (!opts.device_ids.empty()) {
    use_cuda = true;
    dev = at::Device(at::kCUDA, (c10::DeviceIndex)opts.device_ids[0]);
  } else if (!opts.device.has_value() && cuda_ && cuda_->has_comm()) {
    use_cuda = true;
    dev = at::Device(at::kCUDA, (c10::DeviceIndex)cuda_->comm(at::Device(at::kCUDA)).device());
  }
  at::Tensor probe = use_cuda ? at::empty({0}, at::TensorOptions().device(dev)) : at::empty({0});
  CCL_OP_PROLOGUE("barrier", probe, "", std::string("[]"), 0)
  if (on_cuda) {
    return cudaImpl(dev).run(OpType::BARRIER, "oneccl_bindings_for_pytorch::cuda::barrier", dev,
        [](ccl::CudaComm& c, cudaStream_t s) {
          if (c.world() > 1) C10_CUDA_CHECK(c.barrier(s));
          return std::string("barrier");
        }, {}, {}, {}, false, 0, /*host_blocking=*/true);
  }
  const auto tmo = opTimeout(opts.timeout);
  return enqueueCpu(OpType::BARRIER, "oneccl_bindings_for_pytorch::cpu::barrier",
      [tmo](ccl::cpu::ShmComm& c) { ccl::cpu::barrier(c, tmo); }, {}, {}, false, seq, flight__);
}

}  // namespace c10d
