// CUDA half of ProcessGroupCCL: owns the CudaComm (created lazily at the first CUDA collective,
// like the reference creates its communicators lazily, src/gpu/dpcpp_ccl.cpp:255-380), the
// communication stream, the stream fork/join and Work semantics (non-blocking wait = stream
// dependency, CCL_BLOCKING_WAIT = host poll with timeout, CCL_SAME_STREAM = run on the caller's
// stream; cf. src/gpu/dpcpp_ccl.cpp:382-472), the watchdog that turns device-side bounded-wait
// expiries into errors on the Work, and the NCCL point-to-point side channel.
#pragma once
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>

#include <functional>
#include <memory>
#include <mutex>

#include "cuda/CudaComm.h"
#include "pg/ProcessGroupCCL.hpp"

namespace ccl {

class NcclP2P;

// CUDA events are recycled through a process-wide pool: creating and destroying two or three
// events per collective costs more host time than launching the kernel.
struct PooledEvent {
  cudaEvent_t ev = nullptr;
  bool timing = false;
  int device = 0;
  ~PooledEvent();
  bool query() const { return cudaEventQuery(ev) == cudaSuccess; }
};
std::shared_ptr<PooledEvent> acquire_event(int device, bool timing);

class CudaBackendImpl {
 public:
  CudaBackendImpl(c10d::ProcessGroupCCL* pg, c10::intrusive_ptr<c10d::Store> store, int rank, int size);
  ~CudaBackendImpl();

  using LaunchFn = std::function<std::string(CudaComm&, cudaStream_t)>;  // returns the algorithm tag

  // Runs `fn` on the communication stream (or the current stream in same-stream mode) with the
  // proper event dependencies and returns the Work. `keep` tensors are kept alive / recorded on
  // the stream. `host_blocking`: wait() blocks the host until completion (barrier).
  c10::intrusive_ptr<c10d::Work> run(c10d::OpType type, const char* title, const at::Device& device,
                                     const LaunchFn& fn, const std::vector<at::Tensor>& keep,
                                     std::vector<at::Tensor> outs, std::vector<std::vector<at::Tensor>> nested,
                                     bool use_nested, uint64_t bytes, bool host_blocking = false);

  // NCCL p2p (send / recv, batched between start/endCoalescing).
  c10::intrusive_ptr<c10d::Work> p2p(bool is_send, at::Tensor& tensor, int peer, bool batched);
  void p2p_group_start();
  c10::intrusive_ptr<c10d::Work> p2p_group_end();
  bool p2p_batch_active() const { return p2p_batch_ops_ > 0; }

  CudaComm& comm(const at::Device& device);
  std::shared_ptr<CudaComm> comm_ptr(const at::Device& device);
  // Memory from the communicator's symmetric heap (see CudaComm::symm_alloc: collective in order).
  // The block goes back to the heap when the DataPtr / tensor dies; it keeps the communicator alive.
  c10::DataPtr symm_allocate(size_t bytes, const at::Device& device);
  at::Tensor symm_empty(int64_t numel, at::TensorOptions options);
  bool has_comm() const { return comm_ != nullptr; }
  c10::cuda::CUDAStream comm_stream(const at::Device& device);
  void shutdown();
  void abort();
  int status_code() const { return comm_ ? comm_->poll_status() : 0; }

 private:
  c10d::ProcessGroupCCL* pg_;
  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, size_;
  std::mutex mu_;
  std::shared_ptr<CudaComm> comm_;
  std::unique_ptr<c10::cuda::CUDAStream> stream_;
  std::shared_ptr<PooledEvent> fork_event_;
  std::unique_ptr<NcclP2P> nccl_;
  int p2p_batch_ops_ = 0;
  bool p2p_in_group_ = false;
  std::vector<at::Tensor> p2p_batch_tensors_;
  at::Device p2p_device_{at::kCUDA, 0};
};

// The process-wide watchdog: keeps in-flight CUDA work alive until its end event fires, then
// finishes it (or fails it when the communicator reported a device-side timeout).
class Watchdog {
 public:
  static Watchdog& get();
  struct Item {
    c10::intrusive_ptr<c10d::ProcessGroupCCL::AsyncWorkCCL> work;
    std::shared_ptr<PooledEvent> end;
    std::shared_ptr<CudaComm> comm;
    std::vector<at::Tensor> keep;
    uint64_t seq;
    std::chrono::milliseconds timeout{0};  // the group's timeout; 0 = no deadline (see Watchdog::loop)
  };
  void enqueue(Item item);
  void drain();  // blocks until every queued work has completed
  void stop();

 private:
  Watchdog();
  void loop();
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Item> q_;
  bool stop_ = false;
  bool busy_ = false;
  std::thread th_;
};

}  // namespace ccl
