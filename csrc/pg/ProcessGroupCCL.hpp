// c10d backend "ccl" for CPU and CUDA tensors.
//
// Same public surface as intel/torch-ccl's c10d::ProcessGroupCCL (src/ProcessGroupCCL.hpp:
// 111-310): constructor (store, rank, size, timeout), createProcessGroupCCL, every c10d
// Backend collective / point-to-point virtual, start/endCoalescing, the AsyncWork type with a
// future and result(). Differences by design: no runtime stub registry (device routing is a
// switch), no process-global mutex, futures complete when the work completes (CPU) or are
// stream-ordered (CUDA) instead of at enqueue time, and the optional Backend virtuals
// setTimeout / abort / shutdown / sequence numbers / allocateTensor / getMemAllocator are implemented.
#pragma once
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace ccl {
namespace cpu {
class ShmComm;
}
class CudaBackendImpl;
class TaskThread;
}  // namespace ccl

namespace c10d {

constexpr const char* CCL_BACKEND_NAME = "ccl";

class ProcessGroupCCL : public Backend {
 public:
  // Work of one collective or point-to-point operation.
  class AsyncWorkCCL : public Work {
   public:
    AsyncWorkCCL(int rank, OpType op, const char* title, uint64_t seq);
    ~AsyncWorkCCL() override;

    // The future is created on first request (most callers only wait()); for CUDA work it is
    // completed in stream order, for CPU work when the operation has run.
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;
    std::vector<at::Tensor> result() override;
    uint64_t getSequencenumber() const override { return seq_; }
    float getDuration() const override { return duration_ms_; }
    void abort() override;
    bool isAborted() const { return aborted_.load(); }
    // Index of the CUDA device the work's kernels run on, or -1 for host-side work.
    virtual int cudaDevice() const { return -1; }
    // Polls for completion for a few tens of microseconds before blocking on the condition
    // variable: a small CPU collective finishes sooner than a sleeping thread wakes up.
    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;

    // Output tensors: a flat list or (gather-type ops) a list of lists.
    void setOutputs(std::vector<at::Tensor> outs);
    void setOutputs(std::vector<std::vector<at::Tensor>> outs);
    // Completion: marks the future and wakes waiters.
    void finishOk();
    void finishError(std::exception_ptr e);

    size_t flight_slot = 0;

   protected:
    void makeFuture(bool nested, const std::vector<c10::Device>& devices);
    virtual void completeFutureNow();  // marks future_ completed with the outputs
    std::mutex fut_mu_;
    bool done_ok_ = false;
    std::exception_ptr done_err_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
    std::vector<at::Tensor> outputs_;
    std::vector<std::vector<at::Tensor>> nested_outputs_;
    bool nested_ = false;
    uint64_t seq_;
    float duration_ms_ = -1.f;
    std::atomic<bool> aborted_{false};
    std::atomic<bool> finished_{false};
  };

  struct Options : Backend::Options {
    explicit Options(std::chrono::milliseconds timeout = std::chrono::milliseconds(OP_TIMEOUT_MILLIS))
        : Backend::Options(CCL_BACKEND_NAME, timeout) {}
  };

  static constexpr int64_t OP_TIMEOUT_MILLIS = 10 * 1000;

  explicit ProcessGroupCCL(const c10::intrusive_ptr<Store>& store, int rank, int size,
                           std::chrono::milliseconds timeout = std::chrono::milliseconds(OP_TIMEOUT_MILLIS));
  ~ProcessGroupCCL() override;

  static c10::intrusive_ptr<Backend> createProcessGroupCCL(const c10::intrusive_ptr<Store>& store, int rank,
                                                           int size,
                                                           std::chrono::milliseconds timeout = std::chrono::milliseconds(OP_TIMEOUT_MILLIS));
  static void cclInitOnce();

  const std::string getBackendName() const override { return std::string(CCL_BACKEND_NAME); }
  c10::intrusive_ptr<Backend::Options> getBackendOptions() override;

  bool supportsCoalescing() const override { return true; }
  void startCoalescing() override;
  c10::intrusive_ptr<Work> endCoalescing() override;

  c10::intrusive_ptr<Work> broadcast(std::vector<at::Tensor>& tensors, const BroadcastOptions& opts = BroadcastOptions()) override;
  c10::intrusive_ptr<Work> allreduce(std::vector<at::Tensor>& tensors, const AllreduceOptions& opts = AllreduceOptions()) override;
  c10::intrusive_ptr<Work> allreduce_coalesced(std::vector<at::Tensor>& tensors, const AllreduceCoalescedOptions& opts = AllreduceCoalescedOptions()) override;
  c10::intrusive_ptr<Work> reduce(std::vector<at::Tensor>& tensors, const ReduceOptions& opts = ReduceOptions()) override;
  c10::intrusive_ptr<Work> allgather(std::vector<std::vector<at::Tensor>>& outputTensors, std::vector<at::Tensor>& inputTensors, const AllgatherOptions& opts = AllgatherOptions()) override;
  c10::intrusive_ptr<Work> _allgather_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer, const AllgatherOptions& opts = AllgatherOptions()) override;
  c10::intrusive_ptr<Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& outputTensorLists, std::vector<at::Tensor>& inputTensors, const AllgatherOptions& opts = AllgatherOptions()) override;
  c10::intrusive_ptr<Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const AllgatherOptions& opts = AllgatherOptions()) override;
  c10::intrusive_ptr<Work> gather(std::vector<std::vector<at::Tensor>>& outputTensors, std::vector<at::Tensor>& inputTensors, const GatherOptions& opts = GatherOptions()) override;
  c10::intrusive_ptr<Work> scatter(std::vector<at::Tensor>& outputTensors, std::vector<std::vector<at::Tensor>>& inputTensors, const ScatterOptions& opts = ScatterOptions()) override;
  c10::intrusive_ptr<Work> reduce_scatter(std::vector<at::Tensor>& outputTensors, std::vector<std::vector<at::Tensor>>& inputTensors, const ReduceScatterOptions& opts = ReduceScatterOptions()) override;
  c10::intrusive_ptr<Work> _reduce_scatter_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer, const ReduceScatterOptions& opts = ReduceScatterOptions()) override;
  c10::intrusive_ptr<Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const ReduceScatterOptions& opts = ReduceScatterOptions()) override;
  c10::intrusive_ptr<Work> alltoall_base(at::Tensor& outputTensor, at::Tensor& inputTensor, std::vector<int64_t>& outputSplitSizes, std::vector<int64_t>& inputSplitSizes, const AllToAllOptions& opts = AllToAllOptions()) override;
  c10::intrusive_ptr<Work> alltoall(std::vector<at::Tensor>& outputTensors, std::vector<at::Tensor>& inputTensors, const AllToAllOptions& opts = AllToAllOptions()) override;
  c10::intrusive_ptr<Work> send(std::vector<at::Tensor>& tensors, int dstRank, int tag) override;
  c10::intrusive_ptr<Work> recv(std::vector<at::Tensor>& tensors, int srcRank, int tag) override;
  c10::intrusive_ptr<Work> recvAnysource(std::vector<at::Tensor>& tensors, int tag) override;
  c10::intrusive_ptr<Work> barrier(const BarrierOptions& opts = BarrierOptions()) override;

  void setTimeout(std::chrono::milliseconds timeout) override { timeout_ = timeout; }
  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_.load(); }
  void enableCollectivesTiming() override { timing_enabled_ = true; }
  void waitForPendingWorks() override;   // returns when every Work issued so far has been completed (or failed)
  void eagerConnectSingleDevice(at::Device device) override;
  void abort() override;
  void shutdown() override;
  ErrorType getError() override;
  // Symmetric ("registered") tensors: memory that every rank of the group maps, so that collectives
  // on it run zero-copy over NVLink instead of staging through the arena. Allocation is collective
  // in order: every rank allocates the same sizes in the same order (and drops them in the same order).
  bool supportsTensorAlloc(c10::DeviceIndex) override { return true; }
  at::Tensor allocateTensor(long size, at::TensorOptions options = {}) override;
  std::shared_ptr<c10::Allocator> getMemAllocator() override;

  // Extras exposed to Python (fused ops, stats, tuning).
  std::chrono::milliseconds timeout() const { return timeout_; }
  c10::intrusive_ptr<Store> store() const { return store_; }
  ccl::CudaBackendImpl& cudaImpl(const at::Device& device);
  bool blockingWait() const { return blocking_wait_; }
  bool sameStream() const { return same_stream_; }
  uint64_t nextSeq() { return seq_.fetch_add(1); }
  void debugConsistencyCheck(const char* op, at::ScalarType dtype, uint64_t bytes);
  bool timingEnabled() const { return timing_enabled_; }

 private:
  ccl::cpu::ShmComm& shm();
  std::chrono::milliseconds opTimeout(std::chrono::milliseconds op_timeout) const;
  c10::intrusive_ptr<Work> enqueueCpu(OpType type, const char* title, std::function<void(ccl::cpu::ShmComm&)> fn,
                                      std::vector<at::Tensor> outs, std::vector<std::vector<at::Tensor>> nested,
                                      bool use_nested, uint64_t seq, size_t flight_slot);
  c10::intrusive_ptr<Work> enqueueCpuP2P(OpType type, const char* title, int peer, bool is_send,
                                         std::function<void(ccl::cpu::ShmComm&)> fn, std::vector<at::Tensor> outs,
                                         uint64_t seq, size_t flight_slot);

  c10::intrusive_ptr<Store> store_;
  std::chrono::milliseconds timeout_;
  bool blocking_wait_ = false;
  bool same_stream_ = false;
  bool timing_enabled_ = false;
  std::atomic<uint64_t> seq_{0};
  uint64_t check_seq_ = 0;  // collectives seen by debugConsistencyCheck (p2p excluded)
  std::atomic<bool> aborted_{false};
  int coalescing_depth_ = 0;
  std::vector<c10::intrusive_ptr<Work>> coalesced_works_;

  std::mutex init_mu_;
  std::unique_ptr<ccl::cpu::ShmComm> shm_;
  std::unique_ptr<ccl::TaskThread> cpu_worker_;
  std::unordered_map<int, std::unique_ptr<ccl::TaskThread>> p2p_send_workers_, p2p_recv_workers_;
  std::unique_ptr<ccl::CudaBackendImpl> cuda_;
};

}  // namespace c10d
