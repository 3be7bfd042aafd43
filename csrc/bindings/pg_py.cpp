// Backend registration and the Python face of ProcessGroupCCL.
//
// Importing the extension registers backend "ccl" with torch.distributed for devices
// ["cuda", "cpu"] and publishes torch.distributed.ProcessGroupCCL(store, rank, size, timeout)
// — the same entry points as the reference (oneccl_bindings_for_pytorch/csrc/init.cpp:117-155,
// which registers for ["xpu", "cpu"]). On top of that it exposes what the reference has no
// counterpart for: the fused collective ops on a group's CUDA communicator, statistics and the
// flight recorder.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/extension.h>

#include "bindings/common.h"
#include "bindings/fused_ops.h"
#include "cuda/CudaBackend.h"
#include "pg/Env.h"
#include "pg/ProcessGroupCCL.hpp"
#include "pg/Telemetry.h"

namespace py = pybind11;

namespace {

// Holder that drops the GIL while the backend is destroyed (its destructor joins worker
// threads that may themselves need the GIL to release tensors).
template <typename T>
class IntrusivePtrNoGil {
  c10::intrusive_ptr<T> impl_;

 public:
  IntrusivePtrNoGil() = default;
  IntrusivePtrNoGil(const IntrusivePtrNoGil&) = default;
  IntrusivePtrNoGil(IntrusivePtrNoGil&&) noexcept = default;
  IntrusivePtrNoGil& operator=(const IntrusivePtrNoGil&) = default;
  IntrusivePtrNoGil& operator=(IntrusivePtrNoGil&&) noexcept = default;
  /* implicit */ IntrusivePtrNoGil(c10::intrusive_ptr<T> impl) : impl_(std::move(impl)) {}
  explicit IntrusivePtrNoGil(T* impl) : impl_(c10::intrusive_ptr<T>::unsafe_steal_from_new(impl)) {}
  ~IntrusivePtrNoGil() {
    if (impl_) {
      if (PyGILState_Check()) {
        py::gil_scoped_release release;
        impl_.reset();
      } else {
        impl_.reset();
      }
    }
  }
  T& operator*() const noexcept { return *impl_; }
  T* operator->() const noexcept { return impl_.get(); }
  T* get() const noexcept { return impl_.get(); }
  void reset() noexcept { impl_.reset(); }
  operator bool() const noexcept { return impl_; }
};

}  // namespace

PYBIND11_DECLARE_HOLDER_TYPE(T, IntrusivePtrNoGil<T>, true)

namespace ccl_py {

using c10d::ProcessGroupCCL;

using ccl_ops::cuda_comm_of;

void bind_process_group(py::module& m) {
  ProcessGroupCCL::cclInitOnce();
  py::object dist = py::module::import("torch.distributed");
  py::object register_backend = dist.attr("Backend").attr("register_backend");
  py::object backend_base = py::module::import("torch._C._distributed_c10d").attr("Backend");

  register_backend(
      "ccl",
      py::cpp_function(&ProcessGroupCCL::createProcessGroupCCL, py::arg("store"), py::arg("rank"), py::arg("size"),
                       py::arg("timeout") = std::chrono::milliseconds(ProcessGroupCCL::OP_TIMEOUT_MILLIS),
                       py::call_guard<py::gil_scoped_release>()),
      false, std::vector<std::string>{"cuda", "cpu"});

  py::class_<ProcessGroupCCL, IntrusivePtrNoGil<ProcessGroupCCL>>(dist, "ProcessGroupCCL", backend_base)
      .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout) {
             return c10::make_intrusive<ProcessGroupCCL>(store, rank, size, timeout);
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"),
           py::arg("timeout") = std::chrono::milliseconds(10 * 1000), py::call_guard<py::gil_scoped_release>())
      .def("shutdown", &ProcessGroupCCL::shutdown, py::call_guard<py::gil_scoped_release>())
      .def("abort", &ProcessGroupCCL::abort, py::call_guard<py::gil_scoped_release>())
      .def("set_timeout", &ProcessGroupCCL::setTimeout)
      .def("error_state", [](ProcessGroupCCL& pg) { return (int)pg.getError(); })
      // ---- fused ops: run on the CURRENT stream of the tensor's device (capturable) ----
      .def("fused_allreduce_residual_rmsnorm", &ccl_ops::allreduce_residual_rmsnorm, py::arg("x"), py::arg("residual"), py::arg("weight"),
           py::arg("out"), py::arg("eps"), py::arg("tokens") = py::none(), py::arg("vocab_base") = 0, py::arg("zero_residual") = false)
      // residual += sum over ranks of x[rows, K_local] @ w[hidden, K_local]^T ; out = rmsnorm(residual) * weight  (one launch)
      .def("fused_gemm_ar_norm", &ccl_ops::gemm_ar_norm, py::arg("w_packed"), py::arg("x"), py::arg("residual"), py::arg("weight"),
           py::arg("out"), py::arg("eps"), py::arg("splitk") = 0)
      .def("fits_gemm_ar_norm", [](ProcessGroupCCL& pg, const at::Tensor& like, int rows, int hidden, int k) {
        return cuda_comm_of(pg, like).fits_gemm_ar_norm(rows, hidden, k);
      })
      // arg-max over the local logits shard + all-gather of the winners; writes the global winner ids
      .def("fused_sample_allgather", &ccl_ops::sample_allgather, py::arg("logits"), py::arg("next_tokens"), py::arg("tokens") = py::none(),
           py::arg("positions") = py::none())
      .def("fused_allreduce", &ccl_ops::all_reduce_scaled, py::arg("tensor"), py::arg("scale") = 1.0)
      // out (fp32 or input dtype) = scale * sum over ranks of this rank's piece of `inp`
      .def("fused_reduce_scatter_cast", &ccl_ops::reduce_scatter_cast, py::arg("input"), py::arg("output"), py::arg("scale") = 1.0)
      // gathers `shard` from every rank straight into the per-rank destination tensors
      .def("fused_all_gather_copy_out", &ccl_ops::all_gather_copy_out)
      // out[M/W, N] = this rank's rows of sum over ranks of a[M, K_local] @ b[N, K_local]^T
      .def("fused_gemm_rs", &ccl_ops::gemm_reduce_scatter)
      // out[M, N_local] = all_gather(a_shard)[M, K] @ b[N_local, K]^T
      .def("fused_ag_gemm", &ccl_ops::all_gather_gemm)
      .def("fused_moe_dispatch", &ccl_ops::moe_dispatch)
      .def("fused_moe_combine", &ccl_ops::moe_combine)
      // staging capacity (bytes) of the fused GEMM + collective ops: the whole M x N (gemm_rs) or M x K (ag_gemm) bf16 matrix must fit
      .def("fused_gemm_capacity_bytes", [](ProcessGroupCCL& pg, const at::Tensor& like) { return (int64_t)cuda_comm_of(pg, like).config().half_bytes; })
      // symmetric tensor of `numel` elements from the group's heap (collective in order; see ProcessGroupCCL::allocateTensor)
      .def("symm_empty", [](ProcessGroupCCL& pg, int64_t numel, at::ScalarType dtype, c10::optional<at::Device> device) {
        at::TensorOptions o = at::TensorOptions().dtype(dtype);
        if (device.has_value()) o = o.device(*device);
        return pg.allocateTensor((long)numel, o);
      }, py::arg("numel"), py::arg("dtype"), py::arg("device") = py::none())
      .def("is_symmetric", [](ProcessGroupCCL& pg, const at::Tensor& t) {
        return t.is_cuda() && cuda_comm_of(pg, t).symm_offset(t.data_ptr(), t.nbytes(), nullptr);
      })
      .def("wait_for_pending_works", &ProcessGroupCCL::waitForPendingWorks, py::call_guard<py::gil_scoped_release>())
      .def("symm_heap_info", [](ProcessGroupCCL& pg, const at::Tensor& like) {
        auto& c = cuda_comm_of(pg, like);
        py::dict d;
        d["bytes"] = c.config().heap_bytes;
        d["in_use"] = c.heap_in_use();
        d["multicast"] = c.heap_multicast();
        d["symm_min_bytes"] = c.config().symm_min_bytes;
        return d;
      })
      .def("moe_capacity", [](ProcessGroupCCL& pg, const at::Tensor& like) { return cuda_comm_of(pg, like).moe_capacity((int)like.size(-1)); })
      .def("cuda_comm_status", [](ProcessGroupCCL& pg, const at::Tensor& t) {
        auto& c = cuda_comm_of(pg, t);
        int r = 0, p = 0, ph = 0;
        int code = c.poll_status(&r, &p, &ph);
        return std::vector<int>{code, r, p, ph};
      })
      .def("cuda_comm_config", [](ProcessGroupCCL& pg, const at::Tensor& t) {
        const ccl::CommConfig& c = cuda_comm_of(pg, t).config();
        py::dict d;
        d["half_bytes"] = c.half_bytes;
        d["oneshot_max_bytes"] = c.oneshot_max_bytes;
        d["ag_push_max_bytes"] = c.ag_push_max_bytes;
        d["max_blocks"] = c.max_blocks;
        d["threads"] = c.threads;
        d["spin_timeout_ms"] = c.spin_timeout_ms;
        d["symm_mem"] = c.symm == ccl::SymmKind::kVmm ? "vmm" : "ipc";
        d["nvls"] = c.nvls;
        d["nvls_available"] = cuda_comm_of(pg, t).nvls_available();
        d["nvls_min_bytes"] = c.nvls_min_bytes;
        d["symm_min_bytes"] = c.symm_min_bytes;
        return d;
      })
      .def("set_cuda_tuning", [](ProcessGroupCCL& pg, const at::Tensor& t, const py::dict& kv) {
        // every rank of the group must apply the same values before its next collective
        ccl::CommConfig& c = cuda_comm_of(pg, t).mutable_config();
        for (auto item : kv) {
          const std::string k = py::cast<std::string>(item.first);
          const int64_t v = py::cast<int64_t>(item.second);
          TORCH_CHECK(v >= 0, "tuning values are non-negative");
          if (k == "oneshot_max_bytes") c.oneshot_max_bytes = (size_t)v;
          else if (k == "ag_push_max_bytes") c.ag_push_max_bytes = (size_t)v;
          else if (k == "max_blocks") { TORCH_CHECK(v >= 1 && v <= ccl::kMaxBlocks, "max_blocks out of range"); c.max_blocks = (int)v; }
          else if (k == "threads") { TORCH_CHECK(v >= 32 && v <= 512 && v % 32 == 0, "threads out of range"); c.threads = (int)v; }
          else if (k == "nvls_min_bytes") c.nvls_min_bytes = (size_t)v;
          else if (k == "symm_min_bytes") c.symm_min_bytes = (size_t)v;
          else if (k == "algo") { TORCH_CHECK(v >= 0 && v <= 3, "algo: 0 auto, 1 oneshot, 2 twoshot, 3 nvls"); c.algo = static_cast<ccl::Algo>(v); }
          else TORCH_CHECK(false, "unknown tuning key '", k, "'");
        }
      })
      .def("cuda_kernel_launches", [](ProcessGroupCCL& pg, const at::Tensor& t) { return cuda_comm_of(pg, t).launches(); });

  m.def("reparse_env", [] { ccl::Env::reparse(); });
  m.def("env", [] {
    const ccl::Env& e = ccl::Env::get();
    py::dict d;
    d["verbose"] = e.verbose;
    d["blocking_wait"] = e.blocking_wait;
    d["same_stream"] = e.same_stream;
    d["llm_allreduce"] = e.llm_allreduce;
    d["algo"] = e.algo;
    d["oneshot_max_bytes"] = e.oneshot_max_bytes;
    d["spin_timeout_ms"] = e.spin_timeout_ms;
    d["arena_mb"] = e.arena_mb;
    d["symm_heap_mb"] = e.symm_heap_mb;
    d["symm_min_bytes"] = e.symm_min_bytes;
    d["nvls_min_bytes"] = e.nvls_min_bytes;
    d["shm_slot_mb"] = e.shm_slot_mb;
    d["max_blocks"] = e.max_blocks;
    d["threads"] = e.threads;
    d["symm_mem"] = e.symm_mem;
    d["tune_file"] = e.tune_file;
    d["nvls"] = e.nvls;
    d["with_mpirun"] = e.with_mpirun;
    d["local_rank"] = e.local_rank;
    d["local_world_size"] = e.local_world_size;
    return d;
  });
  m.def("stats", [] {
    py::dict out;
    for (const auto& kv : ccl::Telemetry::get().stats()) {
      py::dict d;
      d["count"] = kv.second.count;
      d["bytes"] = kv.second.bytes;
      d["host_us_total"] = kv.second.host_us_total;
      d["host_us_hist"] = std::vector<uint64_t>(kv.second.host_us_hist.begin(), kv.second.host_us_hist.end());
      py::dict al;
      for (const auto& a : kv.second.algos) al[py::str(a.first)] = a.second;
      d["algos"] = al;
      out[py::str(kv.first)] = d;
    }
    return out;
  });
  m.def("reset_stats", [] { ccl::Telemetry::get().reset(); });
  m.def("flight_recorder", [] { return ccl::Telemetry::get().dump_flight(); });
  m.def("drain", [] { ccl::Watchdog::get().drain(); }, py::call_guard<py::gil_scoped_release>());
}

}  // namespace ccl_py
