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

static ccl::CudaComm& cuda_comm_of(ProcessGroupCCL& pg, const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "ccl fused ops need CUDA tensors");
  return pg.cudaImpl(t.device()).comm(t.device());
}

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
      .def("fused_allreduce_residual_rmsnorm",
           [](ProcessGroupCCL& pg, const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, at::Tensor& out, double eps) {
             auto& c = cuda_comm_of(pg, x);
             c10::cuda::CUDAGuard g(x.device());
             ccl::FusedNormArgs a;
             a.x = x.data_ptr();
             a.residual = residual.data_ptr();
             a.weight = weight.data_ptr();
             a.out = out.data_ptr();
             a.rows = (int)(x.numel() / x.size(-1));
             a.hidden = (int)x.size(-1);
             a.eps = (float)eps;
             C10_CUDA_CHECK(c.allreduce_residual_rmsnorm(to_ccl_dtype(x.scalar_type()), {a}, c10::cuda::getCurrentCUDAStream()));
           })
      .def("fused_allreduce",
           [](ProcessGroupCCL& pg, at::Tensor& t, double scale) {
             auto& c = cuda_comm_of(pg, t);
             if (c.world() == 1) {
               if (scale != 1.0) t.mul_(scale);
               return;
             }
             c10::cuda::CUDAGuard g(t.device());
             ccl::CollArgs a;
             a.in = t.data_ptr();
             a.out = t.data_ptr();
             a.count = t.numel();
             if (scale != 1.0) {
               a.has_scale = 1;
               a.scale = (float)scale;
             }
             C10_CUDA_CHECK(c.allreduce(to_ccl_dtype(t.scalar_type()), {a}, c10::cuda::getCurrentCUDAStream()));
           },
           py::arg("tensor"), py::arg("scale") = 1.0)
      .def("fused_reduce_scatter_cast",
           // out (fp32 or input dtype) = scale * sum over ranks of this rank's piece of `inp`
           [](ProcessGroupCCL& pg, const at::Tensor& inp, at::Tensor& out, double scale) {
             auto& c = cuda_comm_of(pg, inp);
             c10::cuda::CUDAGuard g(inp.device());
             const int W = c.world();
             TORCH_CHECK(inp.numel() == out.numel() * W, "input must hold world pieces of the output size");
             ccl::CollArgs a;
             const int64_t n = out.numel();
             for (int p = 0; p < W; ++p) {
               a.in_piece[p] = static_cast<const char*>(inp.data_ptr()) + (size_t)p * n * inp.element_size();
               a.in_cnt[p] = n;
             }
             a.out = out.data_ptr();
             if (scale != 1.0) {
               a.has_scale = 1;
               a.scale = (float)scale;
             }
             if (W == 1) {
               out.copy_(inp.view_as(out));
               if (scale != 1.0) out.mul_(scale);
               return;
             }
             C10_CUDA_CHECK(c.reduce_scatter(to_ccl_dtype(inp.scalar_type()), to_ccl_dtype(out.scalar_type()), {a}, c10::cuda::getCurrentCUDAStream()));
           },
           py::arg("input"), py::arg("output"), py::arg("scale") = 1.0)
      .def("fused_all_gather_copy_out",
           // gathers `shard` from every rank straight into the per-rank destination tensors
           [](ProcessGroupCCL& pg, const at::Tensor& shard, std::vector<at::Tensor> outs) {
             auto& c = cuda_comm_of(pg, shard);
             c10::cuda::CUDAGuard g(shard.device());
             TORCH_CHECK((int)outs.size() == c.world(), "need one destination per rank");
             if (c.world() == 1) {
               outs[0].copy_(shard.view_as(outs[0]));
               return;
             }
             ccl::CollArgs a;
             a.in = shard.data_ptr();
             for (int p = 0; p < c.world(); ++p) {
               a.out_piece[p] = outs[p].data_ptr();
               a.out_cnt[p] = (uint64_t)outs[p].numel() * outs[p].element_size();
             }
             C10_CUDA_CHECK(c.all_gather({a}, c10::cuda::getCurrentCUDAStream()));
           })
      .def("fused_gemm_rs",
           // out[M/W, N] = this rank's rows of sum over ranks of a[M, K_local] @ b[N, K_local]^T
           [](ProcessGroupCCL& pg, const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
             auto& c = cuda_comm_of(pg, a);
             c10::cuda::CUDAGuard g(a.device());
             TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "bf16 tensors required");
             TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.is_contiguous(), "K-contiguous operands, contiguous output");
             ccl::GemmRsArgs r;
             r.a = a.data_ptr();
             r.b = b.data_ptr();
             r.out = out.data_ptr();
             r.M = a.size(0);
             r.K = a.size(1);
             r.N = b.size(0);
             r.lda = a.stride(0);
             r.ldb = b.stride(0);
             TORCH_CHECK(out.size(0) * c.world() == r.M && out.size(1) == r.N, "out must be [M/world, N]");
             C10_CUDA_CHECK(c.gemm_rs({r}, c10::cuda::getCurrentCUDAStream()));
           })
      .def("fused_ag_gemm",
           // out[M, N_local] = all_gather(a_shard)[M, K] @ b[N_local, K]^T
           [](ProcessGroupCCL& pg, const at::Tensor& a_shard, const at::Tensor& b, at::Tensor& out) {
             auto& c = cuda_comm_of(pg, a_shard);
             c10::cuda::CUDAGuard g(a_shard.device());
             TORCH_CHECK(a_shard.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "bf16 tensors required");
             TORCH_CHECK(a_shard.is_contiguous() && b.stride(1) == 1 && out.stride(1) == 1, "packed A shard, K-contiguous B");
             ccl::AgGemmArgs r;
             r.a_shard = a_shard.data_ptr();
             r.b = b.data_ptr();
             r.out = out.data_ptr();
             r.M = a_shard.size(0) * c.world();
             r.K = a_shard.size(1);
             r.N = b.size(0);
             r.lda = a_shard.stride(0);
             r.ldb = b.stride(0);
             r.ldo = out.stride(0);
             TORCH_CHECK(out.size(0) == r.M && out.size(1) == r.N, "out must be [M, N]");
             C10_CUDA_CHECK(c.ag_gemm({r}, c10::cuda::getCurrentCUDAStream()));
           })
      .def("fused_moe_dispatch",
           [](ProcessGroupCCL& pg, const at::Tensor& x, const at::Tensor& idx, at::Tensor& out_x, at::Tensor& meta,
              at::Tensor& count, int experts_per_rank) {
             auto& c = cuda_comm_of(pg, x);
             c10::cuda::CUDAGuard g(x.device());
             ccl::MoeArgs a;
             fill_moe_dispatch(a, x, idx, out_x, meta, count, experts_per_rank);
             C10_CUDA_CHECK(c.moe_dispatch({a}, c10::cuda::getCurrentCUDAStream()));
           })
      .def("fused_moe_combine",
           [](ProcessGroupCCL& pg, const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count,
              const at::Tensor& gate, at::Tensor& out) {
             auto& c = cuda_comm_of(pg, y);
             c10::cuda::CUDAGuard g(y.device());
             ccl::MoeArgs a;
             fill_moe_combine(a, y, meta, count, gate, out);
             C10_CUDA_CHECK(c.moe_combine({a}, c10::cuda::getCurrentCUDAStream()));
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
