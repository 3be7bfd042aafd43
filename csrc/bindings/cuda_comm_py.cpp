// Python bindings of ccl::CudaComm for direct (non-c10d) use: the single-GPU emulated
// communicator that the kernel tests drive, and a real one-rank/one-process communicator for
// tensor-parallel model code that wants the fused ops on its own stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <sys/mman.h>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/extension.h>
#include <unistd.h>

#include "bindings/common.h"
#include "cuda/CudaComm.h"
#include "cuda/Tuner.h"

namespace ccl_py {

using ccl::CollArgs;
using ccl::CudaComm;

int to_ccl_dtype(at::ScalarType t) {
  switch (t) {
    case at::kByte: case at::kBool: return ccl::kU8;
    case at::kChar: return ccl::kI8;
    case at::kShort: return ccl::kI16;
    case at::kInt: return ccl::kI32;
    case at::kLong: return ccl::kI64;
    case at::kHalf: return ccl::kF16;
    case at::kBFloat16: return ccl::kBF16;
    case at::kFloat: return ccl::kF32;
    case at::kDouble: return ccl::kF64;
    default: TORCH_CHECK(false, "ccl: unsupported dtype ", t);
  }
}

ccl::KvStore make_kv(const c10::intrusive_ptr<c10d::Store>& store) {
  ccl::KvStore kv;
  kv.set = [store](const std::string& k, const std::vector<uint8_t>& v) { store->set(k, v); };
  kv.get = [store](const std::string& k) { return store->get(k); };
  kv.add = [store](const std::string& k, int64_t v) { return store->add(k, v); };
  return kv;
}

void fill_moe_dispatch(ccl::MoeArgs& a, const at::Tensor& x, const at::Tensor& idx, at::Tensor& out_x, at::Tensor& meta,
                       at::Tensor& count, int experts_per_rank) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: [tokens, hidden] bf16");
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous() && idx.dim() == 2 && idx.size(0) == x.size(0), "expert_idx: [tokens, topk] int32");
  TORCH_CHECK(out_x.scalar_type() == at::kBFloat16 && out_x.is_contiguous() && out_x.size(1) == x.size(1), "out_x: [rows, hidden] bf16");
  TORCH_CHECK(meta.scalar_type() == at::kInt && meta.is_contiguous() && meta.size(0) >= out_x.size(0) && meta.size(1) == 3, "meta: [rows, 3] int32");
  TORCH_CHECK(count.scalar_type() == at::kInt && count.numel() >= 9, "count: [9] int32");
  a.x = x.data_ptr();
  a.expert_idx = idx.data_ptr<int>();
  a.out_x = out_x.data_ptr();
  a.out_meta = meta.data_ptr<int>();
  a.out_count = count.data_ptr<int>();
  a.tokens = (int)x.size(0);
  a.topk = (int)idx.size(1);
  a.hidden = (int)x.size(1);
  a.experts_per_rank = experts_per_rank;
}

void fill_moe_combine(ccl::MoeArgs& a, const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count,
                      const at::Tensor& gate, at::Tensor& out) {
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.dim() == 2, "y: [rows, hidden] bf16");
  TORCH_CHECK(gate.scalar_type() == at::kFloat && gate.is_contiguous() && gate.dim() == 2, "gate: [tokens, topk] fp32");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.size(0) == gate.size(0) && out.size(1) == y.size(1), "out: [tokens, hidden] bf16");
  a.x = y.data_ptr();
  a.out_meta = const_cast<int*>(meta.data_ptr<int>());
  a.in_rows = count.data_ptr<int>();
  a.gate = gate.data_ptr<float>();
  a.out_x = out.data_ptr();
  a.tokens = (int)gate.size(0);
  a.topk = (int)gate.size(1);
  a.hidden = (int)y.size(1);
}

namespace {

void cu(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "ccl: ", what, " failed: ", cudaGetErrorString(e));
}

struct PyComm {
  std::unique_ptr<CudaComm> comm;

  cudaStream_t stream() const { return c10::cuda::getCurrentCUDAStream(comm->device()).stream(); }
  void check_n(size_t n) const {
    TORCH_CHECK((int)n == comm->nctx(), "expected ", comm->nctx(), " per-rank entries, got ", n);
  }

  std::string allreduce(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int op, double scale,
                        int has_scale, int algo) {
    check_n(ins.size());
    check_n(outs.size());
    std::vector<CollArgs> args(ins.size());
    for (size_t i = 0; i < ins.size(); ++i) {
      TORCH_CHECK(ins[i].is_contiguous() && outs[i].is_contiguous(), "contiguous tensors required");
      args[i].in = ins[i].data_ptr();
      args[i].out = outs[i].data_ptr();
      args[i].count = ins[i].numel();
      args[i].op = op;
      args[i].scale = (float)scale;
      args[i].has_scale = has_scale;
    }
    auto saved = comm->config().algo;
    comm->mutable_config().algo = static_cast<ccl::Algo>(algo);
    ccl::AlgoChoice ch{};
    cudaError_t e = comm->allreduce(to_ccl_dtype(ins[0].scalar_type()), args, stream(), &ch);
    comm->mutable_config().algo = saved;
    cu(e, "allreduce");
    const char* name = ch.algo == ccl::Algo::kOneShot ? "oneshot" : (ch.algo == ccl::Algo::kNvls ? "nvls" : "twoshot");
    return std::string(name) + ":" + std::to_string(ch.nblocks);
  }

  void reduce(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int op, int root) {
    check_n(ins.size());
    std::vector<CollArgs> args(ins.size());
    for (size_t i = 0; i < ins.size(); ++i) {
      args[i].in = ins[i].data_ptr();
      args[i].out = outs[i].data_ptr();
      args[i].count = ins[i].numel();
      args[i].op = op;
      args[i].root = root;
    }
    cu(comm->reduce(to_ccl_dtype(ins[0].scalar_type()), args, stream()), "reduce");
  }

  // ins[r]: list of `world` pieces (piece p goes to rank p); outs[r]: rank r's reduced piece
  struct ForceNvls {  // scoped override used by the tests of the switch-reduction kernels
    CudaComm* c;
    ccl::Algo saved;
    ForceNvls(CudaComm* comm, bool on) : c(comm), saved(comm->config().algo) {
      if (on) c->mutable_config().algo = ccl::Algo::kNvls;
    }
    ~ForceNvls() { c->mutable_config().algo = saved; }
  };

  void reduce_scatter(std::vector<std::vector<at::Tensor>> ins, std::vector<at::Tensor> outs, int op,
                      double scale, int has_scale, bool nvls) {
    ForceNvls force(comm.get(), nvls);
    check_n(ins.size());
    std::vector<CollArgs> args(ins.size());
    const int W = comm->world();
    for (size_t i = 0; i < ins.size(); ++i) {
      TORCH_CHECK((int)ins[i].size() == W, "need one piece per rank");
      for (int p = 0; p < W; ++p) {
        args[i].in_piece[p] = ins[i][p].data_ptr();
        args[i].in_cnt[p] = ins[i][p].numel();
      }
      args[i].out = outs[i].data_ptr();
      args[i].op = op;
      args[i].scale = (float)scale;
      args[i].has_scale = has_scale;
    }
    cu(comm->reduce_scatter(to_ccl_dtype(ins[0][0].scalar_type()), to_ccl_dtype(outs[0].scalar_type()), args, stream()),
       "reduce_scatter");
  }

  void all_gather(std::vector<at::Tensor> ins, std::vector<std::vector<at::Tensor>> outs, bool nvls) {
    ForceNvls force(comm.get(), nvls);
    check_n(ins.size());
    std::vector<CollArgs> args(ins.size());
    const int W = comm->world();
    for (size_t i = 0; i < ins.size(); ++i) {
      args[i].in = ins[i].data_ptr();
      for (int p = 0; p < W; ++p) {
        args[i].out_piece[p] = outs[i][p].data_ptr();
        args[i].out_cnt[p] = outs[i][p].numel() * outs[i][p].element_size();
      }
    }
    cu(comm->all_gather(args, stream()), "all_gather");
  }

  void all_to_all(std::vector<std::vector<at::Tensor>> ins, std::vector<std::vector<at::Tensor>> outs, bool uneven) {
    check_n(ins.size());
    std::vector<CollArgs> args(ins.size());
    const int W = comm->world();
    for (size_t i = 0; i < ins.size(); ++i) {
      for (int p = 0; p < W; ++p) {
        args[i].in_piece[p] = ins[i][p].data_ptr();
        args[i].in_cnt[p] = ins[i][p].numel() * ins[i][p].element_size();
        args[i].out_piece[p] = outs[i][p].data_ptr();
        args[i].out_cnt[p] = outs[i][p].numel() * outs[i][p].element_size();
      }
    }
    cu(comm->all_to_all(args, uneven, stream()), "all_to_all");
  }

  void broadcast(std::vector<at::Tensor> bufs, int root) {
    check_n(bufs.size());
    std::vector<CollArgs> args(bufs.size());
    for (size_t i = 0; i < bufs.size(); ++i) {
      args[i].out = bufs[i].data_ptr();
      args[i].count = bufs[i].numel() * bufs[i].element_size();
      args[i].root = root;
      args[i].mode = ccl::kBroadcast;
    }
    cu(comm->rooted(args, stream()), "broadcast");
  }
  // ins[r]: rank r's piece; outs: root's list of `world` tensors
  void gather(std::vector<at::Tensor> ins, std::vector<at::Tensor> root_outs, int root) {
    check_n(ins.size());
    std::vector<CollArgs> args(ins.size());
    const int W = comm->world();
    for (size_t i = 0; i < ins.size(); ++i) {
      args[i].in = ins[i].data_ptr();
      args[i].count = ins[i].numel() * ins[i].element_size();
      args[i].root = root;
      args[i].mode = ccl::kGather;
      const bool is_root = comm->emulated() ? ((int)i == root) : (comm->rank() == root);
      if (is_root)
        for (int p = 0; p < W; ++p) args[i].out_piece[p] = root_outs[p].data_ptr();
    }
    cu(comm->rooted(args, stream()), "gather");
  }
  void scatter(std::vector<at::Tensor> root_ins, std::vector<at::Tensor> outs, int root) {
    check_n(outs.size());
    std::vector<CollArgs> args(outs.size());
    const int W = comm->world();
    for (size_t i = 0; i < outs.size(); ++i) {
      args[i].out = outs[i].data_ptr();
      args[i].count = outs[i].numel() * outs[i].element_size();
      args[i].root = root;
      args[i].mode = ccl::kScatter;
      const bool is_root = comm->emulated() ? ((int)i == root) : (comm->rank() == root);
      if (is_root)
        for (int p = 0; p < W; ++p) args[i].in_piece[p] = root_ins[p].data_ptr();
    }
    cu(comm->rooted(args, stream()), "scatter");
  }
  void barrier() { cu(comm->barrier(stream()), "barrier"); }

  void allreduce_residual_rmsnorm(std::vector<at::Tensor> xs, std::vector<at::Tensor> residuals,
                                  std::vector<at::Tensor> weights, std::vector<at::Tensor> outs, double eps) {
    check_n(xs.size());
    std::vector<ccl::FusedNormArgs> args(xs.size());
    for (size_t i = 0; i < xs.size(); ++i) {
      TORCH_CHECK(xs[i].is_contiguous() && residuals[i].is_contiguous() && outs[i].is_contiguous(),
                  "contiguous tensors required");
      TORCH_CHECK(xs[i].dim() == 2, "x must be [rows, hidden]");
      args[i].x = xs[i].data_ptr();
      args[i].residual = residuals[i].data_ptr();
      args[i].weight = weights[i].data_ptr();
      args[i].out = outs[i].data_ptr();
      args[i].rows = (int)xs[i].size(0);
      args[i].hidden = (int)xs[i].size(1);
      args[i].eps = (float)eps;
    }
    cu(comm->allreduce_residual_rmsnorm(to_ccl_dtype(xs[0].scalar_type()), args, stream()),
       "allreduce_residual_rmsnorm");
  }

  // a[r]: [M, K_r]; b[r]: [N, K_r]; out[r]: [M/W, N]
  void gemm_rs(std::vector<at::Tensor> as, std::vector<at::Tensor> bs, std::vector<at::Tensor> outs) {
    check_n(as.size());
    std::vector<ccl::GemmRsArgs> args(as.size());
    for (size_t i = 0; i < as.size(); ++i) {
      TORCH_CHECK(as[i].scalar_type() == at::kBFloat16 && bs[i].scalar_type() == at::kBFloat16 && outs[i].scalar_type() == at::kBFloat16, "bf16 tensors required");
      TORCH_CHECK(as[i].stride(1) == 1 && bs[i].stride(1) == 1 && outs[i].is_contiguous(), "K-contiguous operands, contiguous output");
      args[i].a = as[i].data_ptr();
      args[i].b = bs[i].data_ptr();
      args[i].out = outs[i].data_ptr();
      args[i].M = as[i].size(0);
      args[i].K = as[i].size(1);
      args[i].N = bs[i].size(0);
      args[i].lda = as[i].stride(0);
      args[i].ldb = bs[i].stride(0);
      TORCH_CHECK(outs[i].size(0) * comm->world() == args[i].M && outs[i].size(1) == args[i].N, "out must be [M/world, N]");
    }
    cu(comm->gemm_rs(args, stream()), "gemm_rs");
  }
  // a_shard[r]: [M/W, K]; b[r]: [N_r, K]; out[r]: [M, N_r]
  void ag_gemm(std::vector<at::Tensor> as, std::vector<at::Tensor> bs, std::vector<at::Tensor> outs) {
    check_n(as.size());
    std::vector<ccl::AgGemmArgs> args(as.size());
    for (size_t i = 0; i < as.size(); ++i) {
      TORCH_CHECK(as[i].scalar_type() == at::kBFloat16 && bs[i].scalar_type() == at::kBFloat16 && outs[i].scalar_type() == at::kBFloat16, "bf16 tensors required");
      TORCH_CHECK(as[i].is_contiguous() && bs[i].stride(1) == 1 && outs[i].stride(1) == 1, "packed A shard, K-contiguous B");
      args[i].a_shard = as[i].data_ptr();
      args[i].b = bs[i].data_ptr();
      args[i].out = outs[i].data_ptr();
      args[i].M = as[i].size(0) * comm->world();
      args[i].K = as[i].size(1);
      args[i].N = bs[i].size(0);
      args[i].lda = as[i].stride(0);
      args[i].ldb = bs[i].stride(0);
      args[i].ldo = outs[i].stride(0);
      TORCH_CHECK(outs[i].size(0) == args[i].M && outs[i].size(1) == args[i].N, "out must be [M, N]");
    }
    cu(comm->ag_gemm(args, stream()), "ag_gemm");
  }

  // MoE dispatch: x[r] [T, H] bf16, idx[r] [T, K] int32 -> out_x[r] [cap_rows, H], meta[r] [cap_rows, 3] int32, count[r] [1+W] int32
  void moe_dispatch(std::vector<at::Tensor> xs, std::vector<at::Tensor> idx, std::vector<at::Tensor> out_x,
                    std::vector<at::Tensor> meta, std::vector<at::Tensor> count, int experts_per_rank) {
    check_n(xs.size());
    std::vector<ccl::MoeArgs> args(xs.size());
    for (size_t i = 0; i < xs.size(); ++i) fill_moe_dispatch(args[i], xs[i], idx[i], out_x[i], meta[i], count[i], experts_per_rank);
    cu(comm->moe_dispatch(args, stream()), "moe_dispatch");
  }
  // MoE combine: y[r] [rows, H] bf16 (expert outputs, dispatch order) -> out[r] [T, H]
  void moe_combine(std::vector<at::Tensor> ys, std::vector<at::Tensor> meta, std::vector<at::Tensor> count,
                   std::vector<at::Tensor> gate, std::vector<at::Tensor> outs) {
    check_n(ys.size());
    std::vector<ccl::MoeArgs> args(ys.size());
    for (size_t i = 0; i < ys.size(); ++i) fill_moe_combine(args[i], ys[i], meta[i], count[i], gate[i], outs[i]);
    cu(comm->moe_combine(args, stream()), "moe_combine");
  }
  int moe_capacity(int hidden) { return comm->moe_capacity(hidden); }

  std::vector<int> status() {
    int r = 0, p = 0, ph = 0;
    int code = comm->poll_status(&r, &p, &ph);
    return {code, r, p, ph};
  }
};

}  // namespace

// Two probes of the bootstrap layer, for tests and for checking a new machine.
//
// fd_exchange_probe: every rank creates an anonymous memory file holding its rank, the ranks
// all-gather the descriptors over UNIX sockets, and every rank reads every file back. No GPU.
bool fd_exchange_probe(const c10::intrusive_ptr<c10d::Store>& store, int rank, int world, const std::string& prefix) {
  ccl::KvStore kv = make_kv(store);
  const int fd = ::memfd_create("ccl-fdx-probe", MFD_CLOEXEC);
  TORCH_CHECK(fd >= 0, "memfd_create failed");
  const int32_t mine[2] = {0x0cc1, rank};
  TORCH_CHECK(::pwrite(fd, mine, sizeof(mine), 0) == (ssize_t)sizeof(mine), "pwrite failed");
  std::vector<int> fds = ccl::exchange_fds(kv, prefix, rank, world, fd, 30000);
  ::close(fd);
  bool ok = (int)fds.size() == world;
  for (int p = 0; p < world && ok; ++p) {
    int32_t got[2] = {0, -1};
    ok = ::pread(fds[p], got, sizeof(got), 0) == (ssize_t)sizeof(got) && got[0] == 0x0cc1 && got[1] == p;
  }
  for (int f : fds) ::close(f);
  return ok;
}

// symm_mem_probe: every rank allocates `bytes` of symmetric memory on the current device, fills
// it with a pattern of its rank, and after a store barrier reads every peer's buffer through its
// own mapping (plain copies, no kernel waits on another rank, so the ranks may share one GPU).
bool symm_mem_probe(const c10::intrusive_ptr<c10d::Store>& store, int rank, int world, const std::string& kind,
                    int64_t bytes, const std::string& prefix) {
  ccl::KvStore kv = make_kv(store);
  const int dev = (int)c10::cuda::current_device();
  ccl::SymmMem mem(ccl::parse_symm_kind(kind), rank, world, dev, (size_t)bytes, kv, prefix);
  const size_t n = (size_t)bytes / sizeof(uint32_t);
  std::vector<uint32_t> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = (uint32_t)(rank + 1) * 0x01000193u + (uint32_t)i;
  C10_CUDA_CHECK(cudaMemcpy(mem.local(), host.data(), n * sizeof(uint32_t), cudaMemcpyHostToDevice));
  C10_CUDA_CHECK(cudaDeviceSynchronize());
  ccl::barrier_kv(kv, prefix + "/probe/written", world, 30000);
  bool ok = true;
  for (int p = 0; p < world && ok; ++p) {
    C10_CUDA_CHECK(cudaMemcpy(host.data(), mem.peer(p), n * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < n && ok; ++i) ok = host[i] == (uint32_t)(p + 1) * 0x01000193u + (uint32_t)i;
  }
  // nobody unmaps while a peer still reads
  ccl::barrier_kv(kv, prefix + "/probe/read", world, 30000);
  return ok;
}

void bind_cuda_comm(py::module& m) {
  m.def("fd_exchange_probe", &fd_exchange_probe, py::arg("store"), py::arg("rank"), py::arg("world"),
        py::arg("prefix") = "ccl/probe/fdx", py::call_guard<py::gil_scoped_release>());
  m.def("symm_mem_probe", &symm_mem_probe, py::arg("store"), py::arg("rank"), py::arg("world"), py::arg("kind") = "vmm",
        py::arg("bytes") = (int64_t)(4 << 20), py::arg("prefix") = "ccl/probe/symm", py::call_guard<py::gil_scoped_release>());
  m.def("parse_tune_text", [](const std::string& text) {
    py::dict out;
    for (const auto& w : ccl::parse_tune_text(text, "<text>")) {
      py::dict d;
      for (const auto& kv : w.second) d[py::str(kv.first)] = kv.second;
      out[py::int_(w.first)] = d;
    }
    return out;
  });
  m.def("emu_missing_peer_probe", [](PyComm& c) {
    return c.comm->barrier_single_rank(0, c.stream()) == cudaSuccess;
  });
  py::class_<PyComm>(m, "CudaComm")
      .def_static(
          "emulated",
          [](int world, int64_t half_bytes, int64_t spin_ms, int max_blocks) {
            ccl::CommConfig cfg;
            cfg.half_bytes = (size_t)half_bytes;
            cfg.spin_timeout_ms = (uint64_t)spin_ms;
            cfg.max_blocks = max_blocks;
            cfg.threads = 512;
            cfg.oneshot_max_bytes = 512 << 10;
            auto p = std::make_unique<PyComm>();
            p->comm = std::make_unique<CudaComm>(world, (int)c10::cuda::current_device(), cfg);
            return p;
          },
          py::arg("world"), py::arg("half_bytes") = (int64_t)(8 << 20), py::arg("spin_ms") = 2000,
          py::arg("max_blocks") = 8)
      .def_static(
          "create",
          [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int world, int64_t half_bytes,
             int64_t spin_ms, const std::string& prefix, const std::string& symm, bool nvls) {
            ccl::CommConfig cfg;
            cfg.half_bytes = (size_t)half_bytes;
            cfg.spin_timeout_ms = (uint64_t)spin_ms;
            cfg.symm = ccl::parse_symm_kind(symm);
            cfg.nvls = nvls;
            auto p = std::make_unique<PyComm>();
            py::gil_scoped_release nogil;
            p->comm = std::make_unique<CudaComm>(rank, world, (int)c10::cuda::current_device(), cfg,
                                                 store ? make_kv(store) : ccl::KvStore{}, prefix);
            return p;
          },
          py::arg("store"), py::arg("rank"), py::arg("world"), py::arg("half_bytes") = (int64_t)(64 << 20),
          py::arg("spin_ms") = 30000, py::arg("prefix") = "ccl/direct", py::arg("symm") = "ipc", py::arg("nvls") = false)
      .def_property_readonly("nvls_available", [](PyComm& c) { return c.comm->nvls_available(); })
      .def_property_readonly("world", [](PyComm& c) { return c.comm->world(); })
      .def_property_readonly("rank", [](PyComm& c) { return c.comm->rank(); })
      .def_property_readonly("nctx", [](PyComm& c) { return c.comm->nctx(); })
      .def_property_readonly("launches", [](PyComm& c) { return c.comm->launches(); })
      .def("set_oneshot_max_bytes", [](PyComm& c, int64_t b) { c.comm->mutable_config().oneshot_max_bytes = (size_t)b; })
      .def("set_ag_push_max_bytes", [](PyComm& c, int64_t b) { c.comm->mutable_config().ag_push_max_bytes = (size_t)b; })
      .def("set_max_blocks", [](PyComm& c, int b) { c.comm->mutable_config().max_blocks = b; })
      .def("set_ablate", [](PyComm& c, int a) { c.comm->mutable_config().ablate = a; })
      .def("allreduce", &PyComm::allreduce, py::arg("ins"), py::arg("outs"), py::arg("op") = 0,
           py::arg("scale") = 1.0, py::arg("has_scale") = 0, py::arg("algo") = 0)
      .def("reduce", &PyComm::reduce)
      .def("reduce_scatter", &PyComm::reduce_scatter, py::arg("ins"), py::arg("outs"), py::arg("op") = 0,
           py::arg("scale") = 1.0, py::arg("has_scale") = 0, py::arg("nvls") = false)
      .def("all_gather", &PyComm::all_gather, py::arg("ins"), py::arg("outs"), py::arg("nvls") = false)
      .def_property_readonly("last_used_nvls", [](PyComm& c) { return c.comm->last_used_nvls(); })
      .def("all_to_all", &PyComm::all_to_all, py::arg("ins"), py::arg("outs"), py::arg("uneven") = false)
      .def("broadcast", &PyComm::broadcast)
      .def("gather", &PyComm::gather)
      .def("scatter", &PyComm::scatter)
      .def("barrier", &PyComm::barrier)
      .def("allreduce_residual_rmsnorm", &PyComm::allreduce_residual_rmsnorm)
      .def("gemm_rs", &PyComm::gemm_rs)
      .def("ag_gemm", &PyComm::ag_gemm)
      .def("moe_dispatch", &PyComm::moe_dispatch)
      .def("moe_combine", &PyComm::moe_combine)
      .def("moe_capacity", &PyComm::moe_capacity)
      .def("status", &PyComm::status)
      .def("clear_status", [](PyComm& c) { c.comm->clear_status(); });
}

}  // namespace ccl_py
