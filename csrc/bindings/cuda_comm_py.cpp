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

ccl::FusedNormArgs make_norm_args(const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, at::Tensor& out, double eps,
                                  const c10::optional<at::Tensor>& tokens, int64_t vocab_base, bool zero_residual) {
  TORCH_CHECK(x.is_cuda() && residual.is_cuda() && weight.is_cuda() && out.is_cuda(), "allreduce_residual_rmsnorm: CUDA tensors required");
  TORCH_CHECK(x.device() == residual.device() && x.device() == weight.device() && x.device() == out.device(),
              "allreduce_residual_rmsnorm: tensors must be on one device");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "allreduce_residual_rmsnorm: bf16 or f16 tensors required");
  TORCH_CHECK(residual.scalar_type() == x.scalar_type() && weight.scalar_type() == x.scalar_type() && out.scalar_type() == x.scalar_type(),
              "allreduce_residual_rmsnorm: x, residual, weight and out must share one dtype");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && residual.is_contiguous() && out.is_contiguous() && weight.is_contiguous(),
              "allreduce_residual_rmsnorm: contiguous [rows, hidden] tensors required");
  const int64_t hidden = x.size(1);
  TORCH_CHECK(hidden % 8 == 0 && weight.numel() == hidden, "allreduce_residual_rmsnorm: hidden must be a multiple of 8 and weight [hidden]");
  ccl::FusedNormArgs a;
  a.x = x.data_ptr();
  a.residual = residual.data_ptr();
  a.weight = weight.data_ptr();
  a.out = out.data_ptr();
  a.hidden = (int)hidden;
  a.eps = (float)eps;
  a.zero_residual = zero_residual ? 1 : 0;
  int64_t rows = x.size(0);
  if (tokens.has_value()) {
    const at::Tensor& t = *tokens;
    TORCH_CHECK(t.is_cuda() && t.device() == x.device() && t.scalar_type() == at::kLong && t.is_contiguous() && t.dim() == 1,
                "allreduce_residual_rmsnorm: tokens must be a contiguous int64 vector on the same device");
    a.gather_tokens = reinterpret_cast<const long long*>(t.data_ptr<int64_t>());
    a.gather_base = vocab_base;
    a.gather_rows = (int)x.size(0);
    rows = t.numel();
  }
  TORCH_CHECK(residual.dim() == 2 && residual.size(0) == rows && residual.size(1) == hidden && out.sizes() == residual.sizes(),
              "allreduce_residual_rmsnorm: residual and out must be [rows, hidden]");
  a.rows = (int)rows;
  return a;
}

ccl::GemmArNormArgs make_gemm_ar_norm_args(const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual,
                                           const at::Tensor& weight, at::Tensor& out, double eps, int64_t splitk) {
  TORCH_CHECK(w_packed.is_cuda() && x.is_cuda() && residual.is_cuda() && weight.is_cuda() && out.is_cuda(), "gemm_ar_norm: CUDA tensors required");
  TORCH_CHECK(x.device() == w_packed.device() && x.device() == residual.device() && x.device() == weight.device() && x.device() == out.device(),
              "gemm_ar_norm: tensors must be on one device");
  TORCH_CHECK(w_packed.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16 && residual.scalar_type() == at::kBFloat16 &&
                  weight.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "gemm_ar_norm: bf16 tensors required");
  TORCH_CHECK(w_packed.dim() == 2 && w_packed.size(1) == 64 && w_packed.is_contiguous() && w_packed.size(0) % 128 == 0,
              "gemm_ar_norm: weights must be packed with pack_weight ([*, 64])");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0, "gemm_ar_norm: x must be [rows, K] with a contiguous K and a row stride that is a multiple of 8");
  TORCH_CHECK(residual.dim() == 2 && residual.is_contiguous() && out.is_contiguous() && weight.is_contiguous() && out.sizes() == residual.sizes() &&
                  residual.size(0) == x.size(0) && weight.numel() == residual.size(1), "gemm_ar_norm: residual / out [rows, hidden], weight [hidden]");
  ccl::GemmArNormArgs a;
  a.w = w_packed.data_ptr();
  a.w_packed_rows = w_packed.size(0);
  a.x = x.data_ptr();
  a.ldx = x.stride(0);
  a.residual = residual.data_ptr();
  a.weight = weight.data_ptr();
  a.out = out.data_ptr();
  a.rows = (int)x.size(0);
  a.hidden = (int)residual.size(1);
  a.K = (int)x.size(1);
  a.eps = (float)eps;
  a.splitk = (int)splitk;
  const int64_t k_tiles = (a.K + 63) / 64;
  TORCH_CHECK(a.hidden % 128 == 0 && w_packed.size(0) >= (int64_t)a.hidden * k_tiles, "gemm_ar_norm: packed weight does not cover [hidden, K]");
  return a;
}

ccl::SampleArgs make_sample_args(const at::Tensor& logits, at::Tensor& next_tokens, const c10::optional<at::Tensor>& tokens,
                                 const c10::optional<at::Tensor>& positions) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "sample: logits must be [rows, vocab shard] fp32");
  TORCH_CHECK(next_tokens.is_cuda() && next_tokens.device() == logits.device() && next_tokens.scalar_type() == at::kLong &&
                  next_tokens.is_contiguous() && next_tokens.numel() >= logits.size(0), "sample: next_tokens must be int64 [rows]");
  ccl::SampleArgs a;
  a.logits = logits.data_ptr<float>();
  a.ld = logits.stride(0);
  a.vshard = (int)logits.size(1);
  a.rows = (int)logits.size(0);
  a.next_tokens = reinterpret_cast<long long*>(next_tokens.data_ptr<int64_t>());
  if (tokens.has_value()) {
    TORCH_CHECK(tokens->is_cuda() && tokens->device() == logits.device() && tokens->scalar_type() == at::kLong && tokens->is_contiguous() &&
                    tokens->numel() >= logits.size(0), "sample: tokens must be int64 [rows]");
    a.tokens = reinterpret_cast<long long*>(const_cast<int64_t*>(tokens->data_ptr<int64_t>()));
  }
  if (positions.has_value()) {
    TORCH_CHECK(positions->is_cuda() && positions->device() == logits.device() && positions->scalar_type() == at::kInt &&
                    positions->is_contiguous() && positions->numel() >= logits.size(0), "sample: positions must be int32 [rows]");
    a.positions = const_cast<int*>(positions->data_ptr<int>());
  }
  return a;
}

namespace {

void cu(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "ccl: ", what, " failed: ", cudaGetErrorString(e));
}

struct PyComm {
  std::shared_ptr<CudaComm> comm;   // shared with the deleters of symmetric tensors, which may outlive this object

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

  void broadcast(std::vector<at::Tensor> bufs, int root, bool nvls) {
    ForceNvls force(comm.get(), nvls);
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
                                  std::vector<at::Tensor> weights, std::vector<at::Tensor> outs, double eps,
                                  c10::optional<std::vector<at::Tensor>> tokens, std::vector<int64_t> vocab_base, bool zero_residual) {
    check_n(xs.size());
    std::vector<ccl::FusedNormArgs> args(xs.size());
    for (size_t i = 0; i < xs.size(); ++i) {
      c10::optional<at::Tensor> tok;
      if (tokens.has_value()) tok = (*tokens)[i];
      args[i] = make_norm_args(xs[i], residuals[i], weights[i], outs[i], eps, tok, vocab_base.empty() ? 0 : vocab_base[i], zero_residual);
    }
    cu(comm->allreduce_residual_rmsnorm(to_ccl_dtype(xs[0].scalar_type()), args, stream()),
       "allreduce_residual_rmsnorm");
  }

  // w[r]: packed [hidden, K_r]; x[r]: [rows, K_r]; residual[r], out[r]: [rows, hidden]
  void gemm_ar_norm(std::vector<at::Tensor> ws, std::vector<at::Tensor> xs, std::vector<at::Tensor> residuals,
                    std::vector<at::Tensor> weights, std::vector<at::Tensor> outs, double eps, int64_t splitk) {
    check_n(xs.size());
    std::vector<ccl::GemmArNormArgs> args(xs.size());
    for (size_t i = 0; i < xs.size(); ++i) args[i] = make_gemm_ar_norm_args(ws[i], xs[i], residuals[i], weights[i], outs[i], eps, splitk);
    cu(comm->gemm_ar_norm(args, stream()), "gemm_ar_norm");
  }

  void sample_allgather(std::vector<at::Tensor> logits, std::vector<at::Tensor> next_tokens,
                        c10::optional<std::vector<at::Tensor>> tokens, c10::optional<std::vector<at::Tensor>> positions) {
    check_n(logits.size());
    std::vector<ccl::SampleArgs> args(logits.size());
    for (size_t i = 0; i < logits.size(); ++i) {
      c10::optional<at::Tensor> t, p;
      if (tokens.has_value()) t = (*tokens)[i];
      if (positions.has_value()) p = (*positions)[i];
      args[i] = make_sample_args(logits[i], next_tokens[i], t, p);
    }
    cu(comm->sample_allgather(args, stream()), "sample_allgather");
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

  // Batched small-tensor collective: ins[r] / outs[r] = the list of tensors of rank r. mode 0 all_reduce, 1 reduce_scatter
  // (ins[r][t] holds world pieces), 2 all_gather (outs[r][t] holds world pieces). Returns false if the list does not fit.
  bool multi(int mode, std::vector<std::vector<at::Tensor>> ins, std::vector<std::vector<at::Tensor>> outs, int op, double scale, int has_scale) {
    check_n(ins.size());
    std::vector<ccl::MultiArgs> args(ins.size());
    const int W = comm->world();
    for (size_t i = 0; i < ins.size(); ++i) {
      ccl::MultiArgs& m = args[i];
      m.mode = mode;
      m.op = op;
      m.scale = (float)scale;
      m.has_scale = has_scale;
      TORCH_CHECK(ins[i].size() == outs[i].size() && (int)ins[i].size() <= ccl::kMaxMulti, "bad tensor lists");
      for (size_t t = 0; t < ins[i].size(); ++t) {
        TORCH_CHECK(ins[i][t].is_contiguous() && outs[i][t].is_contiguous(), "contiguous tensors required");
        m.in[m.n] = ins[i][t].data_ptr();
        m.out[m.n] = outs[i][t].data_ptr();
        m.count[m.n] = mode == ccl::kMultiAllReduce ? ins[i][t].numel()
                       : mode == ccl::kMultiReduceScatter ? ins[i][t].numel() / W
                                                           : ins[i][t].numel() * ins[i][t].element_size();
        ++m.n;
      }
    }
    const int dt = mode == ccl::kMultiAllGather ? (int)ccl::kU8 : to_ccl_dtype(ins[0][0].scalar_type());
    if (!comm->multi_fits(dt, args[0])) return false;
    cu(comm->multi(dt, args, stream()), "multi");
    return true;
  }

  // One symmetric block of `nbytes`: a uint8 tensor per played rank, all at the same heap offset. The block returns to
  // the heap when the FIRST tensor of the list is released.
  std::vector<at::Tensor> symm_empty(int64_t nbytes) {
    void* p0 = comm->symm_alloc((size_t)nbytes);
    TORCH_CHECK(p0 != nullptr, "symmetric heap exhausted");
    const size_t off = static_cast<char*>(p0) - static_cast<char*>(comm->heap_base(0));
    std::vector<at::Tensor> out;
    auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, comm->device());
    std::shared_ptr<CudaComm> c = comm;
    for (int i = 0; i < comm->nctx(); ++i) {
      void* pi = static_cast<char*>(comm->heap_base(i)) + off;
      if (i == 0) out.push_back(at::from_blob(pi, {nbytes}, [c, p0](void*) { c->symm_free(p0); }, opts));
      else out.push_back(at::from_blob(pi, {nbytes}, [c](void*) {}, opts));
    }
    return out;
  }
  int64_t heap_in_use() { return (int64_t)comm->heap_in_use(); }

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
  m.def("builtin_thresholds", [](int world, int64_t round_mb) {
    ccl::CommConfig cfg;
    if (round_mb >= 0) cfg.round_bytes = (size_t)round_mb << 20;
    ccl::resolve_builtin_thresholds(world, &cfg);
    py::dict d;
    d["symm_min_bytes"] = cfg.symm_min_bytes;
    d["nvls_min_bytes"] = cfg.nvls_min_bytes;
    d["round_bytes"] = cfg.round_bytes;
    d["nvls_round_bytes"] = cfg.nvls_round_bytes;
    d["ag_pull_round_bytes"] = cfg.ag_pull_round_bytes;
    d["ag_nvls_max_bytes"] = cfg.ag_nvls_max_bytes;
    return d;
  }, py::arg("world"), py::arg("round_mb") = (int64_t)-1);
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
            cfg.heap_bytes = 64u << 20;
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
      .def("broadcast", &PyComm::broadcast, py::arg("bufs"), py::arg("root"), py::arg("nvls") = false)
      .def("gather", &PyComm::gather)
      .def("scatter", &PyComm::scatter)
      .def("barrier", &PyComm::barrier)
      .def("allreduce_residual_rmsnorm", &PyComm::allreduce_residual_rmsnorm, py::arg("xs"), py::arg("residuals"), py::arg("weights"),
           py::arg("outs"), py::arg("eps"), py::arg("tokens") = py::none(), py::arg("vocab_base") = std::vector<int64_t>{},
           py::arg("zero_residual") = false)
      .def("gemm_ar_norm", &PyComm::gemm_ar_norm, py::arg("ws"), py::arg("xs"), py::arg("residuals"), py::arg("weights"), py::arg("outs"),
           py::arg("eps"), py::arg("splitk") = 0)
      .def("fits_gemm_ar_norm", [](PyComm& c, int rows, int hidden, int k) { return c.comm->fits_gemm_ar_norm(rows, hidden, k); })
      .def("sample_allgather", &PyComm::sample_allgather, py::arg("logits"), py::arg("next_tokens"), py::arg("tokens") = py::none(),
           py::arg("positions") = py::none())
      .def("multi", &PyComm::multi, py::arg("mode"), py::arg("ins"), py::arg("outs"), py::arg("op") = 0, py::arg("scale") = 1.0,
           py::arg("has_scale") = 0)
      .def("symm_empty", &PyComm::symm_empty)
      .def("heap_in_use", &PyComm::heap_in_use)
      .def("set_symm_min_bytes", [](PyComm& c, int64_t b) { c.comm->mutable_config().symm_min_bytes = (size_t)b; })
      .def("set_algo", [](PyComm& c, int a) { c.comm->mutable_config().algo = static_cast<ccl::Algo>(a); })
      .def("abort", [](PyComm& c) { c.comm->abort(); })
      .def("clear_abort", [](PyComm& c) { c.comm->clear_abort(); })
      .def("gemm_rs", &PyComm::gemm_rs)
      .def("ag_gemm", &PyComm::ag_gemm)
      .def("moe_dispatch", &PyComm::moe_dispatch)
      .def("moe_combine", &PyComm::moe_combine)
      .def("moe_capacity", &PyComm::moe_capacity)
      .def("status", &PyComm::status)
      .def("clear_status", [](PyComm& c) { c.comm->clear_status(); });
}

}  // namespace ccl_py
