// Dispatcher registration of the fused collective + compute ops: `torch.ops.ccl.*`.
//
// The reference registers its collectives with the dispatcher so that torch.distributed's c10d
// ops reach its backend for XPU tensors (TORCH_LIBRARY_IMPL(c10d, XPU, m),
// src/ProcessGroupCCL.cpp:86-738 of intel/torch-ccl). For CUDA tensors torch already owns the
// c10d::* CUDA keys and routes them to whatever Backend object the process group holds, i.e. to
// ProcessGroupCCL's virtuals; what needs registering here is what c10d has no op for: the fused
// ops. Each gets a schema (so that it can be traced, exported and compiled), a CUDA kernel that
// resolves the process group by NAME (the same convention as torch's functional collectives:
// `group.group_name`) and runs on the current stream, and a Meta kernel that only computes
// output shapes, so that fake-tensor tracing needs neither a GPU nor communication.
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/library.h>

#include "bindings/fused_ops.h"

namespace {

using c10d::ProcessGroupCCL;

c10::intrusive_ptr<c10d::ProcessGroup> group_of(const std::string& name) { return c10d::resolve_process_group(name); }

ProcessGroupCCL& backend_of(const std::string& name, const at::Tensor& t) {
  auto pg = group_of(name);
  auto be = pg->getBackend(t.device().type());
  auto* ccl = dynamic_cast<ProcessGroupCCL*>(be.get());
  TORCH_CHECK(ccl != nullptr, "torch.ops.ccl: process group '", name, "' does not run on the 'ccl' backend for ", t.device().type(), " tensors");
  return *ccl;
}
int64_t world_of(const std::string& name) { return group_of(name)->getSize(); }

// ---- CUDA kernels -------------------------------------------------------------------------------
at::Tensor allreduce_residual_rmsnorm_cuda(const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, double eps,
                                           const std::string& group) {
  at::Tensor out = at::empty_like(x);
  ccl_ops::allreduce_residual_rmsnorm(backend_of(group, x), x, residual, weight, out, eps, c10::nullopt, 0, false);
  return out;
}
at::Tensor gemm_ar_norm_cuda(const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight,
                             double eps, const std::string& group) {
  at::Tensor out = at::empty_like(residual);
  ccl_ops::gemm_ar_norm(backend_of(group, x), w_packed, x, residual, weight, out, eps, 0);
  return out;
}
void all_reduce_scaled_cuda(at::Tensor& t, double scale, const std::string& group) {
  ccl_ops::all_reduce_scaled(backend_of(group, t), t, scale);
}
at::Tensor reduce_scatter_cast_cuda(const at::Tensor& inp, at::ScalarType out_dtype, double scale, const std::string& group) {
  const int64_t W = world_of(group);
  TORCH_CHECK(inp.numel() % W == 0, "reduce_scatter_cast: input size must be a multiple of the world size");
  at::Tensor out = at::empty({inp.numel() / W}, inp.options().dtype(out_dtype));
  ccl_ops::reduce_scatter_cast(backend_of(group, inp), inp, out, scale);
  return out;
}
void all_gather_copy_out_cuda(const at::Tensor& shard, at::TensorList outs, const std::string& group) {
  ccl_ops::all_gather_copy_out(backend_of(group, shard), shard, outs.vec());
}
at::Tensor gemm_reduce_scatter_cuda(const at::Tensor& a, const at::Tensor& b, const std::string& group) {
  const int64_t W = world_of(group);
  at::Tensor out = at::empty({a.size(0) / W, b.size(0)}, a.options());
  ccl_ops::gemm_reduce_scatter(backend_of(group, a), a, b, out);
  return out;
}
at::Tensor all_gather_gemm_cuda(const at::Tensor& a_shard, const at::Tensor& b, const std::string& group) {
  const int64_t W = world_of(group);
  at::Tensor out = at::empty({a_shard.size(0) * W, b.size(0)}, a_shard.options());
  ccl_ops::all_gather_gemm(backend_of(group, a_shard), a_shard, b, out);
  return out;
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_dispatch_cuda(const at::Tensor& x, const at::Tensor& expert_idx,
                                                                 int64_t experts_per_rank, int64_t max_rows, const std::string& group) {
  at::Tensor out_x = at::empty({max_rows, x.size(1)}, x.options());
  at::Tensor meta = at::empty({max_rows, 3}, x.options().dtype(at::kInt));
  at::Tensor count = at::zeros({16}, x.options().dtype(at::kInt));
  ccl_ops::moe_dispatch(backend_of(group, x), x, expert_idx, out_x, meta, count, experts_per_rank);
  return {out_x, meta, count};
}
at::Tensor moe_combine_cuda(const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count, const at::Tensor& gate,
                            const std::string& group) {
  at::Tensor out = at::empty({gate.size(0), y.size(1)}, y.options());
  ccl_ops::moe_combine(backend_of(group, y), y, meta, count, gate, out);
  return out;
}

// ---- Meta kernels: shapes only --------------------------------------------------------------------
at::Tensor allreduce_residual_rmsnorm_meta(const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, double, const std::string&) {
  TORCH_CHECK(x.sizes() == residual.sizes() && weight.numel() == x.size(-1), "allreduce_residual_rmsnorm: shape mismatch");
  return at::empty_like(x);
}
at::Tensor gemm_ar_norm_meta(const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, double,
                             const std::string&) {
  TORCH_CHECK(x.dim() == 2 && residual.dim() == 2 && x.size(0) == residual.size(0) && weight.numel() == residual.size(1) &&
                  w_packed.dim() == 2 && w_packed.size(1) == 64, "gemm_ar_norm: shape mismatch");
  return at::empty_like(residual);
}
void all_reduce_scaled_meta(at::Tensor&, double, const std::string&) {}
at::Tensor reduce_scatter_cast_meta(const at::Tensor& inp, at::ScalarType out_dtype, double, const std::string& group) {
  const int64_t W = world_of(group);
  TORCH_CHECK(inp.numel() % W == 0, "reduce_scatter_cast: input size must be a multiple of the world size");
  return at::empty({inp.numel() / W}, inp.options().dtype(out_dtype));
}
void all_gather_copy_out_meta(const at::Tensor&, at::TensorList outs, const std::string& group) {
  TORCH_CHECK((int64_t)outs.size() == world_of(group), "need one destination per rank");
}
at::Tensor gemm_reduce_scatter_meta(const at::Tensor& a, const at::Tensor& b, const std::string& group) {
  const int64_t W = world_of(group);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1) && a.size(0) % W == 0, "gemm_reduce_scatter: shape mismatch");
  return at::empty({a.size(0) / W, b.size(0)}, a.options());
}
at::Tensor all_gather_gemm_meta(const at::Tensor& a_shard, const at::Tensor& b, const std::string& group) {
  TORCH_CHECK(a_shard.dim() == 2 && b.dim() == 2 && a_shard.size(1) == b.size(1), "all_gather_gemm: shape mismatch");
  return at::empty({a_shard.size(0) * world_of(group), b.size(0)}, a_shard.options());
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_dispatch_meta(const at::Tensor& x, const at::Tensor&, int64_t, int64_t max_rows,
                                                                 const std::string&) {
  return {at::empty({max_rows, x.size(1)}, x.options()), at::empty({max_rows, 3}, x.options().dtype(at::kInt)),
          at::empty({16}, x.options().dtype(at::kInt))};
}
at::Tensor moe_combine_meta(const at::Tensor& y, const at::Tensor&, const at::Tensor&, const at::Tensor& gate, const std::string&) {
  return at::empty({gate.size(0), y.size(1)}, y.options());
}

}  // namespace

TORCH_LIBRARY(ccl, m) {
  m.def("allreduce_residual_rmsnorm(Tensor x, Tensor(a!) residual, Tensor weight, float eps, str group) -> Tensor");
  m.def("gemm_ar_norm(Tensor w_packed, Tensor x, Tensor(a!) residual, Tensor weight, float eps, str group) -> Tensor");
  m.def("all_reduce_scaled(Tensor(a!) tensor, float scale, str group) -> ()");
  m.def("reduce_scatter_cast(Tensor input, ScalarType out_dtype, float scale, str group) -> Tensor");
  m.def("all_gather_copy_out(Tensor shard, Tensor(a!)[] outs, str group) -> ()");
  m.def("gemm_reduce_scatter(Tensor a, Tensor b, str group) -> Tensor");
  m.def("all_gather_gemm(Tensor a_shard, Tensor b, str group) -> Tensor");
  m.def("moe_dispatch(Tensor x, Tensor expert_idx, int experts_per_rank, int max_rows, str group) -> (Tensor, Tensor, Tensor)");
  m.def("moe_combine(Tensor y, Tensor meta, Tensor count, Tensor gate, str group) -> Tensor");
}

TORCH_LIBRARY_IMPL(ccl, CUDA, m) {
  m.impl("allreduce_residual_rmsnorm", &allreduce_residual_rmsnorm_cuda);
  m.impl("gemm_ar_norm", &gemm_ar_norm_cuda);
  m.impl("all_reduce_scaled", &all_reduce_scaled_cuda);
  m.impl("reduce_scatter_cast", &reduce_scatter_cast_cuda);
  m.impl("all_gather_copy_out", &all_gather_copy_out_cuda);
  m.impl("gemm_reduce_scatter", &gemm_reduce_scatter_cuda);
  m.impl("all_gather_gemm", &all_gather_gemm_cuda);
  m.impl("moe_dispatch", &moe_dispatch_cuda);
  m.impl("moe_combine", &moe_combine_cuda);
}

TORCH_LIBRARY_IMPL(ccl, Meta, m) {
  m.impl("allreduce_residual_rmsnorm", &allreduce_residual_rmsnorm_meta);
  m.impl("gemm_ar_norm", &gemm_ar_norm_meta);
  m.impl("all_reduce_scaled", &all_reduce_scaled_meta);
  m.impl("reduce_scatter_cast", &reduce_scatter_cast_meta);
  m.impl("all_gather_copy_out", &all_gather_copy_out_meta);
  m.impl("gemm_reduce_scatter", &gemm_reduce_scatter_meta);
  m.impl("all_gather_gemm", &all_gather_gemm_meta);
  m.impl("moe_dispatch", &moe_dispatch_meta);
  m.impl("moe_combine", &moe_combine_meta);
}
