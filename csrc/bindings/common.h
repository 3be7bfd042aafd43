// Shared helpers of the Python binding translation units.
#pragma once
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/extension.h>

#include "cuda/CudaComm.h"

namespace ccl_py {

int to_ccl_dtype(at::ScalarType t);
ccl::KvStore make_kv(const c10::intrusive_ptr<c10d::Store>& store);
void fill_moe_dispatch(ccl::MoeArgs& a, const at::Tensor& x, const at::Tensor& idx, at::Tensor& out_x, at::Tensor& meta,
                       at::Tensor& count, int experts_per_rank);
void fill_moe_combine(ccl::MoeArgs& a, const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count,
                      const at::Tensor& gate, at::Tensor& out);
// Argument builders of the fused tensor-parallel ops: they validate device, dtype, shape and
// contiguity (the kernels take raw pointers and would otherwise read or write out of bounds).
// `tokens` (optional): the fused op starts with a vocabulary-parallel embedding lookup; `x` is then
// this rank's shard [rows_in_shard, hidden] of the table and `vocab_base` its first global id.
ccl::FusedNormArgs make_norm_args(const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight, at::Tensor& out, double eps,
                                  const c10::optional<at::Tensor>& tokens, int64_t vocab_base, bool zero_residual);
ccl::GemmArNormArgs make_gemm_ar_norm_args(const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual,
                                           const at::Tensor& weight, at::Tensor& out, double eps, int64_t splitk);
ccl::SampleArgs make_sample_args(const at::Tensor& logits, at::Tensor& next_tokens, const c10::optional<at::Tensor>& tokens,
                                 const c10::optional<at::Tensor>& positions);
void bind_cuda_comm(py::module& m);
void bind_process_group(py::module& m);
void bind_model_ops(py::module& m);

}  // namespace ccl_py
