// The fused collective + compute ops of a ProcessGroupCCL's CUDA communicator as free functions.
// They run on the CURRENT stream of the tensor's device (so they can be captured in a CUDA graph).
// Two faces share them: the pybind methods of ProcessGroupCCL (pg_py.cpp) and the dispatcher
// registration `torch.ops.ccl.*` (torch_library.cpp).
#pragma once
#include <torch/extension.h>

#include "cuda/CudaComm.h"
#include "pg/ProcessGroupCCL.hpp"

namespace ccl_ops {

using c10d::ProcessGroupCCL;

void allreduce_residual_rmsnorm(ProcessGroupCCL& pg, const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight,
                                at::Tensor& out, double eps, const c10::optional<at::Tensor>& tokens, int64_t vocab_base,
                                bool zero_residual);
void gemm_ar_norm(ProcessGroupCCL& pg, const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual,
                  const at::Tensor& weight, at::Tensor& out, double eps, int64_t splitk);
void sample_allgather(ProcessGroupCCL& pg, const at::Tensor& logits, at::Tensor& next_tokens,
                      const c10::optional<at::Tensor>& tokens, const c10::optional<at::Tensor>& positions);
void all_reduce_scaled(ProcessGroupCCL& pg, at::Tensor& t, double scale);
void reduce_scatter_cast(ProcessGroupCCL& pg, const at::Tensor& inp, at::Tensor& out, double scale);
void all_gather_copy_out(ProcessGroupCCL& pg, const at::Tensor& shard, std::vector<at::Tensor> outs);
void gemm_reduce_scatter(ProcessGroupCCL& pg, const at::Tensor& a, const at::Tensor& b, at::Tensor& out);
void all_gather_gemm(ProcessGroupCCL& pg, const at::Tensor& a_shard, const at::Tensor& b, at::Tensor& out);
void moe_dispatch(ProcessGroupCCL& pg, const at::Tensor& x, const at::Tensor& idx, at::Tensor& out_x, at::Tensor& meta,
                  at::Tensor& count, int64_t experts_per_rank);
void moe_combine(ProcessGroupCCL& pg, const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count,
                 const at::Tensor& gate, at::Tensor& out);

// The CUDA communicator behind `t`'s device (created lazily, collective over the group).
ccl::CudaComm& cuda_comm_of(ProcessGroupCCL& pg, const at::Tensor& t);

}  // namespace ccl_ops
