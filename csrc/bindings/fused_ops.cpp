#include "bindings/fused_ops.h"

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "bindings/common.h"
#include "cuda/CudaBackend.h"

namespace ccl_ops {

using ccl_py::to_ccl_dtype;

ccl::CudaComm& cuda_comm_of(ProcessGroupCCL& pg, const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "ccl fused ops need CUDA tensors");
  return pg.cudaImpl(t.device()).comm(t.device());
}

namespace {
void same_device(const at::Tensor& a, const at::Tensor& b, const char* what) {
  TORCH_CHECK(b.is_cuda() && a.device() == b.device(), what, ": all tensors must be on one CUDA device");
}
}  // namespace

void allreduce_residual_rmsnorm(ProcessGroupCCL& pg, const at::Tensor& x, at::Tensor& residual, const at::Tensor& weight,
                                at::Tensor& out, double eps, const c10::optional<at::Tensor>& tokens, int64_t vocab_base,
                                bool zero_residual) {
  auto& c = cuda_comm_of(pg, x);
  c10::cuda::CUDAGuard g(x.device());
  ccl::FusedNormArgs a = ccl_py::make_norm_args(x, residual, weight, out, eps, tokens, vocab_base, zero_residual);
  C10_CUDA_CHECK(c.allreduce_residual_rmsnorm(to_ccl_dtype(x.scalar_type()), {a}, c10::cuda::getCurrentCUDAStream()));
}

void gemm_ar_norm(ProcessGroupCCL& pg, const at::Tensor& w_packed, const at::Tensor& x, at::Tensor& residual,
                  const at::Tensor& weight, at::Tensor& out, double eps, int64_t splitk) {
  auto& c = cuda_comm_of(pg, x);
  c10::cuda::CUDAGuard g(x.device());
  ccl::GemmArNormArgs a = ccl_py::make_gemm_ar_norm_args(w_packed, x, residual, weight, out, eps, splitk);
  TORCH_CHECK(c.fits_gemm_ar_norm(a.rows, a.hidden, a.K), "gemm_ar_norm: shape [", a.rows, " x ", a.hidden, ", K ", a.K,
              "] does not fit the fused kernel (rows <= ", ccl::gemm_ar_norm_max_rows(a.hidden), "); run the GEMM and allreduce_residual_rmsnorm separately");
  C10_CUDA_CHECK(c.gemm_ar_norm({a}, c10::cuda::getCurrentCUDAStream()));
}

void sample_allgather(ProcessGroupCCL& pg, const at::Tensor& logits, at::Tensor& next_tokens,
                      const c10::optional<at::Tensor>& tokens, const c10::optional<at::Tensor>& positions) {
  auto& c = cuda_comm_of(pg, logits);
  c10::cuda::CUDAGuard g(logits.device());
  ccl::SampleArgs a = ccl_py::make_sample_args(logits, next_tokens, tokens, positions);
  C10_CUDA_CHECK(c.sample_allgather({a}, c10::cuda::getCurrentCUDAStream()));
}

void all_reduce_scaled(ProcessGroupCCL& pg, at::Tensor& t, double scale) {
  auto& c = cuda_comm_of(pg, t);
  TORCH_CHECK(t.is_contiguous(), "all_reduce_scaled: contiguous tensor required");
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
}

void reduce_scatter_cast(ProcessGroupCCL& pg, const at::Tensor& inp, at::Tensor& out, double scale) {
  auto& c = cuda_comm_of(pg, inp);
  same_device(inp, out, "reduce_scatter_cast");
  TORCH_CHECK(inp.is_contiguous() && out.is_contiguous(), "reduce_scatter_cast: contiguous tensors required");
  TORCH_CHECK(out.scalar_type() == inp.scalar_type() || out.scalar_type() == at::kFloat,
              "reduce_scatter_cast: output dtype must be the input dtype or fp32");
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
}

void all_gather_copy_out(ProcessGroupCCL& pg, const at::Tensor& shard, std::vector<at::Tensor> outs) {
  auto& c = cuda_comm_of(pg, shard);
  c10::cuda::CUDAGuard g(shard.device());
  TORCH_CHECK((int)outs.size() == c.world(), "need one destination per rank");
  TORCH_CHECK(shard.is_contiguous(), "all_gather_copy_out: contiguous shard required");
  for (auto& o : outs) {
    same_device(shard, o, "all_gather_copy_out");
    TORCH_CHECK(o.is_contiguous() && o.scalar_type() == shard.scalar_type(), "all_gather_copy_out: contiguous destinations of the shard's dtype required");
  }
  TORCH_CHECK(outs[c.rank()].numel() == shard.numel(), "all_gather_copy_out: the own destination must have the shard's size");
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
}

void gemm_reduce_scatter(ProcessGroupCCL& pg, const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
  auto& c = cuda_comm_of(pg, a);
  same_device(a, b, "gemm_reduce_scatter");
  same_device(a, out, "gemm_reduce_scatter");
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "bf16 tensors required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.is_contiguous(), "K-contiguous operands, contiguous output");
  TORCH_CHECK(a.size(1) == b.size(1), "gemm_reduce_scatter: K mismatch");
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
}

void all_gather_gemm(ProcessGroupCCL& pg, const at::Tensor& a_shard, const at::Tensor& b, at::Tensor& out) {
  auto& c = cuda_comm_of(pg, a_shard);
  same_device(a_shard, b, "all_gather_gemm");
  same_device(a_shard, out, "all_gather_gemm");
  c10::cuda::CUDAGuard g(a_shard.device());
  TORCH_CHECK(a_shard.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "bf16 tensors required");
  TORCH_CHECK(a_shard.dim() == 2 && b.dim() == 2 && a_shard.is_contiguous() && b.stride(1) == 1 && out.stride(1) == 1, "packed A shard, K-contiguous B");
  TORCH_CHECK(a_shard.size(1) == b.size(1), "all_gather_gemm: K mismatch");
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
}

void moe_dispatch(ProcessGroupCCL& pg, const at::Tensor& x, const at::Tensor& idx, at::Tensor& out_x, at::Tensor& meta,
                  at::Tensor& count, int64_t experts_per_rank) {
  auto& c = cuda_comm_of(pg, x);
  c10::cuda::CUDAGuard g(x.device());
  ccl::MoeArgs a;
  ccl_py::fill_moe_dispatch(a, x, idx, out_x, meta, count, (int)experts_per_rank);
  C10_CUDA_CHECK(c.moe_dispatch({a}, c10::cuda::getCurrentCUDAStream()));
}

void moe_combine(ProcessGroupCCL& pg, const at::Tensor& y, const at::Tensor& meta, const at::Tensor& count,
                 const at::Tensor& gate, at::Tensor& out) {
  auto& c = cuda_comm_of(pg, y);
  c10::cuda::CUDAGuard g(y.device());
  ccl::MoeArgs a;
  ccl_py::fill_moe_combine(a, y, meta, count, gate, out);
  C10_CUDA_CHECK(c.moe_combine({a}, c10::cuda::getCurrentCUDAStream()));
}

}  // namespace ccl_ops
