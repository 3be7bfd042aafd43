// Python bindings of torch_ccl_b200._C.
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "bindings/common.h"
#include "cuda/kernels/gemm.h"

namespace {

// out = a · b^T on tcgen05 tensor cores. a: [M,K] bf16, b: [N,K] bf16 (rows may be strided).
// trans_out: out is [N,M]; dual_off>0: SwiGLU over stacked gate/up rows of a.
void gemm_bf16_tn(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, bool trans_out,
                  int64_t dual_off, int64_t splitk, int64_t bn, int64_t a_tiled_rows) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm_bf16_tn: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "gemm_bf16_tn: bf16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm_bf16_tn: 2-D tensors required");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1,
              "gemm_bf16_tn: innermost dimension must be contiguous");
  const bool tiled = a_tiled_rows > 0;
  TORCH_CHECK(tiled ? (a.size(1) == 64 && a.is_contiguous() && a.size(0) % 128 == 0) : (a.size(1) == b.size(1)),
              "gemm_bf16_tn: K mismatch (or malformed packed A)");
  c10::cuda::CUDAGuard guard(a.device());
  ccl::GemmDesc d;
  d.a = a.data_ptr();
  d.b = b.data_ptr();
  d.out = out.data_ptr();
  d.M = tiled ? a_tiled_rows : (dual_off > 0 ? dual_off : a.size(0));
  d.a_tiled = tiled;
  d.a_packed_rows = a.size(0);
  d.N = b.size(0);
  d.K = b.size(1);
  d.lda = a.stride(0);
  d.ldb = b.stride(0);
  d.ldo = out.stride(0);
  d.out_fp32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(d.out_fp32 || out.scalar_type() == at::kBFloat16, "gemm_bf16_tn: out must be bf16 or fp32");
  d.trans_out = trans_out;
  d.dual_off = dual_off;
  if (dual_off > 0 && !tiled) {
    TORCH_CHECK(a.size(0) >= 2 * dual_off, "gemm_bf16_tn: dual needs 2*dual_off rows");
  }
  if (trans_out) {
    TORCH_CHECK(out.size(0) == d.N && out.size(1) == d.M, "gemm_bf16_tn: out must be [N, M]");
  } else {
    TORCH_CHECK(out.size(0) == d.M && out.size(1) == d.N, "gemm_bf16_tn: out must be [M, N]");
  }
  d.splitk = (int)splitk;
  d.bn = (int)bn;
  cudaError_t e = ccl::gemm_bf16_tn(d, c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "gemm_bf16_tn launch failed: ", cudaGetErrorString(e));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_bf16_tn", &gemm_bf16_tn, py::arg("a"), py::arg("b"), py::arg("out"),
        py::arg("trans_out") = false, py::arg("dual_off") = 0, py::arg("splitk") = 0,
        py::arg("bn") = 0, py::arg("a_tiled_rows") = 0);
  ccl_py::bind_cuda_comm(m);
  ccl_py::bind_process_group(m);
  ccl_py::bind_model_ops(m);
  m.def("launch_count", &ccl::launch_count);
  m.def("launch_count_reset", &ccl::launch_count_reset);
}
