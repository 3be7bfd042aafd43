// Python bindings of the single-GPU compute kernels used by the model code (decode attention).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "bindings/common.h"
#include "cuda/kernels/decode_attention.h"
#include "cuda/kernels/gemm.h"

namespace ccl_py {

void bind_model_ops(py::module& m) {
  m.def("decode_attention_scratch_bytes", &ccl::decode_attention_scratch_bytes);
  m.def("decode_attention_default_splits", &ccl::decode_attention_default_splits);
  m.def(
      "decode_attention",
      [](const at::Tensor& qkv, at::Tensor& k_cache, at::Tensor& v_cache, const at::Tensor& positions,
         const at::Tensor& cos, const at::Tensor& sin, at::Tensor& out, at::Tensor& scratch, at::Tensor& counters,
         int64_t n_heads, int64_t n_kv_heads, int64_t nsplit) {
        TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1, "qkv: [batch, (h+2kv)*d] bf16");
        TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.scalar_type() == at::kBFloat16, "caches: [batch, kv_heads, max_seq, d] bf16");
        TORCH_CHECK(positions.scalar_type() == at::kInt && positions.is_contiguous(), "positions: int32");
        TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous(), "cos/sin: fp32");
        TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.stride(1) == 1, "out: bf16");
        const int batch = (int)qkv.size(0);
        const int hd = (int)k_cache.size(3);
        TORCH_CHECK(k_cache.size(0) >= batch && k_cache.size(1) == n_kv_heads, "cache shape mismatch");
        TORCH_CHECK(qkv.size(1) >= (n_heads + 2 * n_kv_heads) * hd, "qkv row too short");
        TORCH_CHECK(cos.size(0) >= k_cache.size(2) && cos.size(1) == hd / 2, "cos/sin: [max_seq, d/2]");
        c10::cuda::CUDAGuard g(qkv.device());
        ccl::DecodeAttnParams p;
        p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr());
        p.qkv_stride = qkv.stride(0);
        p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache.data_ptr());
        p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache.data_ptr());
        p.positions = positions.data_ptr<int>();
        p.cos = cos.data_ptr<float>();
        p.sin = sin.data_ptr<float>();
        p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        p.out_stride = out.stride(0);
        p.scratch = nsplit > 1 ? scratch.data_ptr<float>() : nullptr;
        p.counters = nsplit > 1 ? reinterpret_cast<unsigned int*>(counters.data_ptr<int>()) : nullptr;
        if (nsplit > 1) {
          TORCH_CHECK((size_t)scratch.numel() * 4 >= ccl::decode_attention_scratch_bytes(batch, (int)n_heads, (int)nsplit), "scratch too small");
          TORCH_CHECK(counters.numel() >= batch * n_heads, "counters too small");
        }
        p.n_heads = (int)n_heads;
        p.n_kv_heads = (int)n_kv_heads;
        p.head_dim = hd;
        p.max_seq = (int)k_cache.size(2);
        p.scale = 1.0f / std::sqrt((float)hd);
        cudaError_t e = ccl::decode_attention(p, batch, (int)nsplit, c10::cuda::getCurrentCUDAStream());
        TORCH_CHECK(e == cudaSuccess, "decode_attention launch failed: ", cudaGetErrorString(e));
        ccl::launch_count_add(1);
      },
      py::arg("qkv"), py::arg("k_cache"), py::arg("v_cache"), py::arg("positions"), py::arg("cos"), py::arg("sin"),
      py::arg("out"), py::arg("scratch"), py::arg("counters"), py::arg("n_heads"), py::arg("n_kv_heads"), py::arg("nsplit"));
}

}  // namespace ccl_py
