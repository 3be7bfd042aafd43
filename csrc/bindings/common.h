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
void bind_cuda_comm(py::module& m);
void bind_process_group(py::module& m);
void bind_model_ops(py::module& m);

}  // namespace ccl_py
