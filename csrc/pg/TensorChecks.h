// Argument validation, dtype / reduce-op maps and flattening helpers shared by the CPU and CUDA
// paths. Error messages follow intel/torch-ccl (src/utils.cpp:100-255, src/cpu/cpu_ccl.cpp) so
// that user code and tests matching on them keep working.
#pragma once
#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/Types.hpp>

#include <string>
#include <vector>

namespace ccl {

// One dense, contiguous tensor per call ("CCL process group does not support tensors count N").
void check_single_tensor(const std::vector<at::Tensor>& tensors);
void check_tensor(const at::Tensor& t);
// Same dtype and device type across a list.
void check_same_type(const at::Tensor& first, const std::vector<at::Tensor>& tensors);
void check_same_type(const at::Tensor& first, const std::vector<std::vector<at::Tensor>>& tensors);
// Root validation: throws std::invalid_argument("unexpected rank") -> ValueError in Python.
void check_rank(int64_t rank, int size);
void check_split_sizes(const std::vector<int64_t>& split_sizes, const at::Tensor& tensor, int group_size);

std::string reduce_op_to_string(const c10d::ReduceOp& op);

// Reduce op in the numbering of the kernels (ccl::ReduceKind) plus an optional scale:
// AVG = SUM with scale 1/world; PREMUL_SUM = SUM of pre-scaled inputs, applied as a post-scale
// (the factor is the same on every rank).
struct ReduceSpec {
  int kind = 0;          // kSum..kBxor
  bool has_scale = false;
  double scale = 1.0;
  bool is_avg = false;
};
ReduceSpec make_reduce_spec(const c10d::ReduceOp& op, at::ScalarType dtype, int world);

// If `list` is a sequence of equally-shaped views laid out back to back in one storage, returns
// true and the flat base tensor covering all of them.
bool is_flat_view_list(const std::vector<at::Tensor>& list, at::Tensor* flat);
at::Tensor new_like_flat(const std::vector<at::Tensor>& list);

std::string device_key(const at::Device& d);
std::string p2p_key(int a, int b);

}  // namespace ccl
