#include "pg/TensorChecks.h"

#include <c10/util/Exception.h>

#include <stdexcept>

namespace ccl {

void check_tensor(const at::Tensor& t) {
  TORCH_CHECK(t.is_sparse() || t.is_contiguous(t.suggest_memory_format()),
              "input dense tensor has to be contiguous");
  TORCH_CHECK(!t.is_sparse(), "CCL process group does not support sparse tensors");
  TORCH_CHECK(t.numel() >= 0, "input tensor numel should be non-negative");
}

void check_single_tensor(const std::vector<at::Tensor>& tensors) {
  TORCH_CHECK(tensors.size() == 1,
              "CCL process group does not support tensors count " + std::to_string(tensors.size()));
  check_tensor(tensors[0]);
}

void check_same_type(const at::Tensor& first, const std::vector<at::Tensor>& tensors) {
  for (size_t i = 0; i < tensors.size(); ++i) {
    TORCH_CHECK(tensors[i].scalar_type() == first.scalar_type(), "Tensors are not equal in data type");
    TORCH_CHECK(tensors[i].device().type() == first.device().type(),
                "Tensors are not in same device type. Expect: ", first.device().type(),
                " But got: ", tensors[i].device().type());
    check_tensor(tensors[i]);
  }
}

void check_same_type(const at::Tensor& first, const std::vector<std::vector<at::Tensor>>& tensors) {
  for (const auto& v : tensors) check_same_type(first, v);
}

void check_rank(int64_t rank, int size) {
  if (rank < 0 || rank >= size) throw std::invalid_argument("unexpected rank");
}

void check_split_sizes(const std::vector<int64_t>& split_sizes, const at::Tensor& tensor, int group_size) {
  if (split_sizes.empty()) {
    TORCH_CHECK(tensor.size(0) % group_size == 0,
                "alltoall_base: tensor's dim 0 does not divide equally across group size");
  } else {
    TORCH_CHECK(split_sizes.size() == static_cast<size_t>(group_size),
                "Number of tensor splits not equal to group size");
    int64_t sum = 0;
    for (auto s : split_sizes) sum += s;
    TORCH_CHECK(sum == tensor.size(0), "Split sizes doesn't match total dim 0 size");
  }
}

std::string reduce_op_to_string(const c10d::ReduceOp& op) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return "SUM";
    case c10d::ReduceOp::PRODUCT: return "PRODUCT";
    case c10d::ReduceOp::MIN: return "MIN";
    case c10d::ReduceOp::MAX: return "MAX";
    case c10d::ReduceOp::BAND: return "BAND";
    case c10d::ReduceOp::BOR: return "BOR";
    case c10d::ReduceOp::BXOR: return "BXOR";
    case c10d::ReduceOp::AVG: return "AVG";
    case c10d::ReduceOp::PREMUL_SUM: return "PREMUL_SUM";
    default: return "UNKNOWN";
  }
}

ReduceSpec make_reduce_spec(const c10d::ReduceOp& op, at::ScalarType dtype, int world) {
  ReduceSpec s;
  const bool is_float = at::isFloatingType(dtype);
  switch (op.op_) {
    case c10d::ReduceOp::SUM: s.kind = 0; break;
    case c10d::ReduceOp::PRODUCT: s.kind = 1; break;
    case c10d::ReduceOp::MIN: s.kind = 2; break;
    case c10d::ReduceOp::MAX: s.kind = 3; break;
    case c10d::ReduceOp::BAND:
    case c10d::ReduceOp::BOR:
    case c10d::ReduceOp::BXOR:
      TORCH_CHECK(!is_float, "Cannot use ReduceOp." + reduce_op_to_string(op) + " with non-integral dtype");
      s.kind = op.op_ == c10d::ReduceOp::BAND ? 4 : (op.op_ == c10d::ReduceOp::BOR ? 5 : 6);
      break;
    case c10d::ReduceOp::AVG:
      s.kind = 0;
      s.has_scale = true;
      s.is_avg = true;
      s.scale = is_float ? 1.0 / world : static_cast<double>(world);
      break;
    case c10d::ReduceOp::PREMUL_SUM: {
      TORCH_CHECK(is_float, "Cannot use ReduceOp.PREMUL_SUM with non-floating dtype");
      s.kind = 0;
      s.has_scale = true;
      const auto* sup = static_cast<const c10d::NCCLPreMulSumSupplement*>(op.supplement_.get());
      TORCH_CHECK(sup != nullptr, "ReduceOp.PREMUL_SUM needs a factor");
      if (sup->tensor_factor.defined()) {
        s.scale = sup->tensor_factor.cpu().to(at::kDouble).item<double>();
      } else {
        s.scale = sup->double_factor;
      }
      break;
    }
    default:
      TORCH_CHECK(false, "Cannot use ReduceOp." + reduce_op_to_string(op) + " with CCL");
  }
  if (dtype == at::kBool) {
    // bool travels as uint8: SUM/MAX behave as OR, PRODUCT/MIN as AND
    if (s.kind == 0 || s.kind == 3) s.kind = 5;
    else if (s.kind == 1 || s.kind == 2) s.kind = 4;
    s.has_scale = false;
  }
  return s;
}

bool is_flat_view_list(const std::vector<at::Tensor>& list, at::Tensor* flat) {
  if (list.empty()) return false;
  const auto& t0 = list[0];
  if (!t0.is_contiguous()) return false;
  const int64_t n = t0.numel();
  const int64_t esz = t0.element_size();
  const char* base = static_cast<const char*>(t0.data_ptr());
  for (size_t i = 0; i < list.size(); ++i) {
    const auto& t = list[i];
    if (!t.is_contiguous() || t.numel() != n || t.scalar_type() != t0.scalar_type()) return false;
    if (!t.storage().is_alias_of(t0.storage())) return false;
    if (static_cast<const char*>(t.data_ptr()) != base + (int64_t)i * n * esz) return false;
  }
  if (flat) {
    *flat = at::empty({0}, t0.options())
                .set_(t0.storage(), t0.storage_offset(), {(int64_t)list.size() * n}, {1});
  }
  return true;
}

at::Tensor new_like_flat(const std::vector<at::Tensor>& list) {
  TORCH_CHECK(!list.empty(), "Received an empty list");
  std::vector<int64_t> sizes{static_cast<int64_t>(list.size())};
  sizes.insert(sizes.end(), list[0].sizes().begin(), list[0].sizes().end());
  return at::empty(sizes, list[0].options());
}

std::string device_key(const at::Device& d) {
  return std::string(d.is_cuda() ? "cuda:" : "cpu:") + std::to_string(d.has_index() ? d.index() : 0) + ",";
}

std::string p2p_key(int a, int b) {
  const int lo = a < b ? a : b, hi = a < b ? b : a;
  return std::to_string(lo) + ":" + std::to_string(hi);
}

}  // namespace ccl
