#include "tma_desc.h"

#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace ccl {
namespace tma {

namespace {

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

struct Key {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  bool operator==(const Key& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.ld + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= (uint64_t(k.box_rows) << 32 | k.box_cols) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    return (size_t)h;
  }
};

std::mutex g_mu;
std::unordered_map<Key, CUtensorMap, KeyHash> g_cache;

}  // namespace

bool make_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t box_cols) {
  Key key{base, rows, cols, ld, box_rows, box_cols};
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
      std::memcpy(out, &it->second, sizeof(CUtensorMap));
      return true;
    }
  }
  auto fn = encode_fn();
  if (!fn) return false;
  if (box_cols * 2 != 128 || box_rows > 256 || (ld * 2) % 16 != 0) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(g_mu);
  if (g_cache.size() > 8192) g_cache.clear();
  g_cache.emplace(key, *out);
  return true;
}

}  // namespace tma
}  // namespace ccl
