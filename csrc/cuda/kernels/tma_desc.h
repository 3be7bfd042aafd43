// Host helper that encodes 2-D tiled TMA tensor maps (128-byte swizzle, bf16) through the
// driver entry point obtained at run time, so nothing links against libcuda directly.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace ccl {
namespace tma {

// Tensor of `rows` x `cols` bf16 elements, row stride `ld` elements, copied in boxes of
// box_rows x box_cols (box_cols * 2 bytes must be 128 for the 128-byte swizzle).
// Out-of-range parts of a box read as zero. Returns false on failure.
bool make_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t box_cols);

}  // namespace tma
}  // namespace ccl
