// Host interface of the tcgen05 bf16 GEMM family (no torch dependency).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace ccl {

// Kernel attributes (cudaFuncSetAttribute) are per device. A launcher keeps one DeviceOnce per
// kernel instantiation: `pending()` is true until `done()` was called with the calling thread's
// current device, so a process that drives several GPUs configures each of them exactly once.
class DeviceOnce {
 public:
  bool pending() const {
    int dev = 0;
    cudaGetDevice(&dev);
    return (mask_.load(std::memory_order_acquire) & (1ull << (dev & 63))) == 0;
  }
  void done() {
    int dev = 0;
    cudaGetDevice(&dev);
    mask_.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }

 private:
  std::atomic<uint64_t> mask_{0};
};

// D[M, N] = A[M, K] · B[N, K]^T with bf16 operands (K contiguous) and fp32 accumulation.
// A occupies the 128-row UMMA M side, B the UMMA N side (tile width `bn`, a multiple of 16).
struct GemmDesc {
  const void* a = nullptr;  // [M, K], row stride lda elements
  const void* b = nullptr;  // [N, K], row stride ldb elements
  void* out = nullptr;      // bf16 (out_fp32 = 0) or fp32 (out_fp32 = 1)
  int64_t M = 0, N = 0, K = 0;
  int64_t lda = 0, ldb = 0, ldo = 0;
  int out_fp32 = 0;
  int trans_out = 0;   // 1: out[n*ldo + m] (swap-AB decode: weights are A, activations are B)
  int64_t dual_off = 0;  // >0: SwiGLU mode, out = silu(A[m]·B) * (A[m+dual_off]·B); M counts gate rows
  int splitk = 0;      // 0 = choose automatically
  int bn = 0;          // 0 = choose automatically from N
  // a_tiled: `a` holds the matrix pre-packed for streaming: rows padded to a multiple of 128, K to a
  // multiple of 64, stored as [rows/128][K/64][128][64] (each 128x64 tile is 16 KB contiguous), so a
  // TMA box reads one contiguous block instead of 128 strided 128-byte pieces. With dual_off > 0 the
  // second operand starts dual_off (a multiple of 128) packed rows after the first.
  int a_tiled = 0;
  int64_t a_packed_rows = 0;  // total rows of the packed [*, 64] matrix
  int no_persistent = 0;  // 1: force the one-tile-per-CTA kernel (testing)
  int* status = nullptr;  // optional device error word
};

// Launches on `stream`; returns cudaSuccess or the launch / argument error.
cudaError_t gemm_bf16_tn(const GemmDesc& d, cudaStream_t stream);

// Programmatic dependent launch for the kernels of this library (env CCL_PDL, default on): each
// kernel is launched with the programmatic-serialization attribute, triggers its successor early
// and waits for its predecessor only where it first touches data that an earlier kernel produced.
bool pdl_enabled();
// Fills `attr` for cudaLaunchKernelEx; returns the number of attributes written (0 or 1).
int pdl_launch_attr(cudaLaunchAttribute* attr);

// Number of kernels of this library launched since the last call to reset (per process).
uint64_t launch_count();
void launch_count_add(uint64_t n);
void launch_count_reset();

}  // namespace ccl
