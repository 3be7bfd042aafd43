// Functional check of the CCL_DEBUG_BOUNDS build of the staging accessors (comm.cuh): an access
// inside the arena goes through, an access one vector past its end is skipped and recorded in the
// status word. The "out of bounds" address still lies inside a larger allocation with a sentinel
// pattern, so nothing can fault even if the check were broken - the test then sees the sentinel
// overwritten instead.
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -DCCL_DEBUG_BOUNDS=1 -I../../csrc -I../../csrc/cuda/kernels -o bounds_probe bounds_probe.cu
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "cuda/kernels/comm.cuh"

#define CK(x)                                                                                   \
  do {                                                                                          \
    cudaError_t e_ = (x);                                                                       \
    if (e_ != cudaSuccess) {                                                                    \
      std::fprintf(stderr, "%s:%d: %s failed: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      return 1;                                                                                 \
    }                                                                                           \
  } while (0)

__global__ void probe_kernel(const ccl::RankCtx ctx, float* loaded) {
  __shared__ int s_failed;
  ccl::Sync sy(ctx, &s_failed, false);
  if (threadIdx.x == 0) {
    ccl::Vec<float> v;
    for (int i = 0; i < 4; ++i) v.v[i] = 1.0f + i;
    char* base = ctx.data[0];
    ccl::store_stage(base, v);                                   // first vector of the arena: fine
    ccl::store_stage(base + 2 * ctx.half_bytes - 16, v);         // last vector of the arena: fine
    ccl::store_stage(base + 2 * ctx.half_bytes, v);              // one past the end: must be skipped
    const ccl::Vec<float> r = ccl::load_stage<float>(base + 2 * ctx.half_bytes + 16);  // skipped, zeros
    for (int i = 0; i < 4; ++i) loaded[i] = r.v[i];
  }
}

int main() {
  const size_t half = 1 << 20, sentinel_bytes = 4096;
  char* buf = nullptr;
  CK(cudaMalloc(&buf, 2 * half + sentinel_bytes));
  CK(cudaMemset(buf, 0, 2 * half));
  CK(cudaMemset(buf + 2 * half, 0x5A, sentinel_bytes));
  int* status = nullptr;
  CK(cudaHostAlloc(reinterpret_cast<void**>(&status), 64, cudaHostAllocMapped));
  std::memset(status, 0, 64);
  int* dstatus = nullptr;
  CK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dstatus), status, 0));
  float* loaded = nullptr;
  CK(cudaMalloc(&loaded, 16));
  ccl::RankCtx ctx;
  std::memset(&ctx, 0, sizeof(ctx));
  ctx.data[0] = buf;
  ctx.half_bytes = half;
  ctx.status = dstatus;
  ctx.spin_ns = 1000000;
  ctx.rank = 0;
  ctx.world = 1;
  probe_kernel<<<1, 32>>>(ctx, loaded);
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  std::vector<unsigned char> tail(sentinel_bytes);
  CK(cudaMemcpy(tail.data(), buf + 2 * half, sentinel_bytes, cudaMemcpyDeviceToHost));
  float first[4], last[4], got[4];
  CK(cudaMemcpy(first, buf, 16, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(last, buf + 2 * half - 16, 16, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(got, loaded, 16, cudaMemcpyDeviceToHost));
  bool ok = true;
  for (unsigned char c : tail) ok = ok && c == 0x5A;
  for (int i = 0; i < 4; ++i) ok = ok && first[i] == 1.0f + i && last[i] == 1.0f + i && got[i] == 0.0f;
  ok = ok && status[0] == ccl::kStatusBounds && status[1] == 0 && status[3] == 1;
  std::printf("status {%d, %d, 0x%x, %d}; sentinel %s; in-bounds stores %s\n%s\n", status[0], status[1], status[2], status[3],
              tail[0] == 0x5A ? "intact" : "OVERWRITTEN", first[0] == 1.0f ? "done" : "MISSING", ok ? "PASS" : "FAIL");
  return ok ? 0 : 1;
}
