// Bandwidth of SM-driven copies between two GPUs of one process, as a function of the launch
// shape. The collective kernels move their data with loops of 16-byte loads and stores issued by
// ordinary threads; how fast such a loop drives NVLink depends on how many requests it keeps in
// flight and on how the CTAs walk the buffers. This probe measures that dependence directly, so
// that the copy loops of csrc/cuda/kernels can be shaped from numbers:
//
//   direction   push  (load local, store into the peer's memory)
//               pull  (load from the peer's memory, store local)
//               local (both buffers on the launching GPU: the HBM ceiling of the same loop)
//   traffic     uni   (GPU 0 copies alone)     bi (both GPUs run the mirrored copy at once)
//   grid        CTAs x threads
//   unroll      16-byte loads issued by a thread before its first store
//   walk        contig: CTA b owns one contiguous 1/grid of the buffer
//               tiles:  CTA b owns tiles b, b + grid, b + 2 grid, ... of threads x unroll vectors
//
// and, as the reference the kernels are compared with, cudaMemcpyPeerAsync (copy engines).
// Nothing here waits on another GPU inside a kernel: every kernel is a plain bounded copy.
//
// No counterpart in intel/torch-ccl: its hand-run probes (src/test/writeremote/simple_test.cpp,
// src/test/segfault/simple_test.cpp) check that peer stores and loads work, not how fast they are.
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o peer_bw peer_bw.cu
// Run:   ./peer_bw [megabytes per copy, default 256] [iterations, default 5] [quick: skip the shape table]
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      std::fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      std::exit(1);                                                                    \
    }                                                                                  \
  } while (0)

template <int U, bool TILES>
__global__ void copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  const size_t nt = blockDim.x;
  if (TILES) {
    const size_t tile = nt * U;
    for (size_t t0 = (size_t)blockIdx.x * tile; t0 < nvec; t0 += (size_t)gridDim.x * tile) {
      uint4 v[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t j = t0 + threadIdx.x + k * nt;
        if (j < nvec) v[k] = src[j];
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t j = t0 + threadIdx.x + k * nt;
        if (j < nvec) dst[j] = v[k];
      }
    }
  } else {
    const size_t per = (nvec + gridDim.x - 1) / gridDim.x;
    size_t j0 = (size_t)blockIdx.x * per;
    if (j0 > nvec) j0 = nvec;
    size_t j1 = j0 + per;
    if (j1 > nvec) j1 = nvec;
    for (size_t t0 = j0; t0 < j1; t0 += nt * U) {
      uint4 v[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t j = t0 + threadIdx.x + k * nt;
        if (j < j1) v[k] = src[j];
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t j = t0 + threadIdx.x + k * nt;
        if (j < j1) dst[j] = v[k];
      }
    }
  }
}

// The reduce step of a two-rank reduction: out = a (local) + b (local or peer), 32-bit lanes.
template <int U>
__global__ void add_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out, size_t nvec) {
  const size_t nt = blockDim.x, tile = nt * U;
  for (size_t t0 = (size_t)blockIdx.x * tile; t0 < nvec; t0 += (size_t)gridDim.x * tile) {
    uint4 x[U], y[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const size_t j = t0 + threadIdx.x + k * nt;
      if (j < nvec) { x[k] = a[j]; y[k] = b[j]; }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const size_t j = t0 + threadIdx.x + k * nt;
      if (j < nvec) out[j] = make_uint4(x[k].x + y[k].x, x[k].y + y[k].y, x[k].z + y[k].z, x[k].w + y[k].w);
    }
  }
}

// The same tiled copy with the load flavour of the collective kernels' staging reads as a
// parameter: 0 plain (weak) load, 1 ld.relaxed.sys, 2 ld.volatile, 3 ld.relaxed.gpu.
template <int LD>
__device__ __forceinline__ uint4 load16(const uint4* p) {
  uint4 v;
  if (LD == 1) asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else if (LD == 2) asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else if (LD == 3) asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else v = *p;
  return v;
}
template <int LD, bool TILES>
__global__ void flavour_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  constexpr int U = 4;
  const size_t nt = blockDim.x, tile = nt * U;
  size_t lo = 0, hi = nvec, step = (size_t)gridDim.x * tile, first = (size_t)blockIdx.x * tile;
  if (!TILES) {
    const size_t per = (nvec + gridDim.x - 1) / gridDim.x;
    lo = (size_t)blockIdx.x * per;
    if (lo > nvec) lo = nvec;
    hi = lo + per;
    if (hi > nvec) hi = nvec;
    first = lo;
    step = tile;
  }
  for (size_t t0 = first; t0 < hi; t0 += step) {
    uint4 v[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const size_t j = t0 + threadIdx.x + k * nt;
      if (j < hi) v[k] = load16<LD>(src + j);
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const size_t j = t0 + threadIdx.x + k * nt;
      if (j < hi) dst[j] = v[k];
    }
  }
}

using CopyFn = void (*)(const uint4*, uint4*, size_t);

template <bool TILES>
static CopyFn pick(int u) {
  switch (u) {
    case 1: return copy_kernel<1, TILES>;
    case 2: return copy_kernel<2, TILES>;
    case 4: return copy_kernel<4, TILES>;
    default: return copy_kernel<8, TILES>;
  }
}

struct Gpu {
  int dev;
  uint4 *a, *b;   // two buffers of `bytes`
  cudaStream_t st;
  cudaEvent_t e0, e1;
};

int main(int argc, char** argv) {
  const size_t mb = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 256;
  const int iters = argc > 2 ? std::atoi(argv[2]) : 5;
  const size_t bytes = mb << 20, nvec = bytes / 16;
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  if (ndev < 2) {
    std::printf("peer_bw: needs 2 GPUs, found %d: skipped\n", ndev);
    return 0;
  }
  int can01 = 0, can10 = 0;
  CK(cudaDeviceCanAccessPeer(&can01, 0, 1));
  CK(cudaDeviceCanAccessPeer(&can10, 1, 0));
  if (!can01 || !can10) {
    std::printf("peer_bw: no peer access between GPU 0 and GPU 1: skipped\n");
    return 0;
  }
  Gpu g[2];
  for (int d = 0; d < 2; ++d) {
    g[d].dev = d;
    CK(cudaSetDevice(d));
    CK(cudaDeviceEnablePeerAccess(1 - d, 0));
    CK(cudaMalloc(&g[d].a, bytes));
    CK(cudaMalloc(&g[d].b, bytes));
    CK(cudaMemset(g[d].a, d + 1, bytes));
    CK(cudaMemset(g[d].b, 0, bytes));
    CK(cudaStreamCreateWithFlags(&g[d].st, cudaStreamNonBlocking));
    CK(cudaEventCreate(&g[d].e0));
    CK(cudaEventCreate(&g[d].e1));
  }
  for (int d = 0; d < 2; ++d) {
    CK(cudaSetDevice(d));
    CK(cudaDeviceSynchronize());
  }

  // Runs `launch(d)` on GPU 0 (uni) or on both (bi), iters times back to back; returns GB/s per
  // direction from the slower GPU's event time.
  auto timed = [&](bool bi, auto launch) {
    const int nd = bi ? 2 : 1;
    for (int d = 0; d < nd; ++d) {  // warm-up
      CK(cudaSetDevice(d));
      launch(d);
    }
    for (int d = 0; d < nd; ++d) {
      CK(cudaSetDevice(d));
      CK(cudaStreamSynchronize(g[d].st));
    }
    for (int d = 0; d < nd; ++d) {
      CK(cudaSetDevice(d));
      CK(cudaEventRecord(g[d].e0, g[d].st));
      for (int i = 0; i < iters; ++i) launch(d);
      CK(cudaEventRecord(g[d].e1, g[d].st));
    }
    float worst = 0.f;
    for (int d = 0; d < nd; ++d) {
      CK(cudaSetDevice(d));
      CK(cudaEventSynchronize(g[d].e1));
      float ms = 0.f;
      CK(cudaEventElapsedTime(&ms, g[d].e0, g[d].e1));
      worst = std::max(worst, ms);
    }
    return (double)bytes * iters / (worst * 1e-3) / 1e9;
  };

  std::printf("peer_bw: %zu MB per copy, %d iterations, GB/s per direction (bi: both GPUs at once, slower one)\n", mb, iters);
  for (int bi = 0; bi < 2; ++bi) {
    const double ce = timed(bi, [&](int d) { CK(cudaMemcpyPeerAsync(g[1 - d].b, 1 - d, g[d].a, d, bytes, g[d].st)); });
    std::printf("copy engine (cudaMemcpyPeerAsync) %s: %.0f\n", bi ? "bi " : "uni", ce);
  }

  const bool quick = argc > 3;   // any third argument: skip the shape table
  const int grids[] = {74, 148, 296, 592};
  const int threads[] = {256, 512, 1024};
  const int unrolls[] = {1, 2, 4, 8};
  const char* dirs[] = {"push", "pull", "local"};
  for (int dir = 0; dir < 3 && !quick; ++dir) {
    for (int bi = 0; bi < 2; ++bi) {
      if (dir == 2 && bi) continue;
      std::printf("\n%s %s          ", dirs[dir], bi ? "bi " : "uni");
      for (int u : unrolls) std::printf("  contig u%d", u);
      for (int u : unrolls) std::printf("   tiles u%d", u);
      std::printf("\n");
      for (int G : grids) {
        for (int nt : threads) {
          std::printf("  %3d CTAs x %4d  ", G, nt);
          for (int tiles = 0; tiles < 2; ++tiles) {
            for (int u : unrolls) {
              CopyFn fn = tiles ? pick<true>(u) : pick<false>(u);
              const double bw = timed(bi, [&](int d) {
                const uint4* src = (dir == 1) ? g[1 - d].a : g[d].a;
                uint4* dst = (dir == 0) ? g[1 - d].b : g[d].b;
                fn<<<G, nt, 0, g[d].st>>>(src, dst, nvec);
              });
              std::printf("  %9.0f", bw);
            }
          }
          std::printf("\n");
        }
      }
    }
  }

  // Load flavour and residency, at the shapes the collective kernels use (512 threads, unroll 4).
  // "1/SM": 120 KB of dynamic shared memory per CTA, so that one CTA is resident per SM, as for a
  // kernel with 128 registers per thread.
  {
    CopyFn fl[4][2] = {{flavour_kernel<0, false>, flavour_kernel<0, true>}, {flavour_kernel<1, false>, flavour_kernel<1, true>},
                       {flavour_kernel<2, false>, flavour_kernel<2, true>}, {flavour_kernel<3, false>, flavour_kernel<3, true>}};
    const char* fname[4] = {"plain", "relaxed.sys", "volatile", "relaxed.gpu"};
    for (int d = 0; d < 2; ++d) {
      CK(cudaSetDevice(d));
      for (auto& row : fl)
        for (auto f : row) CK(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 << 10));
    }
    std::printf("\nload flavour x residency (512 threads, unroll 4), GB/s per direction\n");
    std::printf("  flavour      CTAs  walk    resid   push uni  push bi  pull uni  pull bi  local\n");
    for (int f = 0; f < 4; ++f)
      for (int G : {148, 256})
        for (int tiles = 0; tiles < 2; ++tiles)
          for (int one = 0; one < 2; ++one) {
            if (one && tiles) continue;
            const size_t smem = one ? (120 << 10) : 0;
            std::printf("  %-11s  %4d  %-6s  %-5s", fname[f], G, tiles ? "tiles" : "contig", one ? "1/SM" : "free");
            for (int dir = 0; dir < 3; ++dir)
              for (int bi = 0; bi < 2; ++bi) {
                if (dir == 2 && bi) continue;
                const double bw = timed(bi, [&](int d) {
                  const uint4* src = (dir == 1) ? g[1 - d].a : g[d].a;
                  uint4* dst = (dir == 0) ? g[1 - d].b : g[d].b;
                  fl[f][tiles]<<<G, 512, smem, g[d].st>>>(src, dst, nvec);
                });
                std::printf("  %8.0f", bw);
              }
            std::printf("\n");
          }
  }

  // out = a + b with b in the peer's memory (the reduce step of a two-rank reduction done as a
  // remote read) against the same with b local.
  std::printf("\nadd (out = a + b, tiles u4, 296 x 512): ");
  for (int remote = 0; remote < 2; ++remote) {
    const double bw = timed(true, [&](int d) {
      add_kernel<4><<<296, 512, 0, g[d].st>>>(g[d].a, remote ? g[1 - d].a : g[d].b, g[d].b, nvec);
    });
    std::printf("%s b %.0f GB/s of output  ", remote ? "peer" : "local", bw);
  }
  std::printf("\n");
  CK(cudaGetLastError());
  for (int d = 0; d < 2; ++d) {
    CK(cudaSetDevice(d));
    CK(cudaDeviceSynchronize());
    CK(cudaFree(g[d].a));
    CK(cudaFree(g[d].b));
  }
  std::printf("peer_bw: done\n");
  return 0;
}
