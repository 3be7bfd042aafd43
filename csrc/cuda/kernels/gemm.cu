// Host launcher of the tcgen05 bf16 GEMM: builds (and caches) the TMA tensor maps, picks tile
// width / pipeline depth / split-K cluster size, and launches the kernel from gemm_tcgen05.cuh.
#include "gemm.h"
#include "gemm_tcgen05.cuh"
#include "tma_desc.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>

namespace ccl {

namespace {
std::atomic<uint64_t> g_launches{0};
}
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("CCL_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}
int pdl_launch_attr(cudaLaunchAttribute* attr) {
  if (!pdl_enabled()) return 0;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

uint64_t launch_count() { return g_launches.load(); }
void launch_count_add(uint64_t n) { g_launches.fetch_add(n); }
void launch_count_reset() { g_launches.store(0); }

namespace gemm {

template <int BN, bool DUAL, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const Params p) {
  const int m0 = blockIdx.x * kBM;
  gemm_tile_body<BN, DUAL>(&tma_a, &tma_b, p, StoreEpilogue<OutT>{}, TileCoord{m0, m0, (int)blockIdx.y * BN});
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_persistent_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                           const Params p) {
  gemm_persistent_body<BN>(&tma_a, &tma_b, p, StoreEpilogue<OutT>{});
}

// Compute-bound shapes: persistent CTAs, double-buffered TMEM accumulators.
template <int BN, typename OutT>
cudaError_t launch_persistent(const GemmDesc& d, cudaStream_t stream) {
  const int m_tiles = (int)((d.M + kBM - 1) / kBM);
  const int n_tiles = (int)((d.N + BN - 1) / BN);
  constexpr size_t kSmemMax = 200 * 1024;
  int stages = kMaxStages;
  while (stages > 2 && persistent_smem_bytes<BN>(stages) > kSmemMax) --stages;
  const size_t smem = persistent_smem_bytes<BN>(stages);
  CUtensorMap ta, tb;
  if (!tma::make_2d_bf16(&ta, d.a, (uint64_t)d.M, (uint64_t)d.K, (uint64_t)d.lda, kBM, kBK)) return cudaErrorInvalidValue;
  if (!tma::make_2d_bf16(&tb, d.b, (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.ldb, BN, kBK)) return cudaErrorInvalidValue;
  Params p{};
  p.M = (int)d.M;
  p.N = (int)d.N;
  p.K = (int)d.K;
  p.out = d.out;
  p.ldo = d.ldo;
  p.stages = stages;
  p.splitk = 1;
  p.status = d.status;
  auto kern = gemm_persistent_kernel<BN, OutT>;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax + 2048);
    if (e != cudaSuccess) return e;
    configured.done();
  }
  int sms = 148;
  const int total = m_tiles * n_tiles;
  const int grid = total < sms ? total : sms;
  kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches.fetch_add(1);
  return e;
}

// Pipeline depth for a given split: narrow (decode) tiles are memory-bound, so when one CTA per SM
// does not cover the grid the pipeline shrinks until two CTAs fit on an SM.
template <int BN, bool DUAL>
int stages_for(int64_t ctas, int k_iters, int splitk) {
  size_t budget = 200 * 1024;
  if (BN <= 32 && ctas > 148) budget = 104 * 1024;  // measured: 48/64/80 KB budgets were 0.2-6 % slower end to end
  int stages = kMaxStages;
  while (stages > 2 && smem_bytes<BN, DUAL>(stages, splitk) > budget) --stages;
  const int per = (k_iters + splitk - 1) / splitk;
  if (stages > per && per >= 2) stages = per;
  return stages;
}

template <int BN, bool DUAL, typename OutT>
cudaError_t launch(const GemmDesc& d, int splitk, cudaStream_t stream) {
  const int m_tiles = (int)((d.M + kBM - 1) / kBM);
  const int n_tiles = (int)((d.N + BN - 1) / BN);
  const int k_iters = (int)((d.K + kBK - 1) / kBK);

  constexpr size_t kSmemMax = 200 * 1024;
  auto kern = gemm_kernel<BN, DUAL, OutT>;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax + 2048);
    if (e != cudaSuccess) return e;
    // the kernel keeps nothing in L1: give shared memory the whole array so that two CTAs fit
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    // split-K over 16 CTAs is one step beyond the portable cluster size
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
    configured.done();
  }
  // split-K: bounded by the largest cluster and by the amount of K work per CTA
  if (splitk > 16) splitk = 16;
  while (splitk > 1 && k_iters / splitk < 2) --splitk;
  if (splitk > 8 && splitk < 16) splitk = 8;   // between the portable limit and 16: stay portable
  if (splitk < 1) splitk = 1;
  const int stages = stages_for<BN, DUAL>((int64_t)m_tiles * n_tiles * splitk, k_iters, splitk);
  const size_t smem = smem_bytes<BN, DUAL>(stages, splitk);

  CUtensorMap ta, tb;
  const int64_t a_rows = DUAL ? (d.dual_off + d.M) : d.M;
  if (d.a_tiled) {
    if (d.dual_off % kBM != 0) return cudaErrorInvalidValue;
    if (!tma::make_2d_bf16(&ta, d.a, (uint64_t)d.a_packed_rows, (uint64_t)kBK, (uint64_t)kBK, kBM, kBK))
      return cudaErrorInvalidValue;
  } else if (!tma::make_2d_bf16(&ta, d.a, (uint64_t)a_rows, (uint64_t)d.K, (uint64_t)d.lda, kBM, kBK)) {
    return cudaErrorInvalidValue;
  }
  if (!tma::make_2d_bf16(&tb, d.b, (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.ldb, BN, kBK))
    return cudaErrorInvalidValue;

  Params p;
  p.M = (int)d.M;
  p.N = (int)d.N;
  p.K = (int)d.K;
  p.out = d.out;
  p.ldo = d.ldo;
  p.trans_out = d.trans_out;
  p.dual_off = (int)d.dual_off;
  p.stages = stages;
  p.splitk = splitk;
  p.status = d.status;
  p.acquire_a = 0;
  p.a_tiled = d.a_tiled;
  p.a_static = d.a_tiled;  // packed operands are weights: nothing on the stream produces them
  p.a_packed = d.a_tiled ? d.a : nullptr;
  p.k_tiles = k_iters;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(m_tiles, n_tiles, splitk);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splitk;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_launch_attr(&attr[1]);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
  if (e == cudaSuccess) g_launches.fetch_add(1);
  return e;
}

template <int BN>
cudaError_t dispatch_bn(const GemmDesc& d, int splitk, cudaStream_t s) {
  if (d.dual_off > 0) {
    if constexpr (BN <= 128) {
      return d.out_fp32 ? launch<BN, true, float>(d, splitk, s)
                        : launch<BN, true, __nv_bfloat16>(d, splitk, s);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  return d.out_fp32 ? launch<BN, false, float>(d, splitk, s)
                    : launch<BN, false, __nv_bfloat16>(d, splitk, s);
}

}  // namespace gemm

cudaError_t gemm_bf16_tn(const GemmDesc& d, cudaStream_t stream) {
  if (!d.a || !d.b || !d.out || d.M <= 0 || d.N <= 0 || d.K <= 0) return cudaErrorInvalidValue;
  if ((!d.a_tiled && (d.lda % 8)) || (d.ldb % 8)) return cudaErrorInvalidValue;  // TMA strides: 16-byte multiples
  if ((reinterpret_cast<uintptr_t>(d.a) & 15) || (reinterpret_cast<uintptr_t>(d.b) & 15))
    return cudaErrorInvalidValue;
  int bn = d.bn;
  if (bn == 0) {
    if (d.N <= 16) bn = 16;
    else if (d.N <= 32) bn = 32;
    else if (d.N <= 64) bn = 64;
    else if (d.N <= 128 || d.dual_off > 0) bn = 128;
    else bn = 256;
  }
  int splitk = d.splitk;
  if (splitk == 0) {
    const int64_t tiles = ((d.M + 127) / 128) * ((d.N + bn - 1) / bn);
    const int64_t k_iters = (d.K + 63) / 64;
    splitk = 1;
    if (bn <= 32) {
      // memory-bound: the best split measured on B200 is the largest one that keeps the grid at
      // no more than ~264 CTAs (just under two per SM, leaving room for cluster placement inside
      // a GPC): 96 tiles -> 2, 86 SwiGLU tiles -> 3, 32 tiles -> 8, 250 tiles -> 1; one more step
      // (e.g. 96 tiles x 3 = 288 CTAs) no longer fits one wave and costs 40 %. At least 4 K-steps
      // stay in every CTA.
      splitk = (int)(264 / tiles);
      // few tiles (a tensor-parallel shard of a projection): clusters of 16 keep more SMs streaming weights
      // (measured at the shapes one rank of eight sees, batch 16: qkv 12 tiles 7.5 -> 6.9 us with 16; the SwiGLU
      // pair, whose CTAs stream two weight tiles per step, 10.9 -> 11.0 us, so it stays at 8)
      if (splitk > 8) splitk = (splitk >= 16 && d.dual_off == 0) ? 16 : 8;
      while (splitk > 1 && k_iters / splitk < 4) splitk = splitk == 16 ? 8 : splitk - 1;
      if (splitk < 1) splitk = 1;
    } else if (bn <= 64 && tiles < 148) {
      splitk = (int)(148 / tiles);
      if (splitk > 4) splitk = 4;
      if (splitk < 1) splitk = 1;
    }
  }
  // large row-major problems without split-K: the persistent kernel
  if (!d.a_tiled && !d.trans_out && d.dual_off == 0 && splitk == 1 && (bn == 128 || bn == 256) && !d.no_persistent &&
      ((d.M + 127) / 128) * ((d.N + bn - 1) / bn) >= 148) {
    if (bn == 256)
      return d.out_fp32 ? gemm::launch_persistent<256, float>(d, stream) : gemm::launch_persistent<256, __nv_bfloat16>(d, stream);
    return d.out_fp32 ? gemm::launch_persistent<128, float>(d, stream) : gemm::launch_persistent<128, __nv_bfloat16>(d, stream);
  }
  switch (bn) {
    case 16: return gemm::dispatch_bn<16>(d, splitk, stream);
    case 32: return gemm::dispatch_bn<32>(d, splitk, stream);
    case 64: return gemm::dispatch_bn<64>(d, splitk, stream);
    case 128: return gemm::dispatch_bn<128>(d, splitk, stream);
    case 256: return gemm::dispatch_bn<256>(d, splitk, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ccl
