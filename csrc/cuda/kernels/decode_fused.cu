// Tensor-parallel decode kernels that fold the collective into the compute kernel next to it.
//
// gemm_ar_norm — one launch per row-parallel projection (o_proj, down_proj):
//
//     h   <- h + sum over ranks r of  x_r[rows, K_r] · W_r[hidden, K_r]^T        (bf16, fp32 accumulate)
//     out <- rmsnorm(h) * weight
//
//   GEMM part: the swap-AB tcgen05 GEMM of gemm_tcgen05.cuh (weights on the 128-row UMMA M side,
//   the few activation rows on the N side, split-K over a thread-block cluster with the DSMEM
//   reduce-scatter), grid = hidden/128 tiles x split. Its epilogue does not write the partial
//   product to this GPU's memory: each CTA transposes its [features x rows] block inside the quads
//   of a warp and stores it, as bf16 low-latency units {data, epoch, data, epoch}, into slot
//   [parity][this rank] of EVERY rank's low-latency region (peer stores over NVLink, own rank
//   included), so the partial sums never make the round trip through HBM that a separate
//   all_reduce kernel needs.
//   Norm part: split-K cluster i < rows then owns row i, each of its CTAs an equal share of the
//   row's features: it polls the W slots of its rank until every unit of its share carries the
//   epoch, sums in rank order (fp32), adds the residual, exchanges its partial sum of squares
//   with the other CTAs of the cluster over distributed shared memory, normalises and writes the
//   new residual and the normalised output. Rounding points are those of the unfused sequence
//   GEMM -> all_reduce -> add -> rmsnorm, so results are bit-identical to it.
//   No CTA's GEMM part ever waits for another rank, and a row owner only waits for data that GEMM
//   parts push, so the kernel needs no co-residency guarantee across GPUs; all waits are bounded.
//
// sample_allgather — one launch per step: arg-max over the fp32 logits of the rank's vocabulary
//   shard, the {value, global id} pair pushed to every rank through the low-latency slots, choice
//   of the global winner (largest value, lowest rank on ties), bookkeeping for the next step.
//
// Both kernels are one round of the communicator's epoch protocol. With gridDim.y == world they
// play every rank on one GPU (tests).
#include "decode_fused.h"

#include "gemm.h"
#include "gemm_tcgen05.cuh"
#include "ll_norm.cuh"
#include "tma_desc.h"

namespace ccl {
namespace {

using gemm::kBK;
using gemm::kBM;

struct ArNormRank {
  void* residual;
  const void* weight;
  void* out;
};
struct ArNormShape {
  int rows, hidden;
  float eps;
};
template <int NR>
struct alignas(64) ArNormPack {
  CUtensorMap a[NR];
  CUtensorMap b[NR];
  ArNormRank r[NR];
};

// Epilogue of the swap-AB tile: thread = one output feature m, v = 16 activation rows n0..n0+15.
// A 4x4 transpose inside each quad of lanes turns that into 4 consecutive features of one row,
// which is one 16-byte low-latency unit per destination rank.
struct LLPushEpilogue {
  const RankCtx* ctx;
  int rows;
  int hidden;
  __device__ __forceinline__ void operator()(const gemm::Params&, int m, int n0, const float (&v)[16]) const {
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctx->state);
    const uint32_t flag = epoch + 1;
    const int parity = (int)(epoch & 1);
    const int lane = threadIdx.x & 31;
    const int t = lane & 3;
    const unsigned qmask = 0xFu << (lane & ~3);
    const int mq = m & ~3;
    const int W = ctx->world, me = ctx->rank;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float a0 = v[4 * g], a1 = v[4 * g + 1], a2 = v[4 * g + 2], a3 = v[4 * g + 3];
      {
        const float s0 = (t & 1) ? a0 : a1, s1 = (t & 1) ? a2 : a3;
        const float r0 = __shfl_xor_sync(qmask, s0, 1), r1 = __shfl_xor_sync(qmask, s1, 1);
        if (t & 1) { a0 = r0; a2 = r1; } else { a1 = r0; a3 = r1; }
      }
      {
        const float s0 = (t & 2) ? a0 : a2, s1 = (t & 2) ? a1 : a3;
        const float r0 = __shfl_xor_sync(qmask, s0, 2), r1 = __shfl_xor_sync(qmask, s1, 2);
        if (t & 2) { a0 = r0; a1 = r1; } else { a2 = r0; a3 = r1; }
      }
      // a0..a3: features mq..mq+3 of activation row j
      const int j = n0 + 4 * g + t;
      if (j < rows) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(a2, a3);
        const uint32_t w0 = *reinterpret_cast<const uint32_t*>(&lo), w1 = *reinterpret_cast<const uint32_t*>(&hi);
        const size_t off = ((size_t)j * hidden + mq) * 2;
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < W) ll_store8(ll_slot(*ctx, p, parity, me), off, w0, w1, flag);
      }
    }
  }
};

// MV: 16-byte vectors of a row per thread in the norm part (the row is split over the CTAs of the
// split-K cluster, so MV = 1 covers hidden <= 8 * 192 * splitk).
template <int BN, int MV, bool EMU>
__global__ void __launch_bounds__(gemm::kThreads, 3)
    gemm_ar_norm_kernel(const __grid_constant__ ArNormPack<EMU ? kMaxRanks : 1> pk, const gemm::Params p,
                        const __grid_constant__ RankCtx ctx1, const RankCtx* ctx_table, const ArNormShape sh) {
  const int ri = EMU ? blockIdx.y : 0;
  const RankCtx& ctx = EMU ? ctx_table[ri] : ctx1;
  const ArNormRank& rk = pk.r[ri];
  __shared__ float s_red[33];
  __shared__ float s_part[2][8];   // per-CTA partial sums of squares of the cluster, double-buffered over rows
  const int n_ctas = gridDim.x * gridDim.z;
  const int nz = gridDim.z;                      // CTAs per cluster = split-K factor
  const int z = p.splitk > 1 ? (int)ptx::cluster_ctarank() : 0;
  // norm part: cluster c < rows owns row c (then c + gridDim.x, ...); CTA z of the cluster owns
  // vectors [z * hvc, (z + 1) * hvc) of the row
  const int hvc = sh.hidden / 8 / nz;
  const int v0 = z * hvc, v1 = v0 + hvc;
  const bool has_row = (int)blockIdx.x < sh.rows;

  // the norm weights are constants: fetch them before anything that waits
  Vec<__nv_bfloat16> wv[MV];
  if (has_row) ll_load_norm_weight<__nv_bfloat16, MV>(rk.weight, v0, v1, wv);

  const int m0 = blockIdx.x * kBM;
  gemm::gemm_tile_body<BN, false>(&pk.a[ri], &pk.b[ri], p, LLPushEpilogue{&ctx, sh.rows, sh.hidden},
                                  gemm::TileCoord{m0, m0, 0});
  ptx::griddep_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctx.state);
  const size_t row_bytes = (size_t)sh.hidden * 2;
  int it = 0;
  for (int row = blockIdx.x; row < sh.rows; row += gridDim.x, ++it) {
    char* res = static_cast<char*>(rk.residual) + (size_t)row * row_bytes;
    Vec<__nv_bfloat16> hn[MV];
    const float ss = ll_row_gather_add<__nv_bfloat16, MV, 4>(ctx, (int)(epoch & 1), epoch + 1, kOwnInSlot, (size_t)row * row_bytes,
                                                             v0, v1, nullptr, res, res, hn, nullptr);
    float total = block_sum(ss, s_red);
    if (nz > 1) {
      // every CTA of the cluster hands its partial to every other one over distributed shared
      // memory; all of them then add the partials in the same (rank) order
      float* buf = s_part[it & 1];
      if ((int)threadIdx.x < nz) ptx::st_cluster_f32(ptx::mapa(ptx::smem_u32(buf + z), threadIdx.x), total);
      ptx::cluster_arrive();
      ptx::cluster_wait();
      total = 0.f;
      for (int q = 0; q < nz; ++q) total += buf[q];
    }
    const float rstd = rsqrtf(total / (float)sh.hidden + sh.eps);
    ll_row_write_norm<__nv_bfloat16, MV>(hn, wv, rstd, v0, v1, static_cast<char*>(rk.out) + (size_t)row * row_bytes);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(ctx.state + 1, 1u);
    if (t == (uint32_t)n_ctas - 1) {
      ctx.state[1] = 0;
      ctx.state[0] = epoch + 1;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// arg-max + all-gather of the winners
// ---------------------------------------------------------------------------------------------
template <bool EMU>
struct LaunchSample {
  RankCtx ctx;
  SampleArgs args;
  const RankCtx* ctx_table;
  SampleArgs args_table[EMU ? kMaxRanks : 1];
};

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

template <bool EMU>
__global__ void __launch_bounds__(256) sample_allgather_kernel(const __grid_constant__ LaunchSample<EMU> L) {
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;
  const SampleArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;
  __shared__ int s_failed;
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  Sync sy(ctx, &s_failed, true);
  const int W = ctx.world, me = ctx.rank;
  const int row = blockIdx.x;
  const float* lg = a.logits + (size_t)row * a.ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < a.vshard; i += blockDim.x) better(bv, bi, lg[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    s_val[threadIdx.x >> 5] = bv;
    s_idx[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) better(bv, bi, s_val[w], s_idx[w]);
    bi += me * a.vshard;
    if (W > 1) {
      const uint32_t flag = sy.epoch + 1;
      for (int p = 0; p < W; ++p)
        ll_store8(ll_slot(ctx, p, sy.parity(0), me), (size_t)row * 8, __float_as_uint(bv), (uint32_t)bi, flag);
    } else {
      s_val[0] = bv;
      s_idx[0] = bi;
    }
  }
  if (W > 1) {
    __syncthreads();
    if ((int)threadIdx.x < W) {
      const uint32_t flag = sy.epoch + 1;
      const char* src = ll_slot(ctx, me, sy.parity(0), threadIdx.x) + (size_t)row * 16;
      uint4 s = ptx::ld_volatile_v4(src);
      if (!(s.y == flag && s.w == flag)) {
        const uint64_t t0 = ptx::globaltimer_ns();
        uint32_t it = 0;
        while (true) {
          s = ptx::ld_volatile_v4(src);
          if (s.y == flag && s.w == flag) break;
          if ((++it & 63u) == 0 && (ptx::globaltimer_ns() - t0 > ctx.spin_ns || ((it & 1023u) == 0 && comm_aborted(ctx)))) {
            sy.report(threadIdx.x, 0);
            break;
          }
        }
      }
      s_val[threadIdx.x] = __uint_as_float(s.x);
      s_idx[threadIdx.x] = (int)s.z;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = s_val[0];
    int id = s_idx[0];
    for (int p = 1; p < W; ++p)
      if (s_val[p] > v) {  // ties go to the lowest rank, i.e. the lowest global id
        v = s_val[p];
        id = s_idx[p];
      }
    a.next_tokens[row] = id;
    if (a.tokens) a.tokens[row] = id;
    if (a.positions) a.positions[row] += 1;
  }
  if (W > 1) sy.finish(1);
}

// Opt a kernel into large dynamic shared memory, once per device.
template <typename K>
cudaError_t configure_once(K kern, DeviceOnce& once) {
  if (!once.pending()) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 202 * 1024);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  once.done();
  return cudaSuccess;
}

template <int BN, int MV, bool EMU>
cudaError_t launch_ar_norm_bn(const RankCtx* ctx, const RankCtx* dev_ctx_table, const GemmArNormArgs* args, int nctx,
                              int splitk, cudaStream_t stream) {
  constexpr int NR = EMU ? kMaxRanks : 1;
  const GemmArNormArgs& a0 = args[0];
  const int m_tiles = a0.hidden / kBM;
  const int k_iters = (a0.K + kBK - 1) / kBK;
  const int per = (k_iters + splitk - 1) / splitk;
  // two CTAs per SM: the whole grid is resident in one wave
  constexpr size_t kBudget = 100 * 1024;
  int stages = gemm::kMaxStages;
  while (stages > 2 && gemm::smem_bytes<BN, false>(stages, splitk) > kBudget) --stages;
  if (stages > per && per >= 2) stages = per;
  const size_t smem = gemm::smem_bytes<BN, false>(stages, splitk);

  ArNormPack<NR> pk;
  for (int i = 0; i < nctx; ++i) {
    const GemmArNormArgs& a = args[i];
    if (!tma::make_2d_bf16(&pk.a[i], a.w, (uint64_t)a.w_packed_rows, (uint64_t)kBK, (uint64_t)kBK, kBM, kBK))
      return cudaErrorInvalidValue;
    if (!tma::make_2d_bf16(&pk.b[i], a.x, (uint64_t)a.rows, (uint64_t)a.K, (uint64_t)a.ldx, BN, kBK))
      return cudaErrorInvalidValue;
    pk.r[i] = ArNormRank{a.residual, a.weight, a.out};
  }
  for (int i = nctx; i < NR; ++i) {
    pk.a[i] = pk.a[0];
    pk.b[i] = pk.b[0];
    pk.r[i] = pk.r[0];
  }
  gemm::Params p{};
  p.M = a0.hidden;
  p.N = a0.rows;
  p.K = a0.K;
  p.out = nullptr;
  p.ldo = 0;
  p.trans_out = 1;
  p.stages = stages;
  p.splitk = splitk;
  p.status = ctx[0].status;
  p.a_tiled = 1;
  p.a_static = 1;
  p.a_packed = a0.w;
  p.k_tiles = k_iters;
  ArNormShape sh{a0.rows, a0.hidden, a0.eps};

  auto kern = gemm_ar_norm_kernel<BN, MV, EMU>;
  static DeviceOnce configured;
  cudaError_t e = configure_once(kern, configured);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(m_tiles, EMU ? nctx : 1, splitk);
  cfg.blockDim = dim3(gemm::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splitk;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + (EMU ? 0 : pdl_launch_attr(&attr[1]));
  e = cudaLaunchKernelEx(&cfg, kern, pk, p, ctx[0], dev_ctx_table, sh);
  if (e == cudaSuccess) launch_count_add(1);
  return e;
}

}  // namespace

int gemm_ar_norm_max_rows(int hidden) {
  if (hidden <= 0) return 0;
  const size_t r = kLLSlotBytes / ((size_t)hidden * 4);
  return (int)(r < 64 ? r : 64);
}

cudaError_t launch_gemm_ar_norm(const RankCtx* ctx, const RankCtx* dev_ctx_table, const GemmArNormArgs* args, int nctx,
                                cudaStream_t stream) {
  if (nctx < 1 || nctx > kMaxRanks || (nctx > 1 && !dev_ctx_table)) return cudaErrorInvalidValue;
  const GemmArNormArgs& a0 = args[0];
  if (a0.hidden <= 0 || a0.hidden % kBM != 0 || a0.rows <= 0 || a0.K <= 0 || a0.K % 8 != 0) return cudaErrorInvalidValue;
  if (a0.rows > gemm_ar_norm_max_rows(a0.hidden)) return cudaErrorInvalidValue;
  for (int i = 0; i < nctx; ++i) {
    const GemmArNormArgs& a = args[i];
    if (!a.w || !a.x || !a.residual || !a.weight || !a.out) return cudaErrorInvalidValue;
    if (a.rows != a0.rows || a.hidden != a0.hidden || a.K != a0.K || a.ldx % 8 != 0) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.residual) |
         reinterpret_cast<uintptr_t>(a.weight) | reinterpret_cast<uintptr_t>(a.out)) & 15)
      return cudaErrorInvalidValue;
    const int64_t k_tiles = (a.K + kBK - 1) / kBK;
    if (a.w_packed_rows < (int64_t)a.hidden * k_tiles) return cudaErrorInvalidValue;
  }
  const int m_tiles = a0.hidden / kBM;
  const int k_iters = (a0.K + kBK - 1) / kBK;
  int splitk = a0.splitk;
  if (splitk == 0) {
    // memory-bound: the largest power-of-two split that keeps the grid within one wave of two
    // CTAs per SM (~264 CTAs) and leaves every CTA at least two K steps
    splitk = 8;
    while (splitk > 1 && (m_tiles * splitk > 264 || k_iters / splitk < 2)) splitk >>= 1;
  }
  if (splitk != 1 && splitk != 2 && splitk != 4 && splitk != 8) return cudaErrorInvalidValue;
  while (splitk > 1 && k_iters / splitk < 1) splitk >>= 1;
  const bool emu = nctx > 1;
  const int bn = a0.rows <= 16 ? 16 : (a0.rows <= 32 ? 32 : 64);
  // vectors of a row per thread in the norm part: the row is split over the split-K cluster
  const int per_cta = a0.hidden / 8 / splitk;
  const int mv = per_cta <= gemm::kThreads ? 1 : (per_cta <= 3 * gemm::kThreads ? 3 : kLLNormMaxVec);
  if (per_cta > kLLNormMaxVec * gemm::kThreads || (a0.hidden / 8) % splitk != 0) return cudaErrorInvalidValue;
#define CCL_ARNORM_MV(BN, MV)                                                                                 \
  return emu ? launch_ar_norm_bn<BN, MV, true>(ctx, dev_ctx_table, args, nctx, splitk, stream)                \
             : launch_ar_norm_bn<BN, MV, false>(ctx, dev_ctx_table, args, nctx, splitk, stream);
#define CCL_ARNORM_CASE(BN)                                                                                   \
  case BN:                                                                                                    \
    if (mv == 1) { CCL_ARNORM_MV(BN, 1) }                                                                     \
    if (mv == 3) { CCL_ARNORM_MV(BN, 3) }                                                                     \
    CCL_ARNORM_MV(BN, kLLNormMaxVec)
  switch (bn) {
    CCL_ARNORM_CASE(16)
    CCL_ARNORM_CASE(32)
    CCL_ARNORM_CASE(64)
    default: return cudaErrorInvalidValue;
  }
#undef CCL_ARNORM_CASE
#undef CCL_ARNORM_MV
}

cudaError_t launch_sample_allgather(const RankCtx* ctx, const RankCtx* dev_ctx_table, const SampleArgs* args, int nctx,
                                    cudaStream_t stream) {
  if (nctx < 1 || nctx > kMaxRanks || (nctx > 1 && !dev_ctx_table)) return cudaErrorInvalidValue;
  const SampleArgs& a0 = args[0];
  if (a0.rows <= 0 || a0.vshard <= 0 || !a0.logits || !a0.next_tokens) return cudaErrorInvalidValue;
  if ((size_t)a0.rows * 16 > kLLSlotBytes) return cudaErrorInvalidValue;
  cudaError_t e;
  if (nctx == 1) {
    LaunchSample<false> L;
    L.ctx = ctx[0];
    L.args = a0;
    L.ctx_table = nullptr;
    L.args_table[0] = a0;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(a0.rows, 1, 1);
    lc.blockDim = dim3(256, 1, 1);
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    lc.attrs = attr;
    lc.numAttrs = pdl_launch_attr(&attr[0]);
    e = cudaLaunchKernelEx(&lc, sample_allgather_kernel<false>, L);
  } else {
    LaunchSample<true> L;
    L.ctx = RankCtx{};
    L.args = SampleArgs{};
    L.ctx_table = dev_ctx_table;
    for (int i = 0; i < kMaxRanks; ++i) L.args_table[i] = args[i < nctx ? i : 0];
    void* params[] = {&L};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(sample_allgather_kernel<true>), dim3(a0.rows, nctx, 1),
                                    dim3(256, 1, 1), params, 0, stream);
  }
  if (e == cudaSuccess) launch_count_add(1);
  return e;
}

}  // namespace ccl
