// Tensor-parallel GEMMs fused with their collective, on tcgen05 / TMEM tiles fed by TMA (never
// multicast) with the transfer over NVLink peer memory overlapping the math tile by tile.
//
//   gemm_rs  (row-parallel linear + reduce-scatter):  out_r = sum_p (A_p · B_p^T)[rows of rank r]
//     Each rank multiplies its K-shard; the epilogue of every 128 x BN tile stores the bf16
//     partial straight into the arena of the rank that owns those rows (plain peer stores) and
//     bumps that rank's arrival counter. Tiles for the other ranks are computed first, the own
//     rows last. A small second kernel on the same stream waits (bounded) for the arrivals and
//     sums the W partials in rank order.
//
//   ag_gemm  (all-gather + column-parallel linear):  out = [A_0; ...; A_{W-1}] · B_r^T
//     A few "comm" CTAs (lowest block indices) push this rank's A shard into every peer's arena
//     and bump the peers' counters; all other CTAs are GEMM tiles, ordered so that the own shard
//     (read directly from the user's buffer) comes first and shard p is only touched after p's
//     counter arrived. Remote shards are read by TMA from THIS GPU's arena (the data crossed
//     NVLink once, into local memory); the acquire of the counter is ordered before the
//     async-proxy reads with a proxy fence.
//
// Both ops use the communicator's epoch / parity scheme (one round each) and arrival counters
// in flag phase 4; expected totals live in the rank's state words, so the ops are replayable
// from CUDA graphs. The reference has nothing comparable (its device code is two all-reduce
// kernel families); torch + NCCL would run these as a GEMM followed or preceded by a collective.
#include "gemm_collective.h"

#include "comm.cuh"
#include "gemm.h"
#include "gemm_tcgen05.cuh"
#include "tma_desc.h"

namespace ccl {
namespace {

using gemm::kBM;
using gemm::kBK;

constexpr int kRsCounterBlk = 0;
constexpr int kAgCounterBlk = 1;
constexpr int kRsStateBase = 64;   // state[64 + src]: arrivals expected so far (gemm_rs)
constexpr int kAgStateBase = 80;   // state[80 + src]: arrivals expected so far (ag_gemm)

struct RsInfo {
  int rows_per_rank;
  int tile_shift;              // rotation of the m-tile order: other ranks' rows first
  unsigned long long slot_bytes;  // one source's partial of one rank's rows
};

struct RsEpilogue {
  const RankCtx* ctx;
  int parity;
  int rows_per_rank;
  unsigned long long slot_bytes;
  __device__ __forceinline__ void operator()(const gemm::Params& p, int m, int n0, const float (&v)[16]) const {
    if (m >= p.M) return;
    const int d = m / rows_per_rank;
    const int lr = m - d * rows_per_rank;
    char* base = ctx->data[d] + (size_t)parity * ctx->half_bytes + (size_t)ctx->rank * slot_bytes;
    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(base) + (size_t)lr * p.N + n0;
    if (n0 + 16 <= p.N) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      ptx::st_v4(row, make_uint4(w[0], w[1], w[2], w[3]));
      ptx::st_v4(row + 8, make_uint4(w[4], w[5], w[6], w[7]));
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (n0 + j < p.N) row[j] = __float2bfloat16(v[j]);
    }
  }
};

template <int BN>
__global__ void __launch_bounds__(gemm::kThreads, 1)
    gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const gemm::Params p, const __grid_constant__ RankCtx ctx, const RsInfo info) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctx.state);
  const int m_tile = (blockIdx.x + info.tile_shift) % gridDim.x;
  const int m0 = m_tile * kBM;
  RsEpilogue epi{&ctx, (int)(epoch & 1), info.rows_per_rank, info.slot_bytes};
  gemm::gemm_tile_body<BN, false>(&tma_a, &tma_b, p, epi, gemm::TileCoord{m0, m0, (int)blockIdx.y * BN});
  // the body ends with a CTA barrier after the epilogue stores: publish the tile to its owner
  if (threadIdx.x == 0) {
    const int d = m0 / info.rows_per_rank;
    ptx::red_release_sys_add(flag_ptr(ctx.flags[d], 4, ctx.rank, kRsCounterBlk), 1u);
  }
}

struct RsReduceArgs {
  void* out;                   // [rows_per_rank, N] bf16
  unsigned long long nvec;     // rows_per_rank * N * 2 / 16
  unsigned long long slot_bytes;
  unsigned int tiles_per_src;  // arrivals expected from each source per call
};

__global__ void __launch_bounds__(1024) gemm_rs_reduce_kernel(const __grid_constant__ RankCtx ctx, const RsReduceArgs a) {
  __shared__ int s_failed;
  Sync sy(ctx, &s_failed, true);
  const int W = ctx.world, me = ctx.rank;
  if ((int)threadIdx.x < W) {
    const uint32_t target = ctx.state[kRsStateBase + threadIdx.x] + a.tiles_per_src;
    if (!ptx::spin_until_epoch(flag_ptr(ctx.flags[me], 4, threadIdx.x, kRsCounterBlk), target, ctx.spin_ns, ctx.abort_flag))
      sy.report(threadIdx.x, 4);
  }
  __syncthreads();
  if (s_failed == 0) {
    const char* base = sy.half(me, 0);
    const size_t per = ceil_div((size_t)a.nvec, (size_t)gridDim.x);
    const size_t j0 = min((size_t)a.nvec, (size_t)blockIdx.x * per), j1 = min((size_t)a.nvec, j0 + per);
    for (size_t j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) acc[t] = 0.f;
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p) {
        if (p < W) {
          const Vec<__nv_bfloat16> v = load_stage<__nv_bfloat16>(base + (size_t)p * a.slot_bytes + j * 16);
#pragma unroll
          for (int t = 0; t < 8; ++t) acc[t] += __bfloat162float(v.v[t]);
        }
      }
      Vec<__nv_bfloat16> r;
#pragma unroll
      for (int t = 0; t < 8; ++t) r.v[t] = __float2bfloat16(acc[t]);
      *reinterpret_cast<uint4*>(static_cast<char*>(a.out) + j * 16) = *reinterpret_cast<const uint4*>(&r);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(ctx.state + 1, 1u);
    if (t == gridDim.x - 1) {
      for (int p = 0; p < W; ++p) ctx.state[kRsStateBase + p] += a.tiles_per_src;
      ctx.state[1] = 0;
      ctx.state[0] = sy.epoch + 1;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// ag_gemm
// ---------------------------------------------------------------------------------------------
struct AgInfo {
  const void* a_shard;           // [rows_per_rank, K] bf16, this rank's rows
  unsigned long long shard_vecs; // rows_per_rank * K * 2 / 16
  unsigned long long slot_bytes; // rows_per_rank * K * 2
  int rows_per_rank;
  int ncomm;                     // comm CTAs (fused / push mode)
  int mode;                      // 0 fused, 1 push only, 2 GEMM only
  int m_tiles_per_shard;
  int n_tiles;
};

template <int BN>
__global__ void __launch_bounds__(gemm::kThreads, 1)
    ag_gemm_kernel(const __grid_constant__ CUtensorMap tma_own, const __grid_constant__ CUtensorMap tma_arena0,
                   const __grid_constant__ CUtensorMap tma_arena1, const __grid_constant__ CUtensorMap tma_b,
                   const gemm::Params p, const __grid_constant__ RankCtx ctx, const AgInfo info) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctx.state);
  const int parity = epoch & 1;
  const int W = ctx.world, me = ctx.rank;
  const int ncomm = info.mode == 2 ? 0 : info.ncomm;
  __shared__ int s_ok;

  if ((int)blockIdx.x < ncomm) {
    // ---- comm CTA: push a slice of the own shard into every peer's arena ----------------------
    const size_t per = ceil_div((size_t)info.shard_vecs, (size_t)ncomm);
    const size_t j0 = min((size_t)info.shard_vecs, (size_t)blockIdx.x * per), j1 = min((size_t)info.shard_vecs, j0 + per);
    const char* src = static_cast<const char*>(info.a_shard);
    for (size_t j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + j * 16);
#pragma unroll
      for (int q = 1; q < kMaxRanks; ++q) {
        if (q < W) {
          const int d = (me + q) % W;
          ptx::st_v4(ctx.data[d] + (size_t)parity * ctx.half_bytes + (size_t)me * info.slot_bytes + j * 16, v);
        }
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < W && (int)threadIdx.x != me)
      ptx::red_release_sys_add(flag_ptr(ctx.flags[threadIdx.x], 4, me, kAgCounterBlk), 1u);
  } else {
    // ---- GEMM CTA ------------------------------------------------------------------------------
    const int t = blockIdx.x - ncomm;
    const int tiles_per_shard = info.m_tiles_per_shard * info.n_tiles;
    const int si = t / tiles_per_shard;            // 0 = own shard, then me+1, me+2, ...
    const int rem = t - si * tiles_per_shard;
    const int mt = rem / info.n_tiles, nt = rem - mt * info.n_tiles;
    const int s = (me + si) % W;
    const int m0 = s * info.rows_per_rank + mt * kBM;
    if (threadIdx.x == 0) {
      int ok = 1;
      if (s != me) {
        const uint32_t target = ctx.state[kAgStateBase + s] + (uint32_t)info.ncomm;
        if (!ptx::spin_until_epoch(flag_ptr(ctx.flags[me], 4, s, kAgCounterBlk), target, ctx.spin_ns, ctx.abort_flag)) {
          ok = 0;
          if (ctx.status && atomicCAS(ctx.status, kStatusOk, kStatusTimeout) == kStatusOk) {
            ctx.status[1] = me;
            ctx.status[2] = s;
            ctx.status[3] = 4;
            __threadfence_system();
          }
        }
      }
      s_ok = ok;
    }
    __syncthreads();
    if (s_ok) {
      const CUtensorMap* ta = (s == me) ? &tma_own : (parity ? &tma_arena1 : &tma_arena0);
      const int a_row = (s == me) ? mt * kBM : m0;
      gemm::gemm_tile_body<BN, false>(ta, &tma_b, p, gemm::StoreEpilogue<__nv_bfloat16>{},
                                      gemm::TileCoord{a_row, m0, nt * BN});
    }
  }
  if (info.mode == 1) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t tk = atomicAdd(ctx.state + 1, 1u);
    if (tk == gridDim.x - 1) {
      for (int q = 0; q < W; ++q) ctx.state[kAgStateBase + q] += (uint32_t)info.ncomm;
      ctx.state[1] = 0;
      ctx.state[0] = epoch + 1;
      __threadfence();
    }
  }
}

// Opts one kernel instantiation into large dynamic shared memory, once per device.
template <typename K>
cudaError_t set_smem(K kern, size_t smem) {
  static DeviceOnce configured;  // one per instantiation of this template, i.e. per kernel
  if (!configured.pending()) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) configured.done();
  return e;
}

int pick_stages(int bn, int k_iters, size_t* smem_out) {
  constexpr size_t kMax = 200 * 1024;
  int stages = gemm::kMaxStages;
  auto bytes = [&](int st) {
    return bn == 256 ? gemm::smem_bytes<256, false>(st, 1) : gemm::smem_bytes<128, false>(st, 1);
  };
  while (stages > 2 && bytes(stages) > kMax) --stages;
  if (stages > k_iters && k_iters >= 2) stages = k_iters;
  *smem_out = bytes(stages);
  return stages;
}

}  // namespace

size_t gemm_rs_staging_bytes(int64_t M, int64_t N) { return (size_t)M * N * 2; }
size_t ag_gemm_staging_bytes(int64_t M, int64_t K) { return (size_t)M * K * 2; }

cudaError_t launch_gemm_rs(const RankCtx& ctx, const GemmRsArgs& g, cudaStream_t stream) {
  const int W = ctx.world;
  if (g.M % ((int64_t)W * kBM) != 0 || g.N % 16 != 0 || g.K % 8 != 0) return cudaErrorInvalidValue;
  if (gemm_rs_staging_bytes(g.M, g.N) > ctx.half_bytes) return cudaErrorInvalidValue;
  const int bn = g.N >= 256 ? 256 : 128;
  const int m_tiles = (int)(g.M / kBM), n_tiles = (int)((g.N + bn - 1) / bn);
  const int rows_per_rank = (int)(g.M / W);
  const int k_iters = (int)((g.K + kBK - 1) / kBK);
  size_t smem = 0;
  const int stages = pick_stages(bn, k_iters, &smem);
  CUtensorMap ta, tb;
  if (!tma::make_2d_bf16(&ta, g.a, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, kBM, kBK)) return cudaErrorInvalidValue;
  if (!tma::make_2d_bf16(&tb, g.b, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, bn, kBK)) return cudaErrorInvalidValue;
  gemm::Params p{};
  p.M = (int)g.M;
  p.N = (int)g.N;
  p.K = (int)g.K;
  p.out = nullptr;
  p.ldo = g.N;
  p.stages = stages;
  p.splitk = 1;
  p.status = ctx.status;
  RsInfo info;
  info.rows_per_rank = rows_per_rank;
  info.slot_bytes = (unsigned long long)rows_per_rank * g.N * 2;
  // start with the rows of rank me+1 and finish with the own rows
  info.tile_shift = ((ctx.rank + 1) % W) * (rows_per_rank / kBM);
  dim3 grid(m_tiles, n_tiles, 1);
  cudaError_t e;
  if (bn == 256) {
    if ((e = set_smem(gemm_rs_kernel<256>, 202 * 1024)) != cudaSuccess) return e;
    gemm_rs_kernel<256><<<grid, gemm::kThreads, smem, stream>>>(ta, tb, p, ctx, info);
  } else {
    if ((e = set_smem(gemm_rs_kernel<128>, 202 * 1024)) != cudaSuccess) return e;
    gemm_rs_kernel<128><<<grid, gemm::kThreads, smem, stream>>>(ta, tb, p, ctx, info);
  }
  return cudaGetLastError();
}

cudaError_t launch_gemm_rs_reduce(const RankCtx& ctx, const GemmRsArgs& g, int nblocks, cudaStream_t stream) {
  const int W = ctx.world;
  const int bn = g.N >= 256 ? 256 : 128;
  const int rows_per_rank = (int)(g.M / W);
  RsReduceArgs a;
  a.out = g.out;
  a.nvec = (unsigned long long)rows_per_rank * g.N * 2 / 16;
  a.slot_bytes = (unsigned long long)rows_per_rank * g.N * 2;
  a.tiles_per_src = (unsigned int)((rows_per_rank / kBM) * ((g.N + bn - 1) / bn));
  gemm_rs_reduce_kernel<<<nblocks, 512, 0, stream>>>(ctx, a);
  return cudaGetLastError();
}

cudaError_t launch_ag_gemm(const RankCtx& ctx, const AgGemmArgs& g, int mode, int ncomm, cudaStream_t stream) {
  const int W = ctx.world;
  const int rows_per_rank = (int)(g.M / W);
  if (g.M % ((int64_t)W * kBM) != 0 || g.K % 8 != 0) return cudaErrorInvalidValue;
  if (ag_gemm_staging_bytes(g.M, g.K) > ctx.half_bytes) return cudaErrorInvalidValue;
  const int bn = g.N >= 256 ? 256 : 128;
  const int n_tiles = (int)((g.N + bn - 1) / bn);
  const int k_iters = (int)((g.K + kBK - 1) / kBK);
  size_t smem = 0;
  const int stages = pick_stages(bn, k_iters, &smem);
  CUtensorMap t_own, t_a0, t_a1, tb;
  char* mine = ctx.data[ctx.rank];
  if (!tma::make_2d_bf16(&t_own, g.a_shard, (uint64_t)rows_per_rank, (uint64_t)g.K, (uint64_t)g.lda, kBM, kBK)) return cudaErrorInvalidValue;
  if (!tma::make_2d_bf16(&t_a0, mine, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.K, kBM, kBK)) return cudaErrorInvalidValue;
  if (!tma::make_2d_bf16(&t_a1, mine + ctx.half_bytes, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.K, kBM, kBK)) return cudaErrorInvalidValue;
  if (!tma::make_2d_bf16(&tb, g.b, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, bn, kBK)) return cudaErrorInvalidValue;
  if (g.lda != g.K) return cudaErrorInvalidValue;  // the pushed shard is packed
  gemm::Params p{};
  p.M = (int)g.M;
  p.N = (int)g.N;
  p.K = (int)g.K;
  p.out = g.out;
  p.ldo = g.ldo;
  p.stages = stages;
  p.splitk = 1;
  p.status = ctx.status;
  p.acquire_a = 1;
  AgInfo info;
  info.a_shard = g.a_shard;
  info.shard_vecs = (unsigned long long)rows_per_rank * g.K * 2 / 16;
  info.slot_bytes = (unsigned long long)rows_per_rank * g.K * 2;
  info.rows_per_rank = rows_per_rank;
  info.ncomm = W > 1 ? ncomm : 0;
  info.mode = mode;
  info.m_tiles_per_shard = rows_per_rank / kBM;
  info.n_tiles = n_tiles;
  const int gemm_ctas = W * info.m_tiles_per_shard * n_tiles;
  const int grid = mode == 1 ? info.ncomm : (mode == 2 ? gemm_ctas : info.ncomm + gemm_ctas);
  if (grid == 0) return cudaSuccess;
  cudaError_t e;
  if (bn == 256) {
    if ((e = set_smem(ag_gemm_kernel<256>, 202 * 1024)) != cudaSuccess) return e;
    ag_gemm_kernel<256><<<grid, gemm::kThreads, smem, stream>>>(t_own, t_a0, t_a1, tb, p, ctx, info);
  } else {
    if ((e = set_smem(ag_gemm_kernel<128>, 202 * 1024)) != cudaSuccess) return e;
    ag_gemm_kernel<128><<<grid, gemm::kThreads, smem, stream>>>(t_own, t_a0, t_a1, tb, p, ctx, info);
  }
  return cudaGetLastError();
}

}  // namespace ccl
