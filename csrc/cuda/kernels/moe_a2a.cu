// Expert-parallel MoE token exchange fused with the routing permutation.
//
// dispatch: every (token, k) pair whose expert lives on rank d is written — hidden vector plus a
//   small record {source slot t*K+k, local expert id} — straight into rank d's arena over NVLink,
//   at a position taken from a per-destination counter; no intermediate "sorted by destination"
//   copy of the activations and no host-side split sizes. After one flag round the receiver
//   compacts the W source segments into one contiguous [rows, hidden] matrix for the expert GEMMs
//   and keeps the records for the way back.
// combine: each expert-output row is written back into the arena of the rank that owns the token,
//   at its slot t*K+k; after one flag round the owner forms out[t] = sum_k gate[t,k] * row(t,k).
//
// Replaces all_to_all_single with uneven splits (reference call sites src/gpu/dpcpp_ccl.cpp:
// 1371-1466, oneCCL alltoallv) plus the permute / unpermute kernels an MoE layer runs around it.
// Both kernels follow the communicator's epoch / parity protocol (one round each); because a
// receiver needs ALL of a sender's CTAs, it waits for every (source, CTA) flag of the phase.
#include "moe_a2a.h"

#include "comm.cuh"
#include "gemm.h"

namespace ccl {
namespace {

template <bool EMU>
struct LaunchMoe {
  RankCtx ctx;
  MoeArgs args;
  const RankCtx* ctx_table;
  const MoeArgs* args_table;
};

// Publish this CTA's writes to every rank, the own one included (other CTAs of this rank read the
// local segment). All threads call it.
__device__ __forceinline__ void signal_all_incl_self(Sync& sy, int phase) {
  __syncthreads();
  if (*sy.failed == 0 && (int)threadIdx.x < sy.ctx.world)
    ptx::st_release_sys(flag_ptr(sy.ctx.flags[threadIdx.x], phase, sy.ctx.rank, sy.blk), sy.epoch + 1);
}

// Wait for the flags of all CTAs of all ranks for (phase, round 0). All threads call it. The CTAs
// of one rank wait for each other here, so the grid must be small enough to be fully resident.
__device__ __forceinline__ bool wait_all_blocks(Sync& sy, int phase, int nblk) {
  const int W = sy.ctx.world;
  for (int i = threadIdx.x; i < W * nblk; i += blockDim.x) {
    const int src = i / nblk, b = i - src * nblk;
    if (*sy.failed) continue;  // the own rank's CTAs are waited for too: they fill the local segment
    const uint32_t* f = flag_ptr(sy.ctx.flags[sy.ctx.rank], phase, src, b);
    if (!ptx::spin_until_epoch(f, sy.epoch + 1, sy.ctx.spin_ns, sy.ctx.abort_flag)) sy.report(src, phase);
  }
  __syncthreads();
  return *sy.failed == 0;
}

// Arena layout of one parity half during dispatch, per source slot s (stride slot_bytes):
//   [cap rows x hidden bf16][cap x int2 records][kMaxBlocks x uint32 per-CTA row counts]
__device__ __forceinline__ size_t rows_bytes(const MoeArgs& a) { return (size_t)a.cap * a.hidden * 2; }
__device__ __forceinline__ size_t meta_off(const MoeArgs& a) { return rows_bytes(a); }
__device__ __forceinline__ size_t cnt_off(const MoeArgs& a) { return rows_bytes(a) + (size_t)a.cap * 8; }

template <bool EMU>
__global__ void __launch_bounds__(512) moe_dispatch_kernel(const __grid_constant__ LaunchMoe<EMU> L) {
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;
  const MoeArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;
  __shared__ int s_failed;
  Sync sy(ctx, &s_failed, true);
  const int W = ctx.world, me = ctx.rank;
  const int nblk = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int pairs = a.tokens * a.topk;
  const int hv = a.hidden / 8;  // 16-byte vectors per row
  // per-destination counters of this rank live in its state words [96, 104)
  uint32_t* cursor = ctx.state + 96;
  __shared__ uint32_t s_sent[kMaxRanks];
  if (threadIdx.x < kMaxRanks) s_sent[threadIdx.x] = 0;
  __syncthreads();

  // ---- push: one warp per (token, k) pair ---------------------------------------------------
  const int per = (pairs + nblk - 1) / nblk;
  const int p0 = blockIdx.x * per, p1 = min(pairs, p0 + per);
  for (int pi = p0 + warp; pi < p1; pi += nwarp) {
    const int e = a.expert_idx[pi];
    const int d = e / a.experts_per_rank;
    uint32_t pos = 0;
    if (lane == 0) {
      pos = atomicAdd(cursor + d, 1u);
      atomicAdd(&s_sent[d], 1u);
    }
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= (uint32_t)a.cap) {  // over capacity: the row is dropped and the error recorded
      if (lane == 0 && ctx.status) atomicCAS(ctx.status, kStatusOk, kStatusBounds);
      continue;
    }
    char* slot = sy.half(d, 0) + (size_t)me * a.slot_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(a.x) + (size_t)(pi / a.topk) * hv;
    char* dst = slot + (size_t)pos * a.hidden * 2;
    for (int i = lane; i < hv; i += 32) ptx::st_v4(dst + (size_t)i * 16, src[i]);
    if (lane == 0) {
      int2 rec = make_int2(pi, e - d * a.experts_per_rank);
      *reinterpret_cast<int2*>(slot + meta_off(a) + (size_t)pos * 8) = rec;
    }
  }
  __syncthreads();
  // rows this CTA sent to each destination (the receiver sums them over the CTAs)
  if ((int)threadIdx.x < W) {
    char* slot = sy.half(threadIdx.x, 0) + (size_t)me * a.slot_bytes;
    ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(slot + cnt_off(a)) + blockIdx.x, s_sent[threadIdx.x]);
  }
  signal_all_incl_self(sy, 0);
  bool ok = wait_all_blocks(sy, 0, nblk);

  // ---- compact the W source segments into out_x / out_meta ------------------------------------
  if (ok) {
    __shared__ uint32_t s_cnt[kMaxRanks], s_base[kMaxRanks + 1];
    if ((int)threadIdx.x < W) {
      const uint32_t* c = reinterpret_cast<const uint32_t*>(sy.half(me, 0) + (size_t)threadIdx.x * a.slot_bytes + cnt_off(a));
      uint32_t t = 0;
      for (int b = 0; b < nblk; ++b) t += ptx::ld_relaxed_sys(c + b);
      s_cnt[threadIdx.x] = min(t, (uint32_t)a.cap);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t acc = 0;
      for (int s = 0; s < W; ++s) {
        s_base[s] = acc;
        acc += s_cnt[s];
      }
      s_base[W] = acc;
      if (blockIdx.x == 0) {
        a.out_count[0] = (int)acc;
        for (int s = 0; s < W; ++s) a.out_count[1 + s] = (int)s_cnt[s];
      }
    }
    __syncthreads();
    const uint32_t total = s_base[W];
    const uint32_t rper = (total + nblk - 1) / nblk;
    const uint32_t r0 = min(total, blockIdx.x * rper), r1 = min(total, r0 + rper);
    for (uint32_t r = r0 + warp; r < r1; r += nwarp) {
      int s = 0;
      while (s + 1 < W && r >= s_base[s + 1]) ++s;
      const uint32_t i = r - s_base[s];
      const char* slot = sy.half(me, 0) + (size_t)s * a.slot_bytes;
      const char* src = slot + (size_t)i * a.hidden * 2;
      uint4* dst = reinterpret_cast<uint4*>(a.out_x) + (size_t)r * hv;
      for (int v = lane; v < hv; v += 32) dst[v] = ptx::ld_relaxed_sys_v4(src + (size_t)v * 16);
      if (lane == 0) {
        // written by the source GPU: same system-coherent load as the rows above
        const uint32_t* recp = reinterpret_cast<const uint32_t*>(slot + meta_off(a) + (size_t)i * 8);
        const int2 rec = make_int2((int)ptx::ld_relaxed_sys(recp), (int)ptx::ld_relaxed_sys(recp + 1));
        a.out_meta[3 * r] = s;        // source rank
        a.out_meta[3 * r + 1] = rec.x;  // slot t*K+k at the source
        a.out_meta[3 * r + 2] = rec.y;  // local expert
      }
    }
  }
  // re-arm the cursors for the next call and advance the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(ctx.state + 1, 1u);
    if (t == gridDim.x - 1) {
      for (int d = 0; d < kMaxRanks; ++d) cursor[d] = 0;
      ctx.state[1] = 0;
      ctx.state[0] = sy.epoch + 1;
      __threadfence();
    }
  }
}

template <bool EMU>
__global__ void __launch_bounds__(512) moe_combine_kernel(const __grid_constant__ LaunchMoe<EMU> L) {
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;
  const MoeArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;
  __shared__ int s_failed;
  Sync sy(ctx, &s_failed, true);
  const int nblk = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int hv = a.hidden / 8;
  const int rows = a.in_rows[0];  // rows received by dispatch (device value)

  // ---- push every expert-output row back to the slot of its token at the source ----------------
  const int per = (rows + nblk - 1) / nblk;
  const int r0 = min(rows, (int)blockIdx.x * per), r1 = min(rows, r0 + per);
  for (int r = r0 + warp; r < r1; r += nwarp) {
    const int s = a.out_meta[3 * r], slot_idx = a.out_meta[3 * r + 1];
    const uint4* src = reinterpret_cast<const uint4*>(a.x) + (size_t)r * hv;
    char* dst = sy.half(s, 0) + (size_t)slot_idx * a.hidden * 2;
    for (int i = lane; i < hv; i += 32) ptx::st_v4(dst + (size_t)i * 16, src[i]);
  }
  signal_all_incl_self(sy, 0);
  const bool ok = wait_all_blocks(sy, 0, nblk);

  // ---- weighted sum over the K experts of each token -----------------------------------------
  if (ok) {
    const int tper = (a.tokens + nblk - 1) / nblk;
    const int t0 = min(a.tokens, (int)blockIdx.x * tper), t1 = min(a.tokens, t0 + tper);
    const char* buf = sy.half(ctx.rank, 0);
    for (int t = t0 + warp; t < t1; t += nwarp) {
      for (int i = lane; i < hv; i += 32) {
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
        for (int k = 0; k < a.topk; ++k) {
          const float w = a.gate[(size_t)t * a.topk + k];
          const Vec<__nv_bfloat16> v = load_stage<__nv_bfloat16>(buf + ((size_t)(t * a.topk + k) * hv + i) * 16);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] += w * __bfloat162float(v.v[q]);
        }
        Vec<__nv_bfloat16> o;
#pragma unroll
        for (int q = 0; q < 8; ++q) o.v[q] = __float2bfloat16(acc[q]);
        reinterpret_cast<uint4*>(a.out_x)[(size_t)t * hv + i] = *reinterpret_cast<const uint4*>(&o);
      }
    }
  }
  sy.finish(1);
}

template <typename KR, typename KE>
cudaError_t launch_moe(KR kreal, KE kemu, const RankCtx* ctx, const MoeArgs* args, const LaunchCfg& cfg) {
  dim3 block(cfg.nthreads);
  if (!cfg.cooperative) {
    LaunchMoe<false> L;
    L.ctx = *ctx;
    L.args = *args;
    L.ctx_table = nullptr;
    L.args_table = nullptr;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(cfg.nblocks, 1, 1);
    lc.blockDim = block;
    lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    lc.attrs = attr;
    lc.numAttrs = pdl_launch_attr(&attr[0]);
    return cudaLaunchKernelEx(&lc, kreal, L);
  }
  LaunchMoe<true> L;
  L.ctx = RankCtx{};
  L.args = MoeArgs{};
  L.ctx_table = ctx;
  L.args_table = args;
  dim3 grid(cfg.nblocks, cfg.nctx, 1);
  void* params[] = {&L};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kemu), grid, block, params, 0, cfg.stream);
}

}  // namespace

size_t moe_dispatch_slot_bytes(int cap, int hidden) {
  return round_up((size_t)cap * hidden * 2 + (size_t)cap * 8 + (size_t)kMaxBlocks * 4, 256);
}

cudaError_t launch_moe_dispatch(const RankCtx* ctx, const MoeArgs* args, const LaunchCfg& cfg) {
  return launch_moe(moe_dispatch_kernel<false>, moe_dispatch_kernel<true>, ctx, args, cfg);
}
cudaError_t launch_moe_combine(const RankCtx* ctx, const MoeArgs* args, const LaunchCfg& cfg) {
  return launch_moe(moe_combine_kernel<false>, moe_combine_kernel<true>, ctx, args, cfg);
}

}  // namespace ccl
