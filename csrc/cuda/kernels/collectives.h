// Host interface of the peer-memory collective kernels (no torch dependency).
//
// Every launcher takes `nctx` rank contexts: 1 in a real multi-process run (the kernel plays
// this process's rank), or `world` in single-GPU emulation (one launch with gridDim.y == world
// plays every rank; `ctx` and `args` then point to DEVICE tables of `world` entries).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_types.h"

namespace ccl {

enum DType : int {
  kU8 = 0, kI8, kI16, kI32, kI64, kF16, kBF16, kF32, kF64,
};

__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case kU8: case kI8: return 1;
    case kI16: case kF16: case kBF16: return 2;
    case kI32: case kF32: return 4;
    default: return 8;
  }
}

enum RootedMode : int { kBroadcast = 0, kGather = 1, kScatter = 2, kBroadcastSwitch = 3 /* root writes all arenas with multimem.st */ };

// Arguments of one rank. Piece tables are indexed by peer rank.
struct CollArgs {
  const void* in = nullptr;
  void* out = nullptr;
  const void* in_piece[kMaxRanks] = {};   // reduce_scatter / all_to_all / scatter sources
  void* out_piece[kMaxRanks] = {};        // all_gather / all_to_all / gather destinations
  unsigned long long count = 0;           // elements (all_reduce) or bytes (broadcast)
  unsigned long long in_cnt[kMaxRanks] = {};   // per-piece sizes (elements for reductions, bytes otherwise)
  unsigned long long out_cnt[kMaxRanks] = {};
  unsigned long long chunk_vecs = 0;      // staging capacity per round, in 16-byte vectors (per slot)
  float scale = 1.0f;                     // applied after the reduction when has_scale != 0
  int has_scale = 0;
  int op = kSum;
  int root = -1;
  int ablate = kAblateNone;
  int mode = 0;                           // all_gather: 0 pull, 1 push; rooted: RootedMode
  int rounds = 0;                         // number of staging rounds (0: computed on device, all_to_all only)
};

struct LaunchCfg {
  int nblocks = 1;
  int nthreads = 512;
  int nctx = 1;            // 1 = real, world = emulation
  int cooperative = 0;     // 1 = emulation: ctx/args are DEVICE tables of nctx entries and the
                           // launch is cooperative so that all CTAs are co-resident
  cudaStream_t stream = nullptr;
};

// ctx/args: host pointers when nctx == 1, device tables when nctx > 1.
cudaError_t launch_allreduce_oneshot(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_allreduce_twoshot(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
// SUM of bf16 / f16 / f32 through the NVLink multicast mapping (RankCtx::mc_data; emulation plays it in software).
cudaError_t launch_allreduce_nvls(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter_nvls(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);  // in dtype == out dtype
cudaError_t launch_all_gather_nvls(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
// out dtype may differ from in dtype only for (bf16|f16) -> f32 (fused FSDP gradient cast).
cudaError_t launch_reduce_scatter(int in_dtype, int out_dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_all_gather(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_all_to_all(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_rooted(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);
cudaError_t launch_barrier(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg);

// Fused tensor-parallel epilogue: h = residual + all_reduce(x); residual <- h;
// out = rmsnorm(h) * weight. x, residual, out: [rows, hidden] (bf16 or f16), weight: [hidden].
struct FusedNormArgs {
  const void* x = nullptr;
  void* residual = nullptr;
  const void* weight = nullptr;
  void* out = nullptr;
  int rows = 0;
  int hidden = 0;
  float eps = 1e-5f;
  int ablate = kAblateNone;
  int use_ll = 0;   // 1: low-latency protocol (rows * hidden * 4 bytes must fit kLLSlotBytes)
  // Vocabulary-parallel embedding lookup fused in front (decode step start): when gather_tokens
  // is set, `x` is this rank's shard [gather_rows, hidden] of the embedding table and the
  // contribution of row i is x[gather_tokens[i] - gather_base] if that index falls inside the
  // shard, else zeros.
  const long long* gather_tokens = nullptr;
  long long gather_base = 0;
  int gather_rows = 0;
  int zero_residual = 0;   // 1: the incoming residual counts as zero and is not read
};
cudaError_t launch_allreduce_residual_rmsnorm(int dtype, const RankCtx* ctx, const FusedNormArgs* args, const LaunchCfg& cfg);

}  // namespace ccl
