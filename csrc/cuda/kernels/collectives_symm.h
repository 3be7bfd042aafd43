// Host interface of the zero-copy collectives on symmetric memory (no torch dependency).
//
// A symmetric tensor lives at the same offset of every rank's heap (RankCtx::heap), so a kernel
// reaches a peer's copy as heap[peer] + offset and nothing is staged through the arena: the
// all_reduce reads the peers' inputs in place and writes the peers' outputs in place. When the
// heaps are bound to an NVLink multicast object (RankCtx::mc_heap) the reduction runs inside the
// switch (multimem.ld_reduce) and the result is written to all ranks with one multimem.st.
//
// The reference stages every message through a temp buffer in 32 Mi-element chunks
// (src/gpu/allreduce.h:628-662 of intel/torch-ccl); this is the registered-buffer path it lacks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "collectives.h"

namespace ccl {

struct SymmArgs {
  unsigned long long in_off = 0;    // heap offset of the symmetric input (all_reduce, reduce_scatter)
  unsigned long long out_off = 0;   // heap offset of the symmetric output (all_reduce, all_gather)
  const void* in = nullptr;         // local input (all_gather)
  void* out = nullptr;              // local output (reduce_scatter)
  unsigned long long count = 0;     // all_reduce: elements of the whole tensor; reduce_scatter: elements per piece; all_gather: bytes per piece
  float scale = 1.0f;
  int has_scale = 0;
  int op = kSum;
  int use_mc = 0;                   // 1: through the multicast mapping (SUM of bf16 / f16 / f32 only)
};

// ctx/args: host pointers when cfg.nctx == 1, device tables when cfg.cooperative.
cudaError_t launch_allreduce_symm(int dtype, const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter_symm(int in_dtype, int out_dtype, const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg);
cudaError_t launch_all_gather_symm(const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg);

}  // namespace ccl
