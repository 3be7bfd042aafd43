// Batched small-tensor collectives: ONE launch (one flag round) for a list of tensors.
//
// DDP gradient buckets, FSDP2's per-parameter-group collectives and the *_coalesced entry points of
// torch.distributed hand the backend a list of small tensors. Launching one kernel per tensor pays
// the launch and the cross-GPU flag round once per tensor (that is what the reference does:
// src/utils.h:344-358 of intel/torch-ccl loops over the list). Here the list travels as a pointer
// table in the kernel parameters and every tensor goes through the same single exchange.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "collectives.h"

namespace ccl {

constexpr int kMaxMulti = 32;   // tensors per launch (longer lists are split by the caller)

enum MultiMode : int { kMultiAllReduce = 0, kMultiReduceScatter = 1, kMultiAllGather = 2 };

struct MultiArgs {
  int n = 0;                 // tensors
  int mode = kMultiAllReduce;
  int op = kSum;
  int has_scale = 0;
  float scale = 1.0f;
  const void* in[kMaxMulti] = {};
  void* out[kMaxMulti] = {};
  // all_reduce: elements of tensor t; reduce_scatter: elements of ONE piece (in has world pieces);
  // all_gather: bytes of ONE piece (out has world pieces)
  unsigned long long count[kMaxMulti] = {};
  unsigned long long slot_bytes = 0;   // staging bytes per source rank (filled by the launcher)
};

// Staging bytes one source rank needs for the list (every tensor starts on a 16-byte boundary).
size_t multi_slot_bytes(int dtype, const MultiArgs& a);
// dtype: element type of the reductions (ignored for all_gather).
cudaError_t launch_multi(int dtype, const RankCtx* ctx, const MultiArgs* args, const LaunchCfg& cfg);

}  // namespace ccl
