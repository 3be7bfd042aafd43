// Host interface of the fused MoE dispatch / combine kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "collectives.h"
#include "comm_types.h"

namespace ccl {

struct MoeArgs {
  // dispatch: x = tokens [tokens, hidden] bf16; combine: x = expert outputs [rows, hidden] bf16
  const void* x = nullptr;
  const int* expert_idx = nullptr;  // dispatch: [tokens, topk] global expert ids
  const float* gate = nullptr;      // combine: [tokens, topk] routing weights
  void* out_x = nullptr;            // dispatch: [>= rows, hidden] received rows; combine: [tokens, hidden]
  int* out_meta = nullptr;          // [rows, 3]: source rank, source slot t*topk+k, local expert (written by dispatch, read by combine)
  int* out_count = nullptr;         // dispatch: [1 + world]: total rows, rows per source
  const int* in_rows = nullptr;     // combine: device pointer to the number of received rows
  int tokens = 0, topk = 0, hidden = 0;
  int experts_per_rank = 1;
  int cap = 0;                      // rows one source may send to one destination
  unsigned long long slot_bytes = 0;  // moe_dispatch_slot_bytes(cap, hidden)
};

size_t moe_dispatch_slot_bytes(int cap, int hidden);
cudaError_t launch_moe_dispatch(const RankCtx* ctx, const MoeArgs* args, const LaunchCfg& cfg);
cudaError_t launch_moe_combine(const RankCtx* ctx, const MoeArgs* args, const LaunchCfg& cfg);

}  // namespace ccl
