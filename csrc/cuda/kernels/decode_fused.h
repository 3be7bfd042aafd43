// Host interface of the tensor-parallel decode kernels that fold a collective into the compute
// kernel next to it (no torch dependency):
//
//   gemm_ar_norm      row-parallel projection (o_proj, down_proj) + all_reduce + residual add +
//                     RMSNorm in ONE launch: h += sum over ranks of x_r · W_r^T ; out = rmsnorm(h) * w
//   sample_allgather  arg-max over the vocabulary shard + all-gather of the per-rank winners +
//                     choice of the global winner, in one launch
//
// Both run on the communicator's low-latency slots (one round of the epoch protocol each) and
// replace what the reference's tensor-parallel decode loop does with an oneCCL all_reduce between
// separate GEMM and norm kernels (tests/test_allreduce.py:49-76 of intel/torch-ccl).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_types.h"

namespace ccl {

struct GemmArNormArgs {
  const void* w = nullptr;        // this rank's K-shard of the weight [hidden, K], packed as 128x64 tiles (see GemmDesc::a_tiled)
  int64_t w_packed_rows = 0;      // rows of the packed [*, 64] matrix
  const void* x = nullptr;        // [rows, K] bf16 activations of this rank, row stride ldx
  int64_t ldx = 0;
  void* residual = nullptr;       // [rows, hidden] bf16, read and replaced by the new residual stream
  const void* weight = nullptr;   // [hidden] bf16 RMSNorm weight
  void* out = nullptr;            // [rows, hidden] bf16 normalised output
  int rows = 0, hidden = 0, K = 0;
  float eps = 1e-5f;
  int splitk = 0;                 // 0: chosen from the shape; else 1, 2, 4 or 8
};

// Largest number of rows the fused kernel takes for a given hidden size (the rows of all ranks
// travel through one low-latency slot per source).
int gemm_ar_norm_max_rows(int hidden);

// ctx / args: `nctx` host entries. nctx == 1 is the real thing (one process per GPU); nctx ==
// world plays every rank in one launch on one GPU (gridDim.y = world) and then needs
// `dev_ctx_table`, the same contexts in device memory.
cudaError_t launch_gemm_ar_norm(const RankCtx* ctx, const RankCtx* dev_ctx_table, const GemmArNormArgs* args, int nctx,
                                cudaStream_t stream);

struct SampleArgs {
  const float* logits = nullptr;  // [rows, ld] fp32 logits of this rank's vocabulary shard
  int64_t ld = 0;
  int vshard = 0;                 // columns per rank; global id = rank * vshard + column
  int rows = 0;
  long long* next_tokens = nullptr;  // [rows] global winner
  long long* tokens = nullptr;       // [rows] optional second copy (the next step's input ids)
  int* positions = nullptr;          // [rows] optional, incremented by one
};
cudaError_t launch_sample_allgather(const RankCtx* ctx, const RankCtx* dev_ctx_table, const SampleArgs* args, int nctx,
                                    cudaStream_t stream);

}  // namespace ccl
