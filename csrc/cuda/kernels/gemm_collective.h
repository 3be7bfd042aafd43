// Host interface of the fused tensor-parallel GEMM + collective kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_types.h"

namespace ccl {

// out[M/W, N] (bf16) = this rank's rows of sum over ranks of A[M, K_local] · B[N, K_local]^T.
struct GemmRsArgs {
  const void* a = nullptr;  // [M, K_local] bf16, row stride lda
  const void* b = nullptr;  // [N, K_local] bf16, row stride ldb
  void* out = nullptr;      // [M / world, N] bf16, contiguous
  int64_t M = 0, N = 0, K = 0, lda = 0, ldb = 0;
};

// out[M, N] (bf16) = [A_0; ...; A_{W-1}] · B[N, K]^T where rank p contributes A_p [M/W, K].
struct AgGemmArgs {
  const void* a_shard = nullptr;  // [M / world, K] bf16, packed (lda == K)
  const void* b = nullptr;        // [N, K] bf16, row stride ldb
  void* out = nullptr;            // [M, N] bf16, row stride ldo
  int64_t M = 0, N = 0, K = 0, lda = 0, ldb = 0, ldo = 0;
};

size_t gemm_rs_staging_bytes(int64_t M, int64_t N);
size_t ag_gemm_staging_bytes(int64_t M, int64_t K);

// GEMM + push of the partial tiles into the owners' arenas (never waits on another rank).
cudaError_t launch_gemm_rs(const RankCtx& ctx, const GemmRsArgs& args, cudaStream_t stream);
// Waits for every source's tiles and sums them into args.out; advances the communicator epoch.
cudaError_t launch_gemm_rs_reduce(const RankCtx& ctx, const GemmRsArgs& args, int nblocks, cudaStream_t stream);
// mode 0: one fused launch (comm CTAs + GEMM CTAs); mode 1: push only; mode 2: GEMM only (the two
// halves exist so that several ranks can be played one after the other on a single GPU).
cudaError_t launch_ag_gemm(const RankCtx& ctx, const AgGemmArgs& args, int mode, int ncomm, cudaStream_t stream);

}  // namespace ccl
