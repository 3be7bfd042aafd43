// Host-visible types shared by the collective kernels and their launchers: arena geometry,
// the per-rank device context and the reduction / ablation enums.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ccl {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 256;   // CTAs per collective kernel (flag slots per source rank)
constexpr int kNumPhases = 5;     // phases 0-3: epoch flags of the collectives; 4: arrival counters of the fused GEMM ops
constexpr size_t kFlagBytes = (size_t)kNumPhases * kMaxRanks * kMaxBlocks * sizeof(uint32_t);
constexpr size_t kStateBytes = 4096;
// Low-latency ("LL") region: per parity and source rank one slot in which every 16-byte store carries
// 8 bytes of payload and two copies of the call's epoch, so the receiver needs no separate flag.
constexpr size_t kLLSlotBytes = 512 << 10;
constexpr size_t kLLBytes = 2 * kMaxRanks * kLLSlotBytes;  // epoch, ticket, scratch tables (all-to-all counts, ...)

// Status codes written to RankCtx::status[0]; status[1..3] = rank, peer, phase.
enum : int { kStatusOk = 0, kStatusTimeout = 1, kStatusBounds = 2, kStatusAborted = 3 };

struct RankCtx {
  char* data[kMaxRanks];        // peers' arena base addresses as mapped in this rank
  uint32_t* flags[kMaxRanks];   // peers' flag areas
  uint32_t* state;              // own state words: [0] epoch, [1] ticket, [16..] scratch
  int* status;                  // host-visible error record (4 ints)
  int* abort_flag;              // host-written word (mapped host memory): non-zero makes every bounded wait give up
  unsigned long long half_bytes;  // size of one data half
  unsigned long long spin_ns;     // wait budget
  char* ll[kMaxRanks];          // peers' low-latency regions
  char* mc_data;                // NVLS multicast mapping of the arenas (nullptr if unavailable)
  char* heap[kMaxRanks];        // peers' symmetric heaps (user tensors allocated through the backend; null until the first one)
  char* mc_heap;                // NVLS multicast mapping of the heaps (nullptr if unavailable)
  int rank;
  int world;
};

enum ReduceKind : int {
  kSum = 0, kProd = 1, kMin = 2, kMax = 3, kBand = 4, kBor = 5, kBxor = 6,
};

enum Ablate : int { kAblateNone = 0, kAblateWorkOnly = 1, kAblateSyncOnly = 2 };

__host__ __device__ inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
__host__ __device__ inline size_t ceil_div(size_t x, size_t a) { return (x + a - 1) / a; }

}  // namespace ccl
