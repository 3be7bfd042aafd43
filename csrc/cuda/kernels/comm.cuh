// Device-side communicator view and the signalling protocol shared by every collective kernel.
//
// Each rank owns one *arena* (peer-mapped on every other rank of the communicator):
//
//     [ data half 0 | data half 1 | flags | state ]
//
// * data halves: staging space, used alternately ("parity") by consecutive rounds so that a fast
//   rank can start round k+1 while a slow rank still reads round k. A rank can never be two
//   rounds ahead because every round makes each rank wait for every other rank at least once.
// * flags: uint32 words indexed [phase][source rank][CTA]. They carry *monotonic epochs*: a word
//   is only ever written with increasing values and never reset, so there is no reset race and
//   a kernel can be replayed from a CUDA graph. CTA b of one rank only ever synchronises with
//   CTA b of the other ranks, so no grid-wide co-residency is needed.
// * state: the rank's epoch counter (read by every CTA at kernel start, advanced by the last
//   CTA to finish) and the completion ticket.
//
// The intel/torch-ccl prototype kernels signal with atomic counters that are reset one slot
// ahead inside a triple buffer (src/gpu/allreduce_small.h:193-285); the epoch scheme replaces
// that. Every wait is bounded by `spin_ns`; on expiry the kernel writes an error record to
// `status` (host-visible), stops synchronising and returns normally.
//
// Emulation: when launched with gridDim.y == world on ONE GPU, blockIdx.y selects the rank
// context from a device table, so a single (cooperative) launch plays all ranks. That is how
// the kernels are exercised on a single GPU.
#pragma once
#include "comm_types.h"
#include "ptx.cuh"

namespace ccl {

__device__ __forceinline__ uint32_t* flag_ptr(uint32_t* base, int phase, int src, int blk) {
  return base + ((size_t)phase * kMaxRanks + src) * kMaxBlocks + blk;
}

// Checked staging accesses (build with -DCCL_DEBUG_BOUNDS=1; compute-sanitizer's stand-in for
// the one class of bug it would catch here, a staging offset outside the arenas). Every
// load_stage / store_stage first checks that its 16 bytes lie inside the data halves or the
// low-latency region of SOME rank's arena of the communicator the CTA works on. A bad access is
// not performed: the first one is recorded in the host-visible status word as
// {kStatusBounds, rank, low 31 bits of the address >> 4, is_store} and the load returns zeros.
// The communicator then reports the error like an expired wait. Costs a few instructions per
// access, so it is a separate build.
#if defined(CCL_DEBUG_BOUNDS) && CCL_DEBUG_BOUNDS
#define CCL_BOUNDS_CHECKED 1
static __shared__ const RankCtx* s_dbg_ctx;
__device__ __forceinline__ void dbg_bounds_bind(const RankCtx* c) { s_dbg_ctx = c; }  // one thread, before a barrier
__device__ __forceinline__ bool dbg_in_bounds(const void* ptr, int is_store) {
  const RankCtx* c = s_dbg_ctx;
  if (!c) return true;
  const char* p = static_cast<const char*>(ptr);
  bool ok = false;
  for (int r = 0; r < c->world; ++r) {
    ok = ok || (p >= c->data[r] && p + 16 <= c->data[r] + 2 * c->half_bytes);
    ok = ok || (c->ll[r] && p >= c->ll[r] && p + 16 <= c->ll[r] + kLLBytes);
  }
  if (!ok && c->status && atomicCAS(c->status, kStatusOk, kStatusBounds) == kStatusOk) {
    c->status[1] = c->rank;
    c->status[2] = (int)((reinterpret_cast<uintptr_t>(ptr) >> 4) & 0x7fffffff);
    c->status[3] = is_store;
    __threadfence_system();
  }
  return ok;
}
#else
#define CCL_BOUNDS_CHECKED 0
#endif

// True once the host has asked the communicator's kernels to give up (ProcessGroup abort()).
__device__ __forceinline__ bool comm_aborted(const RankCtx& c) {
  return c.abort_flag != nullptr && *reinterpret_cast<const volatile int*>(c.abort_flag) != 0;
}

// Per-CTA protocol helper.
struct Sync {
  const RankCtx& ctx;
  uint32_t epoch;   // epoch at kernel entry; round i signals with value epoch + i + 1
  int blk;
  bool sync_enabled;
  int* failed;      // shared-memory flag

  __device__ Sync(const RankCtx& c, int* failed_smem, bool enabled)
      : ctx(c), blk(blockIdx.x), sync_enabled(enabled), failed(failed_smem) {
    // programmatic dependent launch: let the next kernel start its prologue, then wait for the
    // kernels before this one (they produced the input and advanced the epoch)
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();
    if (threadIdx.x == 0) {
      *failed = 0;
#if CCL_BOUNDS_CHECKED
      dbg_bounds_bind(&ctx);
#endif
    }
    epoch = ctx.state ? *reinterpret_cast<volatile uint32_t*>(ctx.state) : 0u;
    __syncthreads();
  }

  __device__ __forceinline__ int parity(int round) const { return (epoch + round) & 1; }
  __device__ __forceinline__ char* half(int peer, int round) const {
    return ctx.data[peer] + (size_t)parity(round) * ctx.half_bytes;
  }

  // All of this CTA's prior writes (by any thread) become visible to `peer` CTAs that acquire
  // the flag. Must be called by all threads of the CTA.
  __device__ __forceinline__ void signal_all(int phase, int round) {
    __syncthreads();
    if (sync_enabled && *failed == 0 && threadIdx.x < ctx.world && (int)threadIdx.x != ctx.rank) {
      ptx::st_release_sys(flag_ptr(ctx.flags[threadIdx.x], phase, ctx.rank, blk), epoch + round + 1);
    }
  }
  __device__ __forceinline__ void signal_one(int peer, int phase, int round) {
    __syncthreads();
    if (sync_enabled && *failed == 0 && threadIdx.x == 0 && peer != ctx.rank) {
      ptx::st_release_sys(flag_ptr(ctx.flags[peer], phase, ctx.rank, blk), epoch + round + 1);
    }
  }
  // Wait until every peer's CTA `blk` has signalled (phase, round). All threads must call it.
  // Returns false if the communicator is in a failed state.
  __device__ __forceinline__ bool wait_all(int phase, int round) {
    if (sync_enabled && threadIdx.x < ctx.world && (int)threadIdx.x != ctx.rank && *failed == 0) {
      const uint32_t* f = flag_ptr(ctx.flags[ctx.rank], phase, threadIdx.x, blk);
      if (!ptx::spin_until_epoch(f, epoch + round + 1, ctx.spin_ns, ctx.abort_flag)) report(threadIdx.x, phase);
    }
    __syncthreads();
    return *failed == 0;
  }
  __device__ __forceinline__ bool wait_one(int peer, int phase, int round) {
    if (sync_enabled && threadIdx.x == 0 && peer != ctx.rank && *failed == 0) {
      const uint32_t* f = flag_ptr(ctx.flags[ctx.rank], phase, peer, blk);
      if (!ptx::spin_until_epoch(f, epoch + round + 1, ctx.spin_ns, ctx.abort_flag)) report(peer, phase);
    }
    __syncthreads();
    return *failed == 0;
  }
  __device__ void report(int peer, int phase) {
    *failed = 1;
    const int code = comm_aborted(ctx) ? kStatusAborted : kStatusTimeout;
    if (ctx.status && atomicCAS(ctx.status, kStatusOk, code) == kStatusOk) {
      ctx.status[1] = ctx.rank;
      ctx.status[2] = peer;
      ctx.status[3] = phase;
      __threadfence_system();
    }
  }
  // Advance the rank's epoch by `rounds` once all CTAs of the kernel have finished.
  __device__ __forceinline__ void finish(int rounds) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t t = atomicAdd(ctx.state + 1, 1u);
      if (t == gridDim.x - 1) {
        ctx.state[1] = 0;
        ctx.state[0] = epoch + rounds;
        __threadfence();
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// element helpers: everything is reduced in a wider accumulator type and rounded once
// ---------------------------------------------------------------------------------------------
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <> struct Acc<__half> { using type = float; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }

template <typename T, typename A> __device__ __forceinline__ T from_acc(A v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) { return __float2half(v); }

template <typename A, bool kIsInt = (A(1) / A(2) == A(0))>
struct Combine {
  static __device__ __forceinline__ A apply(int op, A a, A b) {
    switch (op) {
      case kSum: return a + b;
      case kProd: return a * b;
      case kMin: return b < a ? b : a;
      case kMax: return b > a ? b : a;
      default: return a + b;
    }
  }
};
template <typename A>
struct Combine<A, true> {
  static __device__ __forceinline__ A apply(int op, A a, A b) {
    switch (op) {
      case kSum: return a + b;
      case kProd: return a * b;
      case kMin: return b < a ? b : a;
      case kMax: return b > a ? b : a;
      case kBand: return a & b;
      case kBor: return a | b;
      case kBxor: return a ^ b;
      default: return a + b;
    }
  }
};

template <typename T>
__device__ __forceinline__ T zero_of() {
  T z;
  unsigned char* b = reinterpret_cast<unsigned char*>(&z);
#pragma unroll
  for (int i = 0; i < (int)sizeof(T); ++i) b[i] = 0;
  return z;
}

// A 16-byte vector of T.
template <typename T>
struct alignas(16) Vec {
  static constexpr int kN = 16 / sizeof(T);
  T v[kN];
};

// Load vector `i` (16-byte units) of a `count`-element array that may be unaligned or end in a
// partial vector. `aligned` is true when base is 16-byte aligned.
template <typename T>
__device__ __forceinline__ Vec<T> load_vec(const T* base, size_t i, size_t count, bool aligned) {
  constexpr int N = Vec<T>::kN;
  Vec<T> r;
  if (aligned && (i + 1) * N <= count) {
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(base + i * N);
  } else {
    // unaligned base or ragged tail: rare, kept as a rolled loop to stay small
#pragma unroll 1
    for (int j = 0; j < N; ++j) r.v[j] = (i * N + j < count) ? base[i * N + j] : zero_of<T>();
  }
  return r;
}
template <typename T>
__device__ __forceinline__ void store_vec(T* base, size_t i, size_t count, bool aligned, const Vec<T>& r) {
  constexpr int N = Vec<T>::kN;
  if (aligned && (i + 1) * N <= count) {
    *reinterpret_cast<uint4*>(base + i * N) = *reinterpret_cast<const uint4*>(&r);
  } else {
#pragma unroll 1
    for (int j = 0; j < N; ++j)
      if (i * N + j < count) base[i * N + j] = r.v[j];
  }
}
// Staging accesses are always whole, aligned vectors. Loads bypass L1 and are system-coherent
// (the data was written by another GPU); stores are plain (released by the flag write).
template <typename T>
__device__ __forceinline__ Vec<T> load_stage(const void* p) {
  Vec<T> r;
#if CCL_BOUNDS_CHECKED
  if (!dbg_in_bounds(p, 0)) {
    *reinterpret_cast<uint4*>(&r) = make_uint4(0, 0, 0, 0);
    return r;
  }
#endif
  *reinterpret_cast<uint4*>(&r) = ptx::ld_relaxed_sys_v4(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void store_stage(void* p, const Vec<T>& r) {
#if CCL_BOUNDS_CHECKED
  if (!dbg_in_bounds(p, 1)) return;
#endif
  ptx::st_v4(p, *reinterpret_cast<const uint4*>(&r));
}


}  // namespace ccl
