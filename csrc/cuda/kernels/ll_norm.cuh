// Low-latency ("LL") exchange of small rows between the ranks of a communicator, and the
// residual-add + RMSNorm that consumes them.
//
// Every 16-byte store into an LL slot is {payload, epoch, payload, epoch}: 8 bytes of data and
// two copies of the round's flag value. The receiver polls the data words themselves, so a row
// needs no release fence and no separate flag: it is complete when every one of its 16-byte units
// carries the flag of the round. Slot [parity][source rank] of the receiving rank's LL region
// holds the source's rows in row-major order at twice their plain byte offset.
//
// The consumer issues the loads of ALL source ranks for one 16-byte payload vector before it
// looks at any flag, so in the common case (data already there) a vector costs one round trip
// to L2 instead of one per source.
#pragma once
#include "comm.cuh"

namespace ccl {

constexpr int kLLNormMaxVec = 6;   // 16-byte vectors of one row per thread (hidden <= 6 * 8 * blockDim)

template <typename T> __device__ __forceinline__ T ll_round_to(float v);
template <> __device__ __forceinline__ __nv_bfloat16 ll_round_to<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half ll_round_to<__half>(float v) { return __float2half(v); }

__device__ __forceinline__ void report_timeout(const RankCtx& ctx, int peer, int phase) {
  const int code = comm_aborted(ctx) ? kStatusAborted : kStatusTimeout;
  if (ctx.status && atomicCAS(ctx.status, kStatusOk, code) == kStatusOk) {
    ctx.status[1] = ctx.rank;
    ctx.status[2] = peer;
    ctx.status[3] = phase;
    __threadfence_system();
  }
}

__device__ __forceinline__ char* ll_slot(const RankCtx& ctx, int dst_rank, int parity, int src_rank) {
  return ctx.ll[dst_rank] + ((size_t)parity * kMaxRanks + src_rank) * kLLSlotBytes;
}

// Writes 8 payload bytes (w0, w1) of `payload_off` (a multiple of 8) into the slot.
__device__ __forceinline__ void ll_store8(char* slot, size_t payload_off, uint32_t w0, uint32_t w1, uint32_t flag) {
  ptx::st_v4(slot + payload_off * 2, make_uint4(w0, flag, w1, flag));
}

__device__ __forceinline__ bool ll_ready(const uint4& a, const uint4& b, uint32_t flag) {
  return a.y == flag && a.w == flag && b.y == flag && b.w == flag;
}

// Where a row's own-rank contribution comes from.
enum LLOwn : int {
  kOwnInSlot = 0,   // the producer pushed it into this rank's slot like every peer's (x_row unused)
  kOwnPtr = 1,      // plain memory at x_row (null = a row of zeros); peers come from the slots
  kLocalOnly = 2,   // no exchange at all: the row is x_row (null = zeros); single-rank communicators
};

// Sum over ranks (in rank order, fp32) of payload vector `vec_off` (byte offset of a 16-byte
// vector inside the row-major payload) as received in this rank's LL slots. With own_in_slot
// false the own rank's contribution is read from `own` (null = zeros) instead of from the slot.
// Returns false if a source did not deliver within the wait budget (reported in the status word).
template <typename T, int BATCH = kMaxRanks>
__device__ __forceinline__ bool ll_gather_sum(const RankCtx& ctx, int parity, uint32_t flag, size_t vec_off,
                                              bool own_in_slot, const char* own, float (&acc)[8]) {
  static_assert(kMaxRanks % BATCH == 0, "BATCH must divide the rank limit");
  const int W = ctx.world, me = ctx.rank;
  const char* base = ll_slot(ctx, me, parity, 0) + vec_off * 2;
  bool ok = true;
  // BATCH source ranks are in flight at a time (2 * BATCH 16-byte registers per thread); kernels
  // with a tight register budget use a smaller batch at the price of one more round trip.
#pragma unroll
  for (int b0 = 0; b0 < kMaxRanks; b0 += BATCH) {
    if (b0 < W) {
      uint4 s[2 * BATCH];
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        const int p = b0 + q;
        if (p < W && (own_in_slot || p != me)) {
          s[2 * q] = ptx::ld_volatile_v4(base + (size_t)p * kLLSlotBytes);
          s[2 * q + 1] = ptx::ld_volatile_v4(base + (size_t)p * kLLSlotBytes + 16);
        }
      }
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        const int p = b0 + q;
        if (p < W && (own_in_slot || p != me)) {
          if (!ll_ready(s[2 * q], s[2 * q + 1], flag)) {
            const uint64_t t0 = ptx::globaltimer_ns();
            uint32_t it = 0;
            while (true) {
              s[2 * q] = ptx::ld_volatile_v4(base + (size_t)p * kLLSlotBytes);
              s[2 * q + 1] = ptx::ld_volatile_v4(base + (size_t)p * kLLSlotBytes + 16);
              if (ll_ready(s[2 * q], s[2 * q + 1], flag)) break;
              if ((++it & 63u) == 0 && (ptx::globaltimer_ns() - t0 > ctx.spin_ns || ((it & 1023u) == 0 && comm_aborted(ctx)))) {
                report_timeout(ctx, p, 0);
                ok = false;
                break;
              }
            }
          }
        }
      }
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        const int p = b0 + q;
        if (p < W) {
          Vec<T> v;
          if (!own_in_slot && p == me)
            *reinterpret_cast<uint4*>(&v) = own ? *reinterpret_cast<const uint4*>(own) : make_uint4(0, 0, 0, 0);
          else
            *reinterpret_cast<uint4*>(&v) = make_uint4(s[2 * q].x, s[2 * q].z, s[2 * q + 1].x, s[2 * q + 1].z);
#pragma unroll
          for (int t = 0; t < 8; ++t) acc[t] = (p == 0) ? to_acc(v.v[t]) : acc[t] + to_acc(v.v[t]);
        }
      }
    }
  }
  return ok;
}

// Block-wide sum; s_red needs 33 floats. All threads of the CTA must call it.
__device__ __forceinline__ float block_sum(float v, float* s_red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < (blockDim.x + 31) / 32) ? s_red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) s_red[32] = t;
  }
  __syncthreads();
  return s_red[32];
}

// A row is finished in three steps so that the caller can choose how wide the sum of squares is
// reduced (one CTA, or the CTAs of a cluster that share the row):
//   1. ll_row_gather_add:  h = round(round(sum over ranks) + residual); residual <- h; returns this
//      thread's part of sum(h^2). Vectors [v0, v1) of the row, vector v0 + threadIdx.x + k * blockDim.x
//      in slot k of `hn`.
//   2. the caller reduces the partial sums and forms rstd = rsqrt(mean(h^2) + eps);
//   3. ll_row_write_norm:  out = round(round(h * rstd) * weight).
// The rounding points are those of the unfused sequence all_reduce -> add -> rmsnorm in the tensor
// dtype. `mode` / `x_row`: see LLOwn. `res_in_row` null means a zero residual that is not read.
template <typename T, int MV, int BATCH = kMaxRanks>
__device__ __forceinline__ float ll_row_gather_add(const RankCtx& ctx, int parity, uint32_t flag, int mode,
                                                   size_t row_off /* byte offset of the row in the payload */, int v0, int v1,
                                                   const char* x_row, const char* res_in_row, char* res_out_row,
                                                   Vec<T> (&hn)[MV], bool* ok_out) {
  float ss = 0.f;
  bool ok = true;
#pragma unroll
  for (int k = 0; k < MV; ++k) {
    const int i = v0 + threadIdx.x + k * blockDim.x;
    if (i < v1) {
      float acc[8];
      if (mode != kLocalOnly) {
        ok = ll_gather_sum<T, BATCH>(ctx, parity, flag, row_off + (size_t)i * 16, mode == kOwnInSlot,
                                     x_row ? x_row + (size_t)i * 16 : nullptr, acc) && ok;
      } else {
        Vec<T> v;
        *reinterpret_cast<uint4*>(&v) = x_row ? *reinterpret_cast<const uint4*>(x_row + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int t = 0; t < 8; ++t) acc[t] = to_acc(v.v[t]);
      }
      Vec<T> r;
      if (res_in_row) *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(res_in_row + (size_t)i * 16);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float s = to_acc(ll_round_to<T>(acc[t]));                                   // all_reduce output, rounded
        const T hr = res_in_row ? ll_round_to<T>(s + to_acc(r.v[t])) : ll_round_to<T>(s);  // residual add, rounded
        hn[k].v[t] = hr;
        const float hf = to_acc(hr);
        ss += hf * hf;
      }
      *reinterpret_cast<uint4*>(res_out_row + (size_t)i * 16) = *reinterpret_cast<const uint4*>(&hn[k]);
    }
  }
  if (ok_out) *ok_out = ok;
  return ss;
}

template <typename T, int MV>
__device__ __forceinline__ void ll_row_write_norm(const Vec<T> (&hn)[MV], const Vec<T> (&wv)[MV], float rstd, int v0, int v1,
                                                  char* out_row) {
#pragma unroll
  for (int k = 0; k < MV; ++k) {
    const int i = v0 + threadIdx.x + k * blockDim.x;
    if (i < v1) {
      Vec<T> o;
#pragma unroll
      for (int t = 0; t < 8; ++t) o.v[t] = ll_round_to<T>(to_acc(ll_round_to<T>(to_acc(hn[k].v[t]) * rstd)) * to_acc(wv[k].v[t]));
      *reinterpret_cast<uint4*>(out_row + (size_t)i * 16) = *reinterpret_cast<const uint4*>(&o);
    }
  }
}

// One CTA finishes one whole row.
template <typename T, int MV, int BATCH = kMaxRanks>
__device__ __forceinline__ bool ll_row_residual_norm(const RankCtx& ctx, int parity, uint32_t flag, int mode, size_t row_off,
                                                     int hidden, const char* x_row, const char* res_in_row,
                                                     char* res_out_row, char* out_row, const Vec<T> (&wv)[MV],
                                                     float eps, float* s_red) {
  Vec<T> hn[MV];   // the new residual row, kept in the tensor dtype (half the registers of fp32)
  bool ok = true;
  const float ss = ll_row_gather_add<T, MV, BATCH>(ctx, parity, flag, mode, row_off, 0, hidden / 8, x_row, res_in_row, res_out_row, hn, &ok);
  const float rstd = rsqrtf(block_sum(ss, s_red) / (float)hidden + eps);
  ll_row_write_norm<T, MV>(hn, wv, rstd, 0, hidden / 8, out_row);
  return ok;
}

// Vectors [v0, v1) of the norm weight, laid out like `hn` above.
template <typename T, int MV>
__device__ __forceinline__ void ll_load_norm_weight(const void* wgt, int v0, int v1, Vec<T> (&wv)[MV]) {
#pragma unroll
  for (int k = 0; k < MV; ++k) {
    const int i = v0 + threadIdx.x + k * blockDim.x;
    if (i < v1) *reinterpret_cast<uint4*>(&wv[k]) = *reinterpret_cast<const uint4*>(static_cast<const char*>(wgt) + (size_t)i * 16);
  }
}

}  // namespace ccl
