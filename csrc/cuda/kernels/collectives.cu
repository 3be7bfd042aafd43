// Peer-memory collective kernels for sm_100a (NVLink 5 / NVSwitch): one-shot and two-shot
// all_reduce, reduce(-to-root), reduce_scatter (with fused scale and bf16->fp32 cast),
// all_gather (pull and push), all_to_all(v) with on-device round agreement, rooted
// broadcast / gather / scatter, barrier, and the fused all_reduce + residual-add + RMSNorm used
// by tensor-parallel decode.
//
// These replace the two SYCL-ESIMD all-reduce families of intel/torch-ccl
// (src/gpu/allreduce_small.h:140-381 one-shot; src/gpu/allreduce.h:305-533 hierarchical
// two-shot, 9 kernels per chunk) and every oneCCL call site of src/gpu/dpcpp_ccl.cpp. NVSwitch
// is uniform, so the reference's card/tile hierarchy collapses into flat shards, its single-
// thread sync kernels become in-kernel epoch flags, and accumulation is fp32 instead of fp16.
//
// Data movement: user buffers are not peer-mapped, so data crosses NVLink through the arenas
// (see comm.cuh). Pushes are plain 16-byte stores into the peer's arena followed by a
// release flag; pulls are system-coherent 16-byte loads from the peer's arena after an acquire.
#include "collectives.h"
#include "comm.cuh"
#include "ll_norm.cuh"
#include "gemm.h"

#include <cstdio>

namespace ccl {
namespace {

template <bool EMU>
struct Launch {
  RankCtx ctx;
  CollArgs args;
  const RankCtx* ctx_table;
  const CollArgs* args_table;
};

struct Range { size_t j0, j1; };
__device__ __forceinline__ Range sub_slice(size_t len) {
  const size_t per = ceil_div(len, (size_t)gridDim.x);
  size_t j0 = (size_t)blockIdx.x * per;
  if (j0 > len) j0 = len;
  size_t j1 = j0 + per;
  if (j1 > len) j1 = len;
  return {j0, j1};
}
__device__ __forceinline__ size_t clamp_len(size_t total, size_t begin, size_t cap) {
  if (begin >= total) return 0;
  const size_t r = total - begin;
  return r < cap ? r : cap;
}
__device__ __forceinline__ bool is_aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// user memory (piece of `count` elements, vector index base `vbase`) -> staging
template <typename T>
__device__ __forceinline__ void copy_user_to_stage(const T* src, size_t count, size_t vbase,
                                                   char* stage, Range r) {
  const bool al = is_aligned16(src);
  const size_t nt = blockDim.x;
  size_t j = r.j0 + threadIdx.x;
  for (; j + 3 * nt < r.j1; j += 4 * nt) {
    Vec<T> a = load_vec(src, vbase + j, count, al);
    Vec<T> b = load_vec(src, vbase + j + nt, count, al);
    Vec<T> c = load_vec(src, vbase + j + 2 * nt, count, al);
    Vec<T> d = load_vec(src, vbase + j + 3 * nt, count, al);
    store_stage(stage + j * 16, a);
    store_stage(stage + (j + nt) * 16, b);
    store_stage(stage + (j + 2 * nt) * 16, c);
    store_stage(stage + (j + 3 * nt) * 16, d);
  }
  for (; j < r.j1; j += nt) store_stage(stage + j * 16, load_vec(src, vbase + j, count, al));
}
// staging -> user memory
template <typename T>
__device__ __forceinline__ void copy_stage_to_user(const char* stage, T* dst, size_t count,
                                                   size_t vbase, Range r) {
  const bool al = is_aligned16(dst);
  const size_t nt = blockDim.x;
  size_t j = r.j0 + threadIdx.x;
  for (; j + 3 * nt < r.j1; j += 4 * nt) {
    Vec<T> a = load_stage<T>(stage + j * 16);
    Vec<T> b = load_stage<T>(stage + (j + nt) * 16);
    Vec<T> c = load_stage<T>(stage + (j + 2 * nt) * 16);
    Vec<T> d = load_stage<T>(stage + (j + 3 * nt) * 16);
    store_vec(dst, vbase + j, count, al, a);
    store_vec(dst, vbase + j + nt, count, al, b);
    store_vec(dst, vbase + j + 2 * nt, count, al, c);
    store_vec(dst, vbase + j + 3 * nt, count, al, d);
  }
  for (; j < r.j1; j += nt) store_vec(dst, vbase + j, count, al, load_stage<T>(stage + j * 16));
}
// user -> user
template <typename T>
__device__ __forceinline__ void copy_user_to_user(const T* src, T* dst, size_t count, size_t vbase,
                                                  Range r) {
  if (src == dst) return;
  const bool als = is_aligned16(src), ald = is_aligned16(dst);
  for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x)
    store_vec(dst, vbase + j, count, ald, load_vec(src, vbase + j, count, als));
}

// Peer-parallel copies: the transfers to / from all peers advance together, so a thread has one
// independent load per peer in flight instead of walking the peers one after the other (the
// per-peer latency, not the bandwidth, dominates mid-sized messages). Used when every peer's
// share has the same length (the equal-split case); `F(q)` describes peer number q = 0..np-1 and
// is evaluated inside fully unrolled loops, so nothing is indexed dynamically and everything
// stays in registers. Long or uneven shares stream one peer after the other instead.
constexpr int kNP = kMaxRanks - 1;
template <typename T>
struct PeerDesc {
  T* user;        // user-memory array (source of a push, destination of a pull)
  size_t count;   // its element count
  size_t vbase;   // vector offset of the transfer in it
  char* stage;    // staging address of vector 0 of the transfer
};

template <typename T, typename F>
__device__ __forceinline__ void push_uniform(int np, Range r, F desc) {
  for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
    Vec<T> v[kNP];
#pragma unroll
    for (int q = 0; q < kNP; ++q) {
      if (q < np) {
        const PeerDesc<T> d = desc(q);
        v[q] = load_vec(d.user, d.vbase + j, d.count, is_aligned16(d.user));
      }
    }
#pragma unroll
    for (int q = 0; q < kNP; ++q) {
      if (q < np) {
        const PeerDesc<T> d = desc(q);
        store_stage(d.stage + j * 16, v[q]);
      }
    }
  }
}

template <typename T, typename F>
__device__ __forceinline__ void pull_uniform(int np, Range r, F desc) {
  for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
    Vec<T> v[kNP];
#pragma unroll
    for (int q = 0; q < kNP; ++q) {
      if (q < np) {
        const PeerDesc<T> d = desc(q);
        v[q] = load_stage<T>(d.stage + j * 16);
      }
    }
#pragma unroll
    for (int q = 0; q < kNP; ++q) {
      if (q < np) {
        const PeerDesc<T> d = desc(q);
        store_vec(d.user, d.vbase + j, d.count, is_aligned16(d.user), v[q]);
      }
    }
  }
}

// `len(q)` is the share length of peer q in vectors. Short equal shares go peer-parallel.
template <typename T, typename F, typename L>
__device__ __forceinline__ void push_auto(int np, F desc, L len) {
  const size_t l0 = len(0);
  bool uniform = true;
  for (int q = 1; q < np; ++q) uniform &= (len(q) == l0);
  const Range r0 = sub_slice(l0);
  if (uniform && (r0.j1 - r0.j0) <= 2 * (size_t)blockDim.x) {
    push_uniform<T>(np, r0, desc);
  } else {
    for (int q = 0; q < np; ++q) {
      const PeerDesc<T> d = desc(q);
      copy_user_to_stage(const_cast<const T*>(d.user), d.count, d.vbase, d.stage, sub_slice(len(q)));
    }
  }
}
template <typename T, typename F, typename L>
__device__ __forceinline__ void pull_auto(int np, F desc, L len) {
  const size_t l0 = len(0);
  bool uniform = true;
  for (int q = 1; q < np; ++q) uniform &= (len(q) == l0);
  const Range r0 = sub_slice(l0);
  if (uniform && (r0.j1 - r0.j0) <= 2 * (size_t)blockDim.x) {
    pull_uniform<T>(np, r0, desc);
  } else {
    for (int q = 0; q < np; ++q) {
      const PeerDesc<T> d = desc(q);
      copy_stage_to_user(d.stage, d.user, d.count, d.vbase, sub_slice(len(q)));
    }
  }
}

template <typename T>
__device__ __forceinline__ Vec<T> finish_vec(const typename Acc<T>::type (&acc)[Vec<T>::kN],
                                             const CollArgs& a) {
  using A = typename Acc<T>::type;
  Vec<T> r;
#pragma unroll
  for (int t = 0; t < Vec<T>::kN; ++t) {
    A v = acc[t];
    if (a.has_scale == 1) v = static_cast<A>(v * static_cast<A>(a.scale));        // floating types
    else if (a.has_scale == 2) v = static_cast<A>(v / static_cast<A>(a.scale));   // integer average
    r.v[t] = from_acc<T, A>(v);
  }
  return r;
}

// acc = v(0) (op) v(1) (op) ... in rank order, where `load(p)` returns rank p's vector. The loads
// go out in groups of kReduceBatch ranks (all loads of a group are issued before the first is
// used): 8 vectors in flight at once cost 32 registers and made the 512-thread kernels spill.
// The SUM case, by far the most common, avoids the per-element dispatch on the reduce kind.
// The one-shot kernel, whose whole point is latency, keeps all ranks in flight for the types that
// fit (one round trip to L2 instead of two).
constexpr int kReduceBatch = 4;
template <typename T>
constexpr int kOneshotBatch = (sizeof(T) >= 4 || std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value) ? kMaxRanks : kReduceBatch;
template <typename T, int BATCH = kReduceBatch, typename F>
__device__ __forceinline__ void reduce_ranks(int W, int op, typename Acc<T>::type (&acc)[Vec<T>::kN], F load) {
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  static_assert(kMaxRanks % BATCH == 0, "the batch must divide the rank limit");
#pragma unroll
  for (int b0 = 0; b0 < kMaxRanks; b0 += BATCH) {
    if (b0 < W) {
      Vec<T> v[BATCH];
#pragma unroll
      for (int q = 0; q < BATCH; ++q)
        if (b0 + q < W) v[q] = load(b0 + q);
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        if (b0 + q < W) {
          if (b0 + q == 0) {
#pragma unroll
            for (int t = 0; t < N; ++t) acc[t] = to_acc(v[q].v[t]);
          } else if (op == kSum) {
#pragma unroll
            for (int t = 0; t < N; ++t) acc[t] = acc[t] + to_acc(v[q].v[t]);
          } else {
#pragma unroll
            for (int t = 0; t < N; ++t) acc[t] = Combine<A>::apply(op, acc[t], to_acc(v[q].v[t]));
          }
        }
      }
    }
  }
}

#define CCL_GET_CTX                                                        \
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;              \
  const CollArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;             \
  __shared__ int s_failed;                                                 \
  Sync sy(ctx, &s_failed, a.ablate != kAblateWorkOnly);                    \
  const bool do_work = a.ablate != kAblateSyncOnly;                        \
  (void)do_work;

// ---------------------------------------------------------------------------------------------
// all_reduce, one-shot: push the whole message to every peer, then everyone reduces everything.
// Latency-optimal: one NVLink traversal plus one flag.
// ---------------------------------------------------------------------------------------------
template <typename T, bool EMU>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  const T* in = reinterpret_cast<const T*>(a.in);
  T* out = reinterpret_cast<T*>(a.out);
  const size_t count = a.count;
  const size_t nvec = ceil_div(count, (size_t)N);
  const size_t slot = round_up(nvec * 16, 128);
  const Range r = sub_slice(nvec);
  const bool al_in = is_aligned16(in), al_out = is_aligned16(out);
  const int W = ctx.world, me = ctx.rank;

  if (do_work) {
    for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
      const Vec<T> x = load_vec(in, j, count, al_in);
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p) {
        if (p < W && p != me) store_stage(sy.half(p, 0) + (size_t)me * slot + j * 16, x);
      }
    }
  }
  sy.signal_all(0, 0);
  const bool ok = sy.wait_all(0, 0);
  if (do_work && ok) {
    const char* mine = sy.half(me, 0);
    for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
      A acc[N];
      reduce_ranks<T, kOneshotBatch<T>>(W, a.op, acc, [&](int p) {
        return (p == me) ? load_vec(in, j, count, al_in) : load_stage<T>(mine + (size_t)p * slot + j * 16);
      });
      store_vec(out, j, count, al_out, finish_vec<T>(acc, a));
    }
  }
  sy.finish(1);
}

// ---------------------------------------------------------------------------------------------
// all_reduce, two-shot (also reduce-to-root when args.root >= 0): push shard p of the input to
// rank p (reduce-scatter phase), reduce the own shard, then pull the other reduced shards from
// the peers (all-gather phase). Bandwidth-optimal: each byte crosses NVLink 2(W-1)/W times.
// Large messages run as several rounds through the double-buffered arena inside ONE launch.
// ---------------------------------------------------------------------------------------------
template <typename T, bool EMU>
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  const T* in = reinterpret_cast<const T*>(a.in);
  T* out = reinterpret_cast<T*>(a.out);
  const size_t count = a.count;
  const size_t nvec = ceil_div(count, (size_t)N);
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;          // vectors per shard slot
  const size_t cv = stride_v * W;                // vectors per round
  const int rounds = (int)ceil_div(nvec, cv);
  const bool al_in = is_aligned16(in), al_out = is_aligned16(out);
  const bool gather_here = (a.root < 0) || (a.root == me);

  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t base = (size_t)rd * cv;
    const size_t n = clamp_len(nvec, base, cv);
    const size_t spr = ceil_div(n, (size_t)W);
    // phase 0: scatter my contribution to each shard's owner
    if (do_work) {
      auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
      push_auto<T>(W - 1,
          [&](int q) {
            const int p = peer(q);
            return PeerDesc<T>{const_cast<T*>(in), count, base + (size_t)p * spr, sy.half(p, rd) + (size_t)me * stride_v * 16};
          },
          [&](int q) { return clamp_len(n, (size_t)peer(q) * spr, spr); });
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    // reduce my shard
    const size_t mylen = clamp_len(n, (size_t)me * spr, spr);
    char* regionA = sy.half(me, rd);
    char* regionB = regionA + (size_t)W * stride_v * 16;
    if (do_work) {
      const Range r = sub_slice(mylen);
      const size_t vb = base + (size_t)me * spr;
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        A acc[N];
        reduce_ranks<T>(W, a.op, acc, [&](int p) {
          return (p == me) ? load_vec(in, vb + j, count, al_in) : load_stage<T>(regionA + ((size_t)p * stride_v + j) * 16);
        });
        const Vec<T> res = finish_vec<T>(acc, a);
        store_stage(regionB + j * 16, res);
        if (gather_here) store_vec(out, vb + j, count, al_out, res);
      }
    }
    // phase 1: publish the reduced shard; gatherers pull the others
    sy.signal_all(1, rd);
    if (gather_here) {
      ok = sy.wait_all(1, rd);
      if (!ok) break;
      if (do_work) {
        auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
        pull_auto<T>(W - 1,
            [&](int q) {
              const int p = peer(q);
              return PeerDesc<T>{out, count, base + (size_t)p * spr, sy.half(p, rd) + (size_t)W * stride_v * 16};
            },
            [&](int q) { return clamp_len(n, (size_t)peer(q) * spr, spr); });
      }
    }
  }
  sy.finish(rounds);
}

// ---------------------------------------------------------------------------------------------
// all_reduce (SUM) through an NVLink multicast object (NVLS). Every rank stages its input in its
// OWN arena half; rank r then reduces shard r inside the switch - one multimem.ld_reduce reads
// the same offset of every rank's arena and returns the fp32-accumulated sum - and writes the
// result into all arenas at once with multimem.st; finally everyone copies the whole result out
// of its own arena. Each GPU sends S/W bytes up and receives S bytes down instead of moving
// 2S(W-1)/W through its own load/store units, which is what the two-shot kernel cannot match at
// large sizes. CTA b of a rank stages sub-slice b of EVERY shard, so that (shard r, slice b) on
// all ranks is produced by CTAs number b: the per-CTA flag pairing of comm.cuh stays sufficient.
//
// EMU (all ranks on one GPU, no multicast object): the two multimem operations are played by
// loops over the ranks' arenas with the same fp32-accumulate / round-once arithmetic, which
// checks every index of the kernel on a single GPU.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Multimem;
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) { return ptx::multimem_ld_reduce_add_bf16x2(p); }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) { return ptx::multimem_ld_reduce_add_f16x2(p); }
};
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) { return ptx::multimem_ld_reduce_add_f32(p); }
};

template <typename T, bool EMU>
__global__ void __launch_bounds__(512) allreduce_nvls_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  const T* in = reinterpret_cast<const T*>(a.in);
  T* out = reinterpret_cast<T*>(a.out);
  const size_t count = a.count;
  const size_t nvec = ceil_div(count, (size_t)N);
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;  // vectors per shard slot
  const size_t cv = stride_v * W;        // vectors per round
  const int rounds = (int)ceil_div(nvec, cv);

  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t base = (size_t)rd * cv;
    const size_t n = clamp_len(nvec, base, cv);
    const size_t spr = ceil_div(n, (size_t)W);
    char* mine = sy.half(me, rd);
    if (do_work) {
      for (int s = 0; s < W; ++s) {
        const Range r = sub_slice(clamp_len(n, (size_t)s * spr, spr));
        copy_user_to_stage(in, count, base + (size_t)s * spr, mine + (size_t)s * stride_v * 16, r);
      }
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      const Range r = sub_slice(clamp_len(n, (size_t)me * spr, spr));
      const size_t off0 = (size_t)sy.parity(rd) * ctx.half_bytes + (size_t)me * stride_v * 16;
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        const size_t off = off0 + j * 16;
        Vec<T> v;
        if constexpr (EMU) {
          A acc[N];
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p) {
            if (p < W) {
              const Vec<T> x = load_stage<T>(ctx.data[p] + off);
#pragma unroll
              for (int t = 0; t < N; ++t) acc[t] = (p == 0) ? to_acc(x.v[t]) : acc[t] + to_acc(x.v[t]);
            }
          }
#pragma unroll
          for (int t = 0; t < N; ++t) v.v[t] = from_acc<T, A>(acc[t]);
        } else {
          *reinterpret_cast<uint4*>(&v) = Multimem<T>::ld_reduce(ctx.mc_data + off);
        }
        if (a.has_scale) {
#pragma unroll
          for (int t = 0; t < N; ++t) v.v[t] = from_acc<T, A>(static_cast<A>(to_acc(v.v[t]) * static_cast<A>(a.scale)));
        }
        if constexpr (EMU) {
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)
            if (p < W) store_stage(ctx.data[p] + off, v);
        } else {
          ptx::multimem_st_v4(ctx.mc_data + off, *reinterpret_cast<const uint4*>(&v));
        }
      }
    }
    sy.signal_all(1, rd);
    ok = sy.wait_all(1, rd);
    if (!ok) break;
    if (do_work) {
      for (int s = 0; s < W; ++s) {
        const Range r = sub_slice(clamp_len(n, (size_t)s * spr, spr));
        copy_stage_to_user(mine + (size_t)s * stride_v * 16, out, count, base + (size_t)s * spr, r);
      }
    }
  }
  sy.finish(rounds);
}

// ---------------------------------------------------------------------------------------------
// reduce_scatter (SUM) and all_gather through the multicast object; same staging layout, flag
// pairing and software emulation as allreduce_nvls_kernel.
//  * reduce_scatter: every rank stages all its W pieces in its own arena (piece s in slot s),
//    then reduces slot `me` inside the switch straight into its output.
//  * all_gather: every rank writes its piece into slot `me` of ALL arenas with one multimem.st
//    per vector (the piece leaves the GPU once instead of W-1 times), then copies the other
//    slots out of its own arena.
// ---------------------------------------------------------------------------------------------
template <typename T, bool EMU>
__global__ void __launch_bounds__(512) reduce_scatter_nvls_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;
  const int rounds = a.rounds;
  T* out = reinterpret_cast<T*>(a.out);
  const size_t mycount = a.in_cnt[me];
  const bool al_out = is_aligned16(out);

  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t vb = (size_t)rd * stride_v;
    char* mine = sy.half(me, rd);
    if (do_work) {
      for (int s = 0; s < W; ++s) {
        const size_t cnt = a.in_cnt[s];
        const Range r = sub_slice(clamp_len(ceil_div(cnt, (size_t)N), vb, stride_v));
        copy_user_to_stage(reinterpret_cast<const T*>(a.in_piece[s]), cnt, vb, mine + (size_t)s * stride_v * 16, r);
      }
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      const Range r = sub_slice(clamp_len(ceil_div(mycount, (size_t)N), vb, stride_v));
      const size_t off0 = (size_t)sy.parity(rd) * ctx.half_bytes + (size_t)me * stride_v * 16;
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        const size_t off = off0 + j * 16;
        Vec<T> v;
        if constexpr (EMU) {
          A acc[N];
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p) {
            if (p < W) {
              const Vec<T> x = load_stage<T>(ctx.data[p] + off);
#pragma unroll
              for (int t = 0; t < N; ++t) acc[t] = (p == 0) ? to_acc(x.v[t]) : acc[t] + to_acc(x.v[t]);
            }
          }
#pragma unroll
          for (int t = 0; t < N; ++t) v.v[t] = from_acc<T, A>(acc[t]);
        } else {
          *reinterpret_cast<uint4*>(&v) = Multimem<T>::ld_reduce(ctx.mc_data + off);
        }
        if (a.has_scale) {
#pragma unroll
          for (int t = 0; t < N; ++t) v.v[t] = from_acc<T, A>(static_cast<A>(to_acc(v.v[t]) * static_cast<A>(a.scale)));
        }
        store_vec(out, vb + j, mycount, al_out, v);
      }
    }
  }
  sy.finish(rounds);
}

template <bool EMU>
__global__ void __launch_bounds__(512) all_gather_nvls_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using T = uint8_t;
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;
  const int rounds = a.rounds;
  const T* in = reinterpret_cast<const T*>(a.in);
  const size_t mybytes = a.out_cnt[me];
  const bool al_in = is_aligned16(in);

  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t vb = (size_t)rd * stride_v;
    if (do_work) {
      const Range r = sub_slice(clamp_len(ceil_div(mybytes, (size_t)16), vb, stride_v));
      const size_t off0 = (size_t)sy.parity(rd) * ctx.half_bytes + (size_t)me * stride_v * 16;
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        const Vec<T> v = load_vec(in, vb + j, mybytes, al_in);
        if constexpr (EMU) {
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)
            if (p < W) store_stage(ctx.data[p] + off0 + j * 16, v);
        } else {
          ptx::multimem_st_v4(ctx.mc_data + off0 + j * 16, *reinterpret_cast<const uint4*>(&v));
        }
      }
      copy_user_to_user(in, reinterpret_cast<T*>(a.out_piece[me]), mybytes, vb, r);
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      const char* mine = sy.half(me, rd);
      for (int q = 1; q < W; ++q) {
        const int p = (me + q) % W;
        const size_t cnt = a.out_cnt[p];
        const Range r = sub_slice(clamp_len(ceil_div(cnt, (size_t)16), vb, stride_v));
        copy_stage_to_user(mine + (size_t)p * stride_v * 16, reinterpret_cast<T*>(a.out_piece[p]), cnt, vb, r);
      }
    }
  }
  sy.finish(rounds);
}

// ---------------------------------------------------------------------------------------------
// reduce_scatter: rank p receives piece p of every rank and reduces. Pieces may have different
// sizes; TOut may be wider than TIn (bf16 gradients reduced and stored as fp32) and the scale
// (gradient average) is applied in the same pass.
// ---------------------------------------------------------------------------------------------
template <typename TIn, typename TOut, bool EMU>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using A = typename Acc<TIn>::type;
  constexpr int N = Vec<TIn>::kN;
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;
  const int rounds = a.rounds;
  TOut* out = reinterpret_cast<TOut*>(a.out);
  const size_t mycount = a.in_cnt[me];
  const TIn* mypiece = reinterpret_cast<const TIn*>(a.in_piece[me]);
  const bool al_mine = is_aligned16(mypiece);
  const bool al_out = is_aligned16(out);

  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t vb = (size_t)rd * stride_v;
    if (do_work) {
      auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
      push_auto<TIn>(W - 1,
          [&](int q) {
            const int p = peer(q);
            return PeerDesc<TIn>{const_cast<TIn*>(reinterpret_cast<const TIn*>(a.in_piece[p])), (size_t)a.in_cnt[p], vb,
                                 sy.half(p, rd) + (size_t)me * stride_v * 16};
          },
          [&](int q) { return clamp_len(ceil_div((size_t)a.in_cnt[peer(q)], (size_t)N), vb, stride_v); });
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      const size_t nv = ceil_div(mycount, (size_t)N);
      const Range r = sub_slice(clamp_len(nv, vb, stride_v));
      const char* regionA = sy.half(me, rd);
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        A acc[N];
        reduce_ranks<TIn>(W, a.op, acc, [&](int p) {
          return (p == me) ? load_vec(mypiece, vb + j, mycount, al_mine) : load_stage<TIn>(regionA + ((size_t)p * stride_v + j) * 16);
        });
        const size_t e0 = (vb + j) * N;
        if constexpr (sizeof(TOut) == sizeof(TIn)) {
          store_vec(reinterpret_cast<TIn*>(out), vb + j, mycount, al_out, finish_vec<TIn>(acc, a));
        } else {
          // widened output (float): N elements = N*4 bytes
          if (al_out && e0 + N <= mycount) {
#pragma unroll
            for (int t = 0; t < N; t += 4) {
              float4 o;
              o.x = acc[t] * (a.has_scale ? a.scale : 1.f);
              o.y = acc[t + 1] * (a.has_scale ? a.scale : 1.f);
              o.z = acc[t + 2] * (a.has_scale ? a.scale : 1.f);
              o.w = acc[t + 3] * (a.has_scale ? a.scale : 1.f);
              *reinterpret_cast<float4*>(out + e0 + t) = o;
            }
          } else {
#pragma unroll
            for (int t = 0; t < N; ++t)
              if (e0 + t < mycount) out[e0 + t] = static_cast<TOut>(acc[t] * (a.has_scale ? a.scale : 1.f));
          }
        }
      }
    }
  }
  sy.finish(rounds);
}

// ---------------------------------------------------------------------------------------------
// all_gather (bytes). mode 0 (pull): stage the own piece locally, peers read it over NVLink
// straight into their outputs. mode 1 (push): write the own piece into every peer's arena, each
// rank then copies locally (lower latency for small pieces). Pieces may differ in size.
// ---------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(512) all_gather_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using T = uint8_t;
  const int W = ctx.world, me = ctx.rank;
  const size_t stride_v = a.chunk_vecs;
  const int rounds = a.rounds;
  const T* in = reinterpret_cast<const T*>(a.in);
  const size_t mybytes = a.out_cnt[me];
  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t vb = (size_t)rd * stride_v;
    const size_t mylen = clamp_len(ceil_div(mybytes, (size_t)16), vb, stride_v);
    if (do_work) {
      const Range r = sub_slice(mylen);
      if (a.mode == 0) {
        copy_user_to_stage(in, mybytes, vb, sy.half(me, rd), r);
      } else {
        for (int q = 1; q < W; ++q) {
          const int p = (me + q) % W;
          copy_user_to_stage(in, mybytes, vb, sy.half(p, rd) + (size_t)me * stride_v * 16, r);
        }
      }
      copy_user_to_user(in, reinterpret_cast<T*>(a.out_piece[me]), mybytes, vb, r);
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
      pull_auto<T>(W - 1,
          [&](int q) {
            const int p = peer(q);
            return PeerDesc<T>{reinterpret_cast<T*>(a.out_piece[p]), (size_t)a.out_cnt[p], vb,
                               (a.mode == 0) ? sy.half(p, rd) : sy.half(me, rd) + (size_t)p * stride_v * 16};
          },
          [&](int q) { return clamp_len(ceil_div((size_t)a.out_cnt[peer(q)], (size_t)16), vb, stride_v); });
    }
  }
  sy.finish(rounds);
}

// ---------------------------------------------------------------------------------------------
// all_to_all(v) (bytes): piece p of the input goes to rank p. With uneven pieces no rank knows
// the largest pair-wise piece, so round 0 exchanges each rank's largest send size through the
// peers' state words and every CTA derives the same number of data rounds from the maximum.
// ---------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(512) all_to_all_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using T = uint8_t;
  const int W = ctx.world, me = ctx.rank;
  size_t stride_v = a.chunk_vecs;
  int rounds = a.rounds;
  int first = 0;
  bool ok = true;
  if (rounds == 0) {
    // scratch words: state[16 + parity*8 + src] = src's largest piece in 16-byte vectors
    size_t mx = 0;
    for (int p = 0; p < W; ++p) {
      const size_t v = ceil_div((size_t)a.in_cnt[p], (size_t)16);
      mx = v > mx ? v : mx;
    }
    const int par = sy.parity(0);
    if (threadIdx.x < W) {
      // every CTA writes the same value; the peer's CTA b reads after CTA b's flag
      uint32_t* peer_state = reinterpret_cast<uint32_t*>(ctx.flags[threadIdx.x]) + kFlagBytes / 4;
      ptx::st_relaxed_sys(peer_state + 16 + par * kMaxRanks + me, (uint32_t)mx);
    }
    sy.signal_all(3, 0);
    ok = sy.wait_all(3, 0);
    size_t gmx = 0;
    for (int p = 0; p < W; ++p) {
      const size_t v = ptx::ld_relaxed_sys(ctx.state + 16 + par * kMaxRanks + p);
      gmx = v > gmx ? v : gmx;
    }
    // every rank now knows the largest piece of the whole group: pack the slots accordingly
    // (slots tens of MB apart cost more in address translation than the transfer itself)
    const size_t want = round_up(gmx > 8 ? gmx : 8, 8);
    if (want < stride_v) stride_v = want;
    rounds = (int)ceil_div(gmx, stride_v);
    first = 1;
  }
  for (int i = 0; i < rounds && ok; ++i) {
    const int rd = first + i;
    const size_t vb = (size_t)i * stride_v;
    if (do_work) {
      auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
      push_auto<T>(W - 1,
          [&](int q) {
            const int p = peer(q);
            return PeerDesc<T>{const_cast<T*>(reinterpret_cast<const T*>(a.in_piece[p])), (size_t)a.in_cnt[p], vb,
                               sy.half(p, rd) + (size_t)me * stride_v * 16};
          },
          [&](int q) { return clamp_len(ceil_div((size_t)a.in_cnt[peer(q)], (size_t)16), vb, stride_v); });
      const size_t sb = a.in_cnt[me];
      copy_user_to_user(reinterpret_cast<const T*>(a.in_piece[me]), reinterpret_cast<T*>(a.out_piece[me]),
                        sb, vb, sub_slice(clamp_len(ceil_div(sb, (size_t)16), vb, stride_v)));
    }
    sy.signal_all(0, rd);
    ok = sy.wait_all(0, rd);
    if (!ok) break;
    if (do_work) {
      auto peer = [&](int q) { const int p = me + q + 1; return p >= W ? p - W : p; };
      pull_auto<T>(W - 1,
          [&](int q) {
            const int p = peer(q);
            return PeerDesc<T>{reinterpret_cast<T*>(a.out_piece[p]), (size_t)a.out_cnt[p], vb,
                               sy.half(me, rd) + (size_t)p * stride_v * 16};
          },
          [&](int q) { return clamp_len(ceil_div((size_t)a.out_cnt[peer(q)], (size_t)16), vb, stride_v); });
    }
  }
  sy.finish(first + rounds);
}

// ---------------------------------------------------------------------------------------------
// rooted ops (bytes): broadcast, gather, scatter. The root and the other ranks acknowledge each
// round so that nobody can run more than one round ahead of a rank that still reads staging.
//
// Every kernel of this file keeps one invariant: a rank leaves round r only after EVERY rank has
// entered round r. The unrooted kernels get it from their all-to-all flag exchange; gather gets it
// because the root answers only after it has heard from everybody. Broadcast and scatter need a
// third step for it: after the last acknowledgement the root releases the other ranks (phase 2).
// Without the release a non-root rank could finish the round knowing only that the ROOT had
// entered it, get two rounds ahead of a third rank that is still pulling from a peer's staging
// half in an earlier all_gather / two-shot kernel, and (as the root of a later broadcast) overwrite
// that half. tests/native/epoch_model.cpp reproduces exactly that on host threads.
// ---------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(512) rooted_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  using T = uint8_t;
  const int W = ctx.world, me = ctx.rank, root = a.root;
  const size_t stride_v = a.chunk_vecs;
  const int rounds = a.rounds;
  const size_t bytes = a.count;  // per piece
  bool ok = true;
  for (int rd = 0; rd < rounds && ok; ++rd) {
    const size_t vb = (size_t)rd * stride_v;
    const size_t len = clamp_len(ceil_div(bytes, (size_t)16), vb, stride_v);
    const Range r = sub_slice(len);
    if (a.mode == kBroadcast) {
      T* buf = reinterpret_cast<T*>(a.out);
      if (me == root) {
        if (do_work)
          for (int q = 1; q < W; ++q) copy_user_to_stage(buf, bytes, vb, sy.half((me + q) % W, rd), r);
        sy.signal_all(0, rd);
        ok = sy.wait_all(1, rd);
        sy.signal_all(2, rd);  // release, see the note above the kernel
      } else {
        ok = sy.wait_one(root, 0, rd);
        if (ok && do_work) copy_stage_to_user(sy.half(me, rd), buf, bytes, vb, r);
        sy.signal_one(root, 1, rd);
        if (ok) ok = sy.wait_one(root, 2, rd);
      }
    } else if (a.mode == kBroadcastSwitch) {
      // The root stores each vector ONCE into the multicast address: the switch replicates it into
      // every rank's arena (S bytes leave the root instead of (W-1) * S). All ranks exchange flags
      // with all ranks, like the unrooted kernels, so no release step is needed.
      T* buf = reinterpret_cast<T*>(a.out);
      if (me == root && do_work) {
        const size_t off0 = (size_t)sy.parity(rd) * ctx.half_bytes;
        const bool al = is_aligned16(buf);
        for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
          const Vec<T> v = load_vec(const_cast<const T*>(buf), vb + j, bytes, al);
          if constexpr (EMU) {
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
              if (p < W) store_stage(ctx.data[p] + off0 + j * 16, v);
          } else {
            ptx::multimem_st_v4(ctx.mc_data + off0 + j * 16, *reinterpret_cast<const uint4*>(&v));
          }
        }
      }
      sy.signal_all(0, rd);
      ok = sy.wait_all(0, rd);
      if (ok && me != root && do_work) copy_stage_to_user(sy.half(me, rd), buf, bytes, vb, r);
    } else if (a.mode == kGather) {
      const T* in = reinterpret_cast<const T*>(a.in);
      if (me == root) {
        if (do_work) copy_user_to_user(in, reinterpret_cast<T*>(a.out_piece[me]), bytes, vb, r);
        ok = sy.wait_all(0, rd);
        if (ok && do_work)
          for (int q = 1; q < W; ++q) {
            const int p = (me + q) % W;
            copy_stage_to_user(sy.half(me, rd) + (size_t)p * stride_v * 16,
                               reinterpret_cast<T*>(a.out_piece[p]), bytes, vb, r);
          }
        sy.signal_all(1, rd);
      } else {
        if (do_work) copy_user_to_stage(in, bytes, vb, sy.half(root, rd) + (size_t)me * stride_v * 16, r);
        sy.signal_one(root, 0, rd);
        ok = sy.wait_one(root, 1, rd);
      }
    } else {  // scatter
      T* out = reinterpret_cast<T*>(a.out);
      if (me == root) {
        if (do_work) {
          for (int q = 1; q < W; ++q) {
            const int p = (me + q) % W;
            copy_user_to_stage(reinterpret_cast<const T*>(a.in_piece[p]), bytes, vb, sy.half(p, rd), r);
          }
          copy_user_to_user(reinterpret_cast<const T*>(a.in_piece[me]), out, bytes, vb, r);
        }
        sy.signal_all(0, rd);
        ok = sy.wait_all(1, rd);
        sy.signal_all(2, rd);  // release
      } else {
        ok = sy.wait_one(root, 0, rd);
        if (ok && do_work) copy_stage_to_user(sy.half(me, rd), out, bytes, vb, r);
        sy.signal_one(root, 1, rd);
        if (ok) ok = sy.wait_one(root, 2, rd);
      }
    }
  }
  sy.finish(rounds);
}

template <bool EMU>
__global__ void __launch_bounds__(64) barrier_kernel(const __grid_constant__ Launch<EMU> L) {
  CCL_GET_CTX
  sy.signal_all(0, 0);
  sy.wait_all(0, 0);
  sy.finish(1);
}

// ---------------------------------------------------------------------------------------------
// fused all_reduce + residual add + RMSNorm (tensor-parallel decode). One CTA owns whole rows:
// it pushes its rows of the partial sums to every peer, waits for the peers' rows, then adds
// the partials in rank order (fp32), adds the residual, writes the new residual and the
// normalised output. Rounding points match the unfused sequence all_reduce -> add -> rmsnorm.
// ---------------------------------------------------------------------------------------------
template <bool EMU>
struct LaunchNorm {
  RankCtx ctx;
  FusedNormArgs args;
  const RankCtx* ctx_table;
  const FusedNormArgs* args_table;
};

constexpr int kNormMaxVecPerThread = 4;

template <typename T, bool EMU>
__global__ void __launch_bounds__(512) allreduce_residual_rmsnorm_kernel(const __grid_constant__ LaunchNorm<EMU> L) {
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;
  const FusedNormArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;
  __shared__ int s_failed;
  __shared__ float s_red[33];
  Sync sy(ctx, &s_failed, a.ablate != kAblateWorkOnly);
  constexpr int N = 8;
  const int W = ctx.world, me = ctx.rank;
  const int hv = a.hidden / N;  // vectors per row
  const char* x = reinterpret_cast<const char*>(a.x);
  char* res = reinterpret_cast<char*>(a.residual);
  char* out = reinterpret_cast<char*>(a.out);
  const size_t row_bytes = (size_t)a.hidden * sizeof(T);
  const size_t slot = round_up((size_t)a.rows * row_bytes, 128);
  // this rank's contribution to a row: the row itself, or (embedding lookup) a table row / zeros
  auto x_row = [&](int row) -> const char* {
    if (!a.gather_tokens) return x + (size_t)row * row_bytes;
    const long long idx = a.gather_tokens[row] - a.gather_base;
    return (idx >= 0 && idx < a.gather_rows) ? x + (size_t)idx * row_bytes : nullptr;
  };

  const bool ll = a.use_ll != 0 && W > 1;
  const uint32_t llflag = sy.epoch + 1;
  if (ll) {
    // low-latency push: each 16-byte store = {payload, epoch, payload, epoch}; the receiver polls the
    // payload slots themselves, so there is no release fence and no flag round trip
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
      const char* src = x_row(row);
      for (int i = threadIdx.x; i < hv; i += blockDim.x) {
        const size_t off = (size_t)row * row_bytes + (size_t)i * 16;
        const uint4 v = src ? *reinterpret_cast<const uint4*>(src + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p) {
          if (p < W && p != me) {
            char* dst = ll_slot(ctx, p, sy.parity(0), me);
            ll_store8(dst, off, v.x, v.y, llflag);
            ll_store8(dst, off + 8, v.z, v.w, llflag);
          }
        }
      }
    }
  } else if (W > 1 && a.ablate != kAblateSyncOnly) {
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
      const char* src = x_row(row);
      for (int i = threadIdx.x; i < hv; i += blockDim.x) {
        const size_t off = (size_t)row * row_bytes + (size_t)i * 16;
        const uint4 v = src ? *reinterpret_cast<const uint4*>(src + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < W && p != me) ptx::st_v4(sy.half(p, 0) + (size_t)me * slot + off, v);
      }
    }
  }
  bool ok = true;
  if (W > 1 && !ll) {
    sy.signal_all(0, 0);
    ok = sy.wait_all(0, 0);
  }
  if (ok && a.ablate != kAblateSyncOnly) {
    // the norm weights do not depend on the reduction: fetch them first so that their latency
    // overlaps the peer waits and the block reduction
    Vec<T> wv[kNormMaxVecPerThread];
    ll_load_norm_weight<T, kNormMaxVecPerThread>(a.weight, 0, hv, wv);
    if (ll || W == 1) {
      for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
        char* rrow = res + (size_t)row * row_bytes;
        ll_row_residual_norm<T, kNormMaxVecPerThread, 4>(ctx, sy.parity(0), llflag, W == 1 ? kLocalOnly : kOwnPtr, (size_t)row * row_bytes,
                                                      a.hidden, x_row(row), a.zero_residual ? nullptr : rrow, rrow,
                                                      out + (size_t)row * row_bytes, wv, a.eps, s_red);
      }
    } else {
      // larger inputs (prefill): the peers' rows were staged in the data half and published by the flag round
      const char* mine = sy.half(me, 0);
      for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const char* src = x_row(row);
        float h[kNormMaxVecPerThread][N];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < kNormMaxVecPerThread; ++k) {
          const int i = threadIdx.x + k * blockDim.x;
          if (i < hv) {
            const size_t off = (size_t)row * row_bytes + (size_t)i * 16;
            float acc[N];
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p) {
              if (p < W) {
                Vec<T> v;
                if (p == me)
                  *reinterpret_cast<uint4*>(&v) = src ? *reinterpret_cast<const uint4*>(src + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
                else
                  v = load_stage<T>(mine + (size_t)p * slot + off);
#pragma unroll
                for (int t = 0; t < N; ++t) acc[t] = (p == 0) ? to_acc(v.v[t]) : acc[t] + to_acc(v.v[t]);
              }
            }
            Vec<T> r, hn;
            if (!a.zero_residual) *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(res + off);
#pragma unroll
            for (int t = 0; t < N; ++t) {
              const float s = to_acc(ll_round_to<T>(acc[t]));                                        // all_reduce output, rounded
              const T hr = a.zero_residual ? ll_round_to<T>(s) : ll_round_to<T>(s + to_acc(r.v[t]));  // residual add, rounded
              hn.v[t] = hr;
              h[k][t] = to_acc(hr);
              ss += h[k][t] * h[k][t];
            }
            *reinterpret_cast<uint4*>(res + off) = *reinterpret_cast<const uint4*>(&hn);
          }
        }
        const float rstd = rsqrtf(block_sum(ss, s_red) / (float)a.hidden + a.eps);
#pragma unroll
        for (int k = 0; k < kNormMaxVecPerThread; ++k) {
          const int i = threadIdx.x + k * blockDim.x;
          if (i < hv) {
            Vec<T> o;
#pragma unroll
            for (int t = 0; t < N; ++t) o.v[t] = ll_round_to<T>(to_acc(ll_round_to<T>(h[k][t] * rstd)) * to_acc(wv[k].v[t]));
            *reinterpret_cast<uint4*>(out + (size_t)row * row_bytes + (size_t)i * 16) = *reinterpret_cast<const uint4*>(&o);
          }
        }
      }
    }
  }
  if (W > 1) sy.finish(1);
}

// ---------------------------------------------------------------------------------------------
// launch plumbing
// ---------------------------------------------------------------------------------------------
template <typename ArgsT, template <bool> class LT, typename KR, typename KE>
cudaError_t launch_pair(KR kreal, KE kemu, const RankCtx* ctx, const ArgsT* args, const LaunchCfg& cfg) {
  dim3 block(cfg.nthreads);
  if (!cfg.cooperative) {
    LT<false> L;
    L.ctx = *ctx;
    L.args = *args;
    L.ctx_table = nullptr;
    L.args_table = nullptr;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(cfg.nblocks, 1, 1);
    lc.blockDim = block;
    lc.dynamicSmemBytes = 0;
    lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    lc.attrs = attr;
    lc.numAttrs = pdl_launch_attr(&attr[0]);
    return cudaLaunchKernelEx(&lc, kreal, L);
  }
  LT<true> L;
  L.ctx = RankCtx{};
  L.args = ArgsT{};
  L.ctx_table = ctx;
  L.args_table = args;
  dim3 grid(cfg.nblocks, cfg.nctx, 1);
  void* params[] = {&L};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kemu), grid, block, params, 0, cfg.stream);
}

#define CCL_DISPATCH_REDUCE_DTYPE(DT, KERNEL)                                                          \
  switch (DT) {                                                                                        \
    case kU8: return launch_pair<CollArgs, Launch>(KERNEL<uint8_t, false>, KERNEL<uint8_t, true>, ctx, args, cfg);       \
    case kI8: return launch_pair<CollArgs, Launch>(KERNEL<int8_t, false>, KERNEL<int8_t, true>, ctx, args, cfg);         \
    case kI16: return launch_pair<CollArgs, Launch>(KERNEL<int16_t, false>, KERNEL<int16_t, true>, ctx, args, cfg);      \
    case kI32: return launch_pair<CollArgs, Launch>(KERNEL<int32_t, false>, KERNEL<int32_t, true>, ctx, args, cfg);      \
    case kI64: return launch_pair<CollArgs, Launch>(KERNEL<int64_t, false>, KERNEL<int64_t, true>, ctx, args, cfg);      \
    case kF16: return launch_pair<CollArgs, Launch>(KERNEL<__half, false>, KERNEL<__half, true>, ctx, args, cfg);        \
    case kBF16: return launch_pair<CollArgs, Launch>(KERNEL<__nv_bfloat16, false>, KERNEL<__nv_bfloat16, true>, ctx, args, cfg); \
    case kF32: return launch_pair<CollArgs, Launch>(KERNEL<float, false>, KERNEL<float, true>, ctx, args, cfg);          \
    case kF64: return launch_pair<CollArgs, Launch>(KERNEL<double, false>, KERNEL<double, true>, ctx, args, cfg);        \
    default: return cudaErrorInvalidValue;                                                             \
  }

}  // namespace

cudaError_t launch_allreduce_oneshot(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  CCL_DISPATCH_REDUCE_DTYPE(dtype, allreduce_oneshot_kernel)
}
cudaError_t launch_allreduce_twoshot(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  CCL_DISPATCH_REDUCE_DTYPE(dtype, allreduce_twoshot_kernel)
}

cudaError_t launch_reduce_scatter(int in_dtype, int out_dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  if (in_dtype != out_dtype) {
    if (out_dtype != kF32) return cudaErrorInvalidValue;
    if (in_dtype == kBF16)
      return launch_pair<CollArgs, Launch>(reduce_scatter_kernel<__nv_bfloat16, float, false>, reduce_scatter_kernel<__nv_bfloat16, float, true>, ctx, args, cfg);
    if (in_dtype == kF16)
      return launch_pair<CollArgs, Launch>(reduce_scatter_kernel<__half, float, false>, reduce_scatter_kernel<__half, float, true>, ctx, args, cfg);
    return cudaErrorInvalidValue;
  }
  switch (in_dtype) {
#define RS_CASE(E, T) case E: return launch_pair<CollArgs, Launch>(reduce_scatter_kernel<T, T, false>, reduce_scatter_kernel<T, T, true>, ctx, args, cfg);
    RS_CASE(kU8, uint8_t) RS_CASE(kI8, int8_t) RS_CASE(kI16, int16_t) RS_CASE(kI32, int32_t)
    RS_CASE(kI64, int64_t) RS_CASE(kF16, __half) RS_CASE(kBF16, __nv_bfloat16) RS_CASE(kF32, float)
    RS_CASE(kF64, double)
#undef RS_CASE
    default: return cudaErrorInvalidValue;
  }
}
cudaError_t launch_allreduce_nvls(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  switch (dtype) {
    case kBF16: return launch_pair<CollArgs, Launch>(allreduce_nvls_kernel<__nv_bfloat16, false>, allreduce_nvls_kernel<__nv_bfloat16, true>, ctx, args, cfg);
    case kF16: return launch_pair<CollArgs, Launch>(allreduce_nvls_kernel<__half, false>, allreduce_nvls_kernel<__half, true>, ctx, args, cfg);
    case kF32: return launch_pair<CollArgs, Launch>(allreduce_nvls_kernel<float, false>, allreduce_nvls_kernel<float, true>, ctx, args, cfg);
    default: return cudaErrorInvalidValue;
  }
}
cudaError_t launch_reduce_scatter_nvls(int dtype, const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  switch (dtype) {
    case kBF16: return launch_pair<CollArgs, Launch>(reduce_scatter_nvls_kernel<__nv_bfloat16, false>, reduce_scatter_nvls_kernel<__nv_bfloat16, true>, ctx, args, cfg);
    case kF16: return launch_pair<CollArgs, Launch>(reduce_scatter_nvls_kernel<__half, false>, reduce_scatter_nvls_kernel<__half, true>, ctx, args, cfg);
    case kF32: return launch_pair<CollArgs, Launch>(reduce_scatter_nvls_kernel<float, false>, reduce_scatter_nvls_kernel<float, true>, ctx, args, cfg);
    default: return cudaErrorInvalidValue;
  }
}
cudaError_t launch_all_gather_nvls(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  return launch_pair<CollArgs, Launch>(all_gather_nvls_kernel<false>, all_gather_nvls_kernel<true>, ctx, args, cfg);
}
cudaError_t launch_all_gather(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  return launch_pair<CollArgs, Launch>(all_gather_kernel<false>, all_gather_kernel<true>, ctx, args, cfg);
}
cudaError_t launch_all_to_all(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  return launch_pair<CollArgs, Launch>(all_to_all_kernel<false>, all_to_all_kernel<true>, ctx, args, cfg);
}
cudaError_t launch_rooted(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  return launch_pair<CollArgs, Launch>(rooted_kernel<false>, rooted_kernel<true>, ctx, args, cfg);
}
cudaError_t launch_barrier(const RankCtx* ctx, const CollArgs* args, const LaunchCfg& cfg) {
  LaunchCfg c = cfg;
  c.nblocks = 1;
  c.nthreads = 32;
  return launch_pair<CollArgs, Launch>(barrier_kernel<false>, barrier_kernel<true>, ctx, args, c);
}
cudaError_t launch_allreduce_residual_rmsnorm(int dtype, const RankCtx* ctx, const FusedNormArgs* args, const LaunchCfg& cfg) {
  if (dtype == kBF16)
    return launch_pair<FusedNormArgs, LaunchNorm>(allreduce_residual_rmsnorm_kernel<__nv_bfloat16, false>, allreduce_residual_rmsnorm_kernel<__nv_bfloat16, true>, ctx, args, cfg);
  if (dtype == kF16)
    return launch_pair<FusedNormArgs, LaunchNorm>(allreduce_residual_rmsnorm_kernel<__half, false>, allreduce_residual_rmsnorm_kernel<__half, true>, ctx, args, cfg);
  return cudaErrorInvalidValue;
}

}  // namespace ccl
