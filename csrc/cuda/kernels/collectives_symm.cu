// Zero-copy collectives on symmetric memory: see collectives_symm.h.
//
// Every kernel is: flag round (all ranks have entered, so their symmetric inputs are complete and
// their symmetric outputs may be overwritten) -> one pass over the data straight between the
// user buffers -> flag round (all ranks have finished reading this rank's input and writing this
// rank's output). CTA b works on sub-slice b of its rank's share and pairs with CTA b of the
// peers, as everywhere in this library; a rank's kernel ends only when all its CTAs have seen
// the closing flags, i.e. when every sub-slice is done.
//
// With `use_mc` the share is reduced inside the NVSwitch (multimem.ld_reduce over the multicast
// mapping of the heaps) and broadcast with multimem.st; the emulation (all ranks on one GPU, no
// multicast object) plays both with loops over the ranks' heaps.
#include "collectives_symm.h"

#include "comm.cuh"
#include "gemm.h"

namespace ccl {
namespace {

template <bool EMU>
struct LaunchSymm {
  RankCtx ctx;
  SymmArgs args;
  const RankCtx* ctx_table;
  const SymmArgs* args_table;
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
// Types the switch cannot reduce never take the multicast path (the launcher refuses use_mc for them).
template <typename T> struct Multimem {
  static __device__ __forceinline__ uint4 ld_reduce(const void*) { return make_uint4(0, 0, 0, 0); }
};

constexpr int kUnrollMc = 4;   // multicast loads in flight per thread

// N output elements as one aligned store (16 bytes, or 32 when bf16 / f16 is widened to fp32).
template <typename TOut, int N>
struct alignas(sizeof(TOut) * N >= 32 ? 32 : 16) OutVec {
  TOut v[N];
};

#define CCL_SYMM_CTX                                               \
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;      \
  const SymmArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;     \
  __shared__ int s_failed;                                         \
  Sync sy(ctx, &s_failed, true);                                   \
  const int W = ctx.world, me = ctx.rank;

// Sum (or other op) of vector `off` over all ranks' heaps, in rank order, rounded once.
template <typename T, bool EMU>
__device__ __forceinline__ Vec<T> reduce_at(const RankCtx& ctx, size_t off, int W, int op, bool use_mc) {
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  Vec<T> r;
  if (use_mc && !EMU) {
    *reinterpret_cast<uint4*>(&r) = Multimem<T>::ld_reduce(ctx.mc_heap + off);
    return r;
  }
  Vec<T> v[kMaxRanks];
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p)
    if (p < W) v[p] = load_stage<T>(ctx.heap[p] + off);
  A acc[N];
#pragma unroll
  for (int t = 0; t < N; ++t) acc[t] = to_acc(v[0].v[t]);
#pragma unroll
  for (int p = 1; p < kMaxRanks; ++p) {
    if (p < W) {
#pragma unroll
      for (int t = 0; t < N; ++t) acc[t] = (op == kSum) ? acc[t] + to_acc(v[p].v[t]) : Combine<A>::apply(op, acc[t], to_acc(v[p].v[t]));
    }
  }
#pragma unroll
  for (int t = 0; t < N; ++t) r.v[t] = from_acc<T, A>(acc[t]);
  return r;
}

template <typename T>
__device__ __forceinline__ Vec<T> scale_vec(Vec<T> v, const SymmArgs& a) {
  using A = typename Acc<T>::type;
  if (a.has_scale) {
#pragma unroll
    for (int t = 0; t < Vec<T>::kN; ++t) {
      A x = to_acc(v.v[t]);
      x = a.has_scale == 2 ? static_cast<A>(x / static_cast<A>(a.scale)) : static_cast<A>(x * static_cast<A>(a.scale));
      v.v[t] = from_acc<T, A>(x);
    }
  }
  return v;
}

// ---------------------------------------------------------------------------------------------
// all_reduce: rank r reduces share r of every rank's input and writes it into every rank's output
// ---------------------------------------------------------------------------------------------
template <typename T, bool EMU>
__global__ void __launch_bounds__(512) allreduce_symm_kernel(const __grid_constant__ LaunchSymm<EMU> L) {
  CCL_SYMM_CTX
  const size_t nvec = a.count * sizeof(T) / 16;
  const size_t spr = ceil_div(nvec, (size_t)W);
  const size_t vb = (size_t)me * spr;
  const Range r = sub_slice(clamp_len(nvec, vb, spr));
  sy.signal_all(0, 0);
  bool ok = sy.wait_all(0, 0);
  if (ok) {
    const bool mc = a.use_mc != 0;
    const size_t nt = blockDim.x;
    size_t j = r.j0 + threadIdx.x;
    if (mc && !EMU) {
      // through the switch: one reducing load and one multicast store per vector; kUnrollMc of them are
      // in flight per thread, which is what covers the NVLink round trip at full rate
      for (; j + (kUnrollMc - 1) * nt < r.j1; j += kUnrollMc * nt) {
        Vec<T> res[kUnrollMc];
#pragma unroll
        for (int u = 0; u < kUnrollMc; ++u) *reinterpret_cast<uint4*>(&res[u]) = Multimem<T>::ld_reduce(ctx.mc_heap + a.in_off + (vb + j + u * nt) * 16);
#pragma unroll
        for (int u = 0; u < kUnrollMc; ++u) {
          res[u] = scale_vec<T>(res[u], a);
          ptx::multimem_st_v4(ctx.mc_heap + a.out_off + (vb + j + u * nt) * 16, *reinterpret_cast<const uint4*>(&res[u]));
        }
      }
      for (; j < r.j1; j += nt) {
        const Vec<T> res = scale_vec<T>(reduce_at<T, EMU>(ctx, a.in_off + (vb + j) * 16, W, a.op, true), a);
        ptx::multimem_st_v4(ctx.mc_heap + a.out_off + (vb + j) * 16, *reinterpret_cast<const uint4*>(&res));
      }
    } else {
      // peer loads: one load per rank is in flight per thread already
      for (; j < r.j1; j += nt) {
        const Vec<T> res = scale_vec<T>(reduce_at<T, EMU>(ctx, a.in_off + (vb + j) * 16, W, a.op, false), a);
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < W) ptx::st_v4(ctx.heap[p] + a.out_off + (vb + j) * 16, *reinterpret_cast<const uint4*>(&res));
      }
    }
  }
  sy.signal_all(1, 0);
  sy.wait_all(1, 0);
  sy.finish(1);
}

// ---------------------------------------------------------------------------------------------
// reduce_scatter: rank r reduces piece r of every rank's symmetric input into its local output
// ---------------------------------------------------------------------------------------------
template <typename TIn, typename TOut, bool EMU>
__global__ void __launch_bounds__(512) reduce_scatter_symm_kernel(const __grid_constant__ LaunchSymm<EMU> L) {
  CCL_SYMM_CTX
  using A = typename Acc<TIn>::type;
  constexpr int N = Vec<TIn>::kN;
  const size_t pv = a.count * sizeof(TIn) / 16;   // vectors per piece
  const Range r = sub_slice(pv);
  TOut* out = reinterpret_cast<TOut*>(a.out);
  sy.signal_all(0, 0);
  bool ok = sy.wait_all(0, 0);
  if (ok) {
    const bool mc = a.use_mc != 0;
    const size_t base = a.in_off + (size_t)me * pv * 16;
    const size_t nt = blockDim.x;
    // widen (bf16 / f16 gradients kept as fp32) and scale in the same pass
    auto emit = [&](size_t j, const Vec<TIn>& red) {
      OutVec<TOut, N> o;
#pragma unroll
      for (int t = 0; t < N; ++t) {
        A x = to_acc(red.v[t]);
        if (a.has_scale == 1) x = static_cast<A>(x * static_cast<A>(a.scale));
        else if (a.has_scale == 2) x = static_cast<A>(x / static_cast<A>(a.scale));
        o.v[t] = static_cast<TOut>(from_acc<TOut, A>(x));
      }
      *reinterpret_cast<OutVec<TOut, N>*>(out + j * N) = o;
    };
    size_t j = r.j0 + threadIdx.x;
    if (mc && !EMU) {
      for (; j + (kUnrollMc - 1) * nt < r.j1; j += kUnrollMc * nt) {
        Vec<TIn> red[kUnrollMc];
#pragma unroll
        for (int u = 0; u < kUnrollMc; ++u) *reinterpret_cast<uint4*>(&red[u]) = Multimem<TIn>::ld_reduce(ctx.mc_heap + base + (j + u * nt) * 16);
#pragma unroll
        for (int u = 0; u < kUnrollMc; ++u) emit(j + u * nt, red[u]);
      }
    }
    for (; j < r.j1; j += nt) emit(j, reduce_at<TIn, EMU>(ctx, base + j * 16, W, a.op, mc));
  }
  sy.signal_all(1, 0);
  sy.wait_all(1, 0);   // the peers have finished reading this rank's input
  sy.finish(1);
}

// ---------------------------------------------------------------------------------------------
// all_gather: rank r writes its local piece into slot r of every rank's symmetric output
// ---------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(512) all_gather_symm_kernel(const __grid_constant__ LaunchSymm<EMU> L) {
  CCL_SYMM_CTX
  const size_t pv = a.count / 16;   // vectors per piece
  const Range r = sub_slice(pv);
  const char* in = static_cast<const char*>(a.in);
  sy.signal_all(0, 0);
  bool ok = sy.wait_all(0, 0);      // every rank's output buffer may be written now
  if (ok) {
    const size_t base = a.out_off + (size_t)me * pv * 16;
    const bool mc = a.use_mc != 0 && !EMU;
    const size_t nt = blockDim.x;
    size_t j = r.j0 + threadIdx.x;
    for (; j + 3 * nt < r.j1; j += 4 * nt) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(in + (j + u * nt) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (mc) {
          ptx::multimem_st_v4(ctx.mc_heap + base + (j + u * nt) * 16, v[u]);
        } else {
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)
            if (p < W) ptx::st_v4(ctx.heap[p] + base + (j + u * nt) * 16, v[u]);
        }
      }
    }
    for (; j < r.j1; j += nt) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + j * 16);
      if (mc) {
        ptx::multimem_st_v4(ctx.mc_heap + base + j * 16, v);
      } else {
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < W) ptx::st_v4(ctx.heap[p] + base + j * 16, v);
      }
    }
  }
  sy.signal_all(1, 0);
  sy.wait_all(1, 0);
  sy.finish(1);
}

template <typename KR, typename KE>
cudaError_t launch_symm(KR kreal, KE kemu, const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg) {
  dim3 block(cfg.nthreads);
  if (!cfg.cooperative) {
    LaunchSymm<false> L;
    L.ctx = *ctx;
    L.args = *args;
    L.ctx_table = nullptr;
    L.args_table = nullptr;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(cfg.nblocks, 1, 1);
    lc.blockDim = block;
    lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    lc.attrs = attr;
    lc.numAttrs = pdl_launch_attr(&attr[0]);
    return cudaLaunchKernelEx(&lc, kreal, L);
  }
  LaunchSymm<true> L;
  L.ctx = RankCtx{};
  L.args = SymmArgs{};
  L.ctx_table = ctx;
  L.args_table = args;
  void* params[] = {&L};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kemu), dim3(cfg.nblocks, cfg.nctx, 1), block, params, 0, cfg.stream);
}

bool switch_reducible(int dtype) { return dtype == kBF16 || dtype == kF16 || dtype == kF32; }

}  // namespace

cudaError_t launch_allreduce_symm(int dtype, const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg) {
  switch (dtype) {
#define AR_CASE(E, T) case E: return launch_symm(allreduce_symm_kernel<T, false>, allreduce_symm_kernel<T, true>, ctx, args, cfg);
    AR_CASE(kU8, uint8_t) AR_CASE(kI8, int8_t) AR_CASE(kI16, int16_t) AR_CASE(kI32, int32_t) AR_CASE(kI64, int64_t)
    AR_CASE(kF16, __half) AR_CASE(kBF16, __nv_bfloat16) AR_CASE(kF32, float) AR_CASE(kF64, double)
#undef AR_CASE
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_reduce_scatter_symm(int in_dtype, int out_dtype, const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg) {
  if (in_dtype != out_dtype) {
    if (out_dtype != kF32) return cudaErrorInvalidValue;
    if (in_dtype == kBF16) return launch_symm(reduce_scatter_symm_kernel<__nv_bfloat16, float, false>, reduce_scatter_symm_kernel<__nv_bfloat16, float, true>, ctx, args, cfg);
    if (in_dtype == kF16) return launch_symm(reduce_scatter_symm_kernel<__half, float, false>, reduce_scatter_symm_kernel<__half, float, true>, ctx, args, cfg);
    return cudaErrorInvalidValue;
  }
  switch (in_dtype) {
#define RS_CASE(E, T) case E: return launch_symm(reduce_scatter_symm_kernel<T, T, false>, reduce_scatter_symm_kernel<T, T, true>, ctx, args, cfg);
    RS_CASE(kU8, uint8_t) RS_CASE(kI8, int8_t) RS_CASE(kI16, int16_t) RS_CASE(kI32, int32_t) RS_CASE(kI64, int64_t)
    RS_CASE(kF16, __half) RS_CASE(kBF16, __nv_bfloat16) RS_CASE(kF32, float) RS_CASE(kF64, double)
#undef RS_CASE
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_all_gather_symm(const RankCtx* ctx, const SymmArgs* args, const LaunchCfg& cfg) {
  return launch_symm(all_gather_symm_kernel<false>, all_gather_symm_kernel<true>, ctx, args, cfg);
}

}  // namespace ccl
