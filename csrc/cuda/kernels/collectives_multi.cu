// Batched small-tensor collectives: see collectives_multi.h.
//
// All three modes are one-shot exchanges through the staging half of the round:
//   all_reduce      push every tensor to every peer's slot [me]; after the flag round reduce the W
//                   copies (own one from user memory) in rank order into the output;
//   reduce_scatter  push piece p of every tensor to rank p's slot [me]; after the flag round reduce
//                   the W pieces of the own shard;
//   all_gather      push every tensor to every peer's slot [me]; after the flag round copy slot [p]
//                   to piece p of the output.
// Tensor t starts at the same 16-byte aligned offset of every slot. CTA b moves sub-slice b of
// every tensor, so it pairs with CTA b of the peers like every other kernel of the library.
#include "collectives_multi.h"

#include "comm.cuh"
#include "gemm.h"

namespace ccl {
namespace {

template <bool EMU>
struct LaunchMulti {
  RankCtx ctx;
  MultiArgs args;
  const RankCtx* ctx_table;
  const MultiArgs* args_table;
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
__device__ __forceinline__ bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, bool EMU>
__global__ void __launch_bounds__(512) multi_kernel(const __grid_constant__ LaunchMulti<EMU> L) {
  const RankCtx& ctx = EMU ? L.ctx_table[blockIdx.y] : L.ctx;
  const MultiArgs& a = EMU ? L.args_table[blockIdx.y] : L.args;
  __shared__ int s_failed;
  Sync sy(ctx, &s_failed, true);
  using A = typename Acc<T>::type;
  constexpr int N = Vec<T>::kN;
  const int W = ctx.world, me = ctx.rank;
  const size_t slot = a.slot_bytes;

  // ---- push ------------------------------------------------------------------------------------
  size_t off = 0;
  for (int t = 0; t < a.n; ++t) {
    const size_t cnt = a.count[t];  // elements (reductions) or bytes (all_gather; T is uint8_t there)
    const size_t nvec = ceil_div(cnt, (size_t)N);
    const Range r = sub_slice(nvec);
    if (a.mode == kMultiReduceScatter) {
      for (int q = 1; q < W; ++q) {
        const int p = me + q >= W ? me + q - W : me + q;
        const T* src = reinterpret_cast<const T*>(a.in[t]) + (size_t)p * cnt;
        const bool al = al16(src);
        char* dst = sy.half(p, 0) + (size_t)me * slot + off;
        for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) store_stage(dst + j * 16, load_vec(src, j, cnt, al));
      }
    } else {
      const T* src = reinterpret_cast<const T*>(a.in[t]);
      const bool al = al16(src);
      for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
        const Vec<T> v = load_vec(src, j, cnt, al);
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < W && p != me) store_stage(sy.half(p, 0) + (size_t)me * slot + off + j * 16, v);
      }
    }
    off += nvec * 16;
  }
  sy.signal_all(0, 0);
  const bool ok = sy.wait_all(0, 0);
  // ---- consume ---------------------------------------------------------------------------------
  if (ok) {
    const char* mine = sy.half(me, 0);
    off = 0;
    for (int t = 0; t < a.n; ++t) {
      const size_t cnt = a.count[t];
      const size_t nvec = ceil_div(cnt, (size_t)N);
      const Range r = sub_slice(nvec);
      if (a.mode == kMultiAllGather) {
        T* out = reinterpret_cast<T*>(a.out[t]);
        const T* in = reinterpret_cast<const T*>(a.in[t]);
        for (int p = 0; p < W; ++p) {
          T* dst = out + (size_t)p * cnt;
          const bool al = al16(dst);
          if (p == me) {
            if (dst != in) {
              const bool ali = al16(in);
              for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) store_vec(dst, j, cnt, al, load_vec(in, j, cnt, ali));
            }
          } else {
            const char* src = mine + (size_t)p * slot + off;
            for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) store_vec(dst, j, cnt, al, load_stage<T>(src + j * 16));
          }
        }
      } else {
        const T* own = reinterpret_cast<const T*>(a.in[t]) + (a.mode == kMultiReduceScatter ? (size_t)me * cnt : 0);
        T* out = reinterpret_cast<T*>(a.out[t]);
        const bool al_own = al16(own), al_out = al16(out);
        for (size_t j = r.j0 + threadIdx.x; j < r.j1; j += blockDim.x) {
          A acc[N];
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p) {
            if (p < W) {
              const Vec<T> v = (p == me) ? load_vec(own, j, cnt, al_own) : load_stage<T>(mine + (size_t)p * slot + off + j * 16);
#pragma unroll
              for (int e = 0; e < N; ++e)
                acc[e] = (p == 0) ? to_acc(v.v[e]) : (a.op == kSum ? acc[e] + to_acc(v.v[e]) : Combine<A>::apply(a.op, acc[e], to_acc(v.v[e])));
            }
          }
          Vec<T> res;
#pragma unroll
          for (int e = 0; e < N; ++e) {
            A x = acc[e];
            if (a.has_scale == 1) x = static_cast<A>(x * static_cast<A>(a.scale));
            else if (a.has_scale == 2) x = static_cast<A>(x / static_cast<A>(a.scale));
            res.v[e] = from_acc<T, A>(x);
          }
          store_vec(out, j, cnt, al_out, res);
        }
      }
      off += nvec * 16;
    }
  }
  sy.finish(1);
}

template <typename T>
cudaError_t launch_t(const RankCtx* ctx, const MultiArgs* args, const LaunchCfg& cfg) {
  dim3 block(cfg.nthreads);
  if (!cfg.cooperative) {
    LaunchMulti<false> L;
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
    return cudaLaunchKernelEx(&lc, multi_kernel<T, false>, L);
  }
  LaunchMulti<true> L;
  L.ctx = RankCtx{};
  L.args = MultiArgs{};
  L.ctx_table = ctx;
  L.args_table = args;
  void* params[] = {&L};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(multi_kernel<T, true>), dim3(cfg.nblocks, cfg.nctx, 1), block, params, 0,
                                     cfg.stream);
}

}  // namespace

size_t multi_slot_bytes(int dtype, const MultiArgs& a) {
  const size_t esz = a.mode == kMultiAllGather ? 1 : dtype_size(dtype);
  size_t total = 0;
  for (int t = 0; t < a.n; ++t) total += round_up((size_t)a.count[t] * esz, 16);
  return round_up(total, 128);
}

cudaError_t launch_multi(int dtype, const RankCtx* ctx, const MultiArgs* args, const LaunchCfg& cfg) {
  if (args == nullptr) return cudaErrorInvalidValue;
  // (all_gather moves bytes whatever the tensors hold: its callers pass kU8 and byte counts)
  switch (dtype) {
    case kU8: return launch_t<uint8_t>(ctx, args, cfg);
    case kI8: return launch_t<int8_t>(ctx, args, cfg);
    case kI16: return launch_t<int16_t>(ctx, args, cfg);
    case kI32: return launch_t<int32_t>(ctx, args, cfg);
    case kI64: return launch_t<int64_t>(ctx, args, cfg);
    case kF16: return launch_t<__half>(ctx, args, cfg);
    case kBF16: return launch_t<__nv_bfloat16>(ctx, args, cfg);
    case kF32: return launch_t<float>(ctx, args, cfg);
    case kF64: return launch_t<double>(ctx, args, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ccl
