// Device side of the bf16 "TN" GEMM on 5th-generation tensor cores:
//
//     D[M, N] = A[M, K] · B[N, K]^T          (both operands K-contiguous, fp32 accumulation)
//
// One CTA computes one 128 x BN output tile. TMA (cp.async.bulk.tensor, 128-byte swizzle, never
// multicast) streams 128x64 A tiles and BNx64 B tiles into a multi-stage shared-memory ring;
// one elected thread issues tcgen05.mma (UMMA 128 x BN x 16) with the accumulator in TMEM; four
// epilogue warps read the accumulator back with tcgen05.ld. Warp roles:
//
//     warp 0      TMA producer (one elected lane)
//     warp 1      TMEM allocator + MMA issuer (one elected lane)
//     warps 2..5  epilogue; warp w owns TMEM lanes 32*(w%4) .. 32*(w%4)+31
//
// Optional features, all used by the tensor-parallel decode / training paths:
//   * split-K across a thread-block cluster (cluster dim z) with a reduce-scatter over DSMEM:
//     CTA r of the cluster owns rows [r*rpc, (r+1)*rpc) of the tile, every CTA pushes its fp32
//     partial of those rows into the owner's shared memory, and each owner sums in a fixed
//     order (deterministic) and runs the epilogue for its rows, so the epilogue is parallel too;
//   * "dual A": a second A tile `dual_off` rows further down shares the same B tile and gets
//     its own TMEM columns; the epilogue then emits silu(acc0) * acc1 (SwiGLU with the gate and
//     up projections stacked in one weight matrix);
//   * transposed output for the swap-AB decode trick (weights on the 128-row UMMA M side, the
//     few activation rows on the N side), row-major output otherwise;
//   * `EpiFn`: a functor invoked per 16-column accumulator chunk instead of the plain store —
//     this is the hook the GEMM->reduce-scatter kernel uses to scatter tiles into peer memory.
//
// All waits are bounded; on expiry the kernel records an error code in `status` and drains.
#pragma once
#include <cuda.h>
#include "ptx.cuh"

namespace ccl {
namespace gemm {

constexpr int kBM = 128;         // UMMA M
constexpr int kBK = 64;          // 64 bf16 = one 128-byte swizzle row
constexpr int kMaxStages = 12;
constexpr int kThreads = 192;

struct Params {
  int M, N, K;          // logical problem (A rows, B rows, reduction)
  void* out;            // bf16 or fp32
  long long ldo;        // leading dimension of out, in elements
  int trans_out;        // 0: out[m*ldo + n]; 1: out[n*ldo + m]
  int dual_off;         // row offset of the second A operand (DUAL only)
  int stages;           // pipeline depth
  int splitk;           // cluster size along z (1 = no split)
  int* status;          // device-visible error word (0 = ok)
  int a_tiled;          // 1: A is pre-packed as contiguous 128x64 tiles, tile (mt, kt) at packed
                        //    row (mt * k_tiles + kt) * 128 of a [*, 64] matrix (see gemm.h)
  int k_tiles;          // K / 64 of the packed A
  int a_static;         // 1: A is constant data (weights): it may be fetched before the
                        //    predecessor kernel on the stream has finished (programmatic dependent launch)
  int acquire_a;        // 1: A was written by another GPU and observed through a flag; order the
                        //    TMA (async proxy) reads after that acquire with a proxy fence
  const void* a_packed; // base of the packed A (a_tiled only; may be null): lets the producer pull the tiles
                        //    that do not fit the shared-memory ring towards L2 ahead of the dependency wait
};

// Where a CTA's tile lives: `a_row` is the TMA row coordinate of the A tile (it differs from the
// logical output row `m0` when A is read from a gathered staging buffer), `n0` the B/N offset.
struct TileCoord {
  int a_row;
  int m0;
  int n0;
};

struct __align__(8) Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t accum;
  uint32_t tmem_base;
  uint32_t failed;
};

template <typename OutT>
__device__ __forceinline__ void store_elem(OutT* p, float v);
template <>
__device__ __forceinline__ void store_elem<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_elem<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16(v);
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// Default epilogue: plain (optionally transposed) store with tail guards.
template <typename OutT>
struct StoreEpilogue {
  __device__ __forceinline__ void operator()(const Params& p, int m, int n0, const float (&v)[16]) const {
    if (m >= p.M) return;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    if (p.trans_out) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (n0 + j < p.N) store_elem<OutT>(out + (long long)(n0 + j) * p.ldo + m, v[j]);
      }
    } else {
      OutT* row = out + (long long)m * p.ldo + n0;
      if (n0 + 16 <= p.N && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
        if constexpr (sizeof(OutT) == 2) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(row)[0] = make_uint4(w[0], w[1], w[2], w[3]);
          reinterpret_cast<uint4*>(row)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<float4*>(row)[j] =
                make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (n0 + j < p.N) store_elem<OutT>(row + j, v[j]);
      }
    }
  }
};

template <int BN, bool DUAL>
__host__ __device__ constexpr int stage_bytes() {
  return kBM * kBK * 2 * (DUAL ? 2 : 1) + BN * kBK * 2;
}
template <int BN, bool DUAL>
__host__ __device__ constexpr int acc_cols() { return BN * (DUAL ? 2 : 1); }
template <int BN, bool DUAL>
__host__ __device__ constexpr int tmem_cols() {
  int c = acc_cols<BN, DUAL>();
  int a = 32;
  while (a < c) a <<= 1;
  return a;
}
// Rows of the 128-row tile that each CTA of a split-K cluster finalises.
__host__ __device__ constexpr int rows_per_owner(int splitk) { return (kBM + splitk - 1) / splitk; }
// Dynamic shared memory: [<=1023 B alignment slack][stages][split-K reduce buffer][barriers].
// The reduce buffer holds, for the rows this CTA owns, one partial row from every other CTA.
template <int BN, bool DUAL>
__host__ __device__ constexpr size_t smem_bytes(int stages, int splitk) {
  return 1024 + (size_t)stages * stage_bytes<BN, DUAL>() +
         (size_t)(splitk > 1 ? (splitk - 1) : 0) * rows_per_owner(splitk) * acc_cols<BN, DUAL>() * 4 +
         sizeof(Barriers);
}

template <int BN, bool DUAL, typename EpiFn>
__device__ __forceinline__ void gemm_tile_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                               const Params& p, const EpiFn& epi, const TileCoord tc) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA M=128 needs N % 16 == 0");
  static_assert(acc_cols<BN, DUAL>() <= 512, "TMEM has 512 columns");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kStage = stage_bytes<BN, DUAL>();
  constexpr int kABytes = kBM * kBK * 2;
  constexpr int kAcc = acc_cols<BN, DUAL>();
  constexpr uint32_t kTmemCols = tmem_cols<BN, DUAL>();
  const int stages = p.stages;
  float* red = reinterpret_cast<float*>(smem + (size_t)stages * kStage);
  const int nred = p.splitk > 1 ? p.splitk - 1 : 0;
  const int rpc = rows_per_owner(p.splitk);
  Barriers* bars = reinterpret_cast<Barriers*>(reinterpret_cast<uint8_t*>(red) +
                                               (size_t)nred * rpc * kAcc * 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = tc.m0;
  const int n0 = tc.n0;
  const uint32_t crank = p.splitk > 1 ? ptx::cluster_ctarank() : 0;

  // K range of this split.
  const int k_iters_total = (p.K + kBK - 1) / kBK;
  const int per = (k_iters_total + p.splitk - 1) / p.splitk;
  const int it_begin = (int)crank * per;
  int it_end = it_begin + per;
  if (it_end > k_iters_total) it_end = k_iters_total;
  const int n_iters = it_end > it_begin ? it_end - it_begin : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    ptx::mbar_init(&bars->accum, 1);
    bars->failed = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  ptx::griddep_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tmap(tma_a);
      ptx::prefetch_tmap(tma_b);
      if (p.acquire_a) asm volatile("fence.proxy.async;" ::: "memory");
      auto load_a = [&](int i) {
        const int s = i % stages;
        uint8_t* st = smem + (size_t)s * kStage;
        const int kx = (it_begin + i) * kBK;
        ptx::mbar_arrive_expect_tx(&bars->full[s], kStage);
        if (p.a_tiled) {
          // one contiguous 16 KB tile per load
          const int kt = it_begin + i;
          ptx::tma_load_2d(st, tma_a, &bars->full[s], 0, ((tc.a_row / kBM) * p.k_tiles + kt) * kBM);
          if (DUAL)
            ptx::tma_load_2d(st + kABytes, tma_a, &bars->full[s], 0,
                             (((tc.a_row + p.dual_off) / kBM) * p.k_tiles + kt) * kBM);
        } else {
          ptx::tma_load_2d(st, tma_a, &bars->full[s], kx, tc.a_row);
          if (DUAL) ptx::tma_load_2d(st + kABytes, tma_a, &bars->full[s], kx, tc.a_row + p.dual_off);
        }
      };
      auto load_b = [&](int i) {
        const int s = i % stages;
        uint8_t* st = smem + (size_t)s * kStage;
        ptx::tma_load_2d(st + kABytes * (DUAL ? 2 : 1), tma_b, &bars->full[s], (it_begin + i) * kBK, n0);
      };
      int i0 = 0;
      if (p.a_static) {
        // A (weights) is not produced by any earlier kernel: fill the pipeline with A tiles while
        // the predecessor kernel is still running, then wait for it and fetch the B tiles.
        const int pre = n_iters < stages ? n_iters : stages;
        for (int i = 0; i < pre; ++i) load_a(i);
        if (p.a_tiled && p.a_packed != nullptr) {
          // the rest of this CTA's weight tiles: a hint towards L2 while the predecessor still runs
          const char* base = static_cast<const char*>(p.a_packed);
          // (at most four tiles ahead: a CTA with a long K range would otherwise push its neighbours' tiles out of L2)
          const int ahead = n_iters < pre + 4 ? n_iters : pre + 4;
          for (int i = pre; i < ahead; ++i) {
            const size_t kt = (size_t)(it_begin + i);
            ptx::bulk_prefetch_l2(base + ((size_t)(tc.a_row / kBM) * p.k_tiles + kt) * kABytes, kABytes);
            if (DUAL) ptx::bulk_prefetch_l2(base + ((size_t)((tc.a_row + p.dual_off) / kBM) * p.k_tiles + kt) * kABytes, kABytes);
          }
        }
        ptx::griddep_wait();
        for (int i = 0; i < pre; ++i) load_b(i);
        i0 = pre;
      } else {
        ptx::griddep_wait();
      }
      for (int i = i0; i < n_iters; ++i) {
        const int s = i % stages;
        const uint32_t ph = (i / stages) & 1;
        if (!ptx::mbar_wait(&bars->empty[s], ph ^ 1)) {
          bars->failed = 1;
          if (p.status) atomicExch(p.status, 101);
          break;
        }
        load_a(i);
        load_b(i);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16(kBM, BN);
      bool ok = true;
      for (int i = 0; i < n_iters && ok; ++i) {
        const int s = i % stages;
        const uint32_t ph = (i / stages) & 1;
        if (!ptx::mbar_wait(&bars->full[s], ph)) {
          bars->failed = 1;
          if (p.status) atomicExch(p.status, 102);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t a_addr = ptx::smem_u32(smem + (size_t)s * kStage);
        const uint32_t b_addr = a_addr + kABytes * (DUAL ? 2 : 1);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          const uint64_t db = ptx::make_desc_sw128(b_addr + k * 32);
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          ptx::umma_bf16_ss(tmem_base, ptx::make_desc_sw128(a_addr + k * 32), db, idesc, acc);
          if (DUAL)
            ptx::umma_bf16_ss(tmem_base + BN, ptx::make_desc_sw128(a_addr + kABytes + k * 32), db,
                              idesc, acc);
        }
        ptx::umma_commit(&bars->empty[s]);  // frees the stage once these MMAs have read it
      }
      ptx::umma_commit(&bars->accum);
    }
  } else {
    // ---- epilogue warps -------------------------------------------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    bool ok = ptx::mbar_wait(&bars->accum, 0);
    if (!ok) {
      bars->failed = 1;
      if (p.status) atomicExch(p.status, 103);
    }
    ptx::tc_fence_after();
    // the producer already waited for the predecessor grid before it fetched B; the epilogue
    // threads repeat the (by now satisfied) wait so that whatever they read or overwrite from an
    // earlier kernel is ordered for them too
    ptx::griddep_wait();
    if (p.splitk > 1) {
      // reduce-scatter: send this row's partial to the CTA that owns the row
      // (buffer layout at the owner: [source slot][column group of 4][local row] float4)
      const int owner = row / rpc;
      const int rl = row - owner * rpc;
      const uint32_t slot = crank < (uint32_t)owner ? crank : crank - 1;
      const uint32_t base = ptx::mapa(ptx::smem_u32(red), (uint32_t)owner) + slot * (uint32_t)(rpc * kAcc * 4);
      for (int c = 0; c < kAcc; c += 16) {
        uint32_t r[16];
        if (n_iters > 0 && ok) {
          ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + c, r);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0;
        }
        if ((uint32_t)owner != crank) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float4 v = make_float4(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]),
                                   __uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
            ptx::st_cluster_v4(base + (uint32_t)((((c >> 2) + g) * rpc + rl) * 16), v);
          }
        }
      }
    }
  }

  if (p.splitk > 1) {
    ptx::tc_fence_before();
    __syncwarp();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tc_fence_after();
  }

  if (warp >= 2) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = (bars->failed == 0);
    const bool mine = (p.splitk == 1) || ((uint32_t)(row / rpc) == crank);
    const int rl = row - (int)crank * rpc;
    for (int c = 0; c < BN; c += 16) {
      float v[16], u[16];
      {
        uint32_t r[16];
        if (n_iters > 0 && ok) {
          ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + c, r);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        if (DUAL) {
          if (n_iters > 0 && ok) {
            ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + BN + c, r);
            ptx::tmem_ld_wait();
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) u[j] = __uint_as_float(r[j]);
        }
      }
      if (mine) {
        // own partial first, then the other CTAs in rank order: a fixed summation order
        for (int s = 0; s < nred; ++s) {
          const float4* pr = reinterpret_cast<const float4*>(red + (size_t)s * rpc * kAcc);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float4 t = pr[((c >> 2) + g) * rpc + rl];
            v[4 * g] += t.x; v[4 * g + 1] += t.y; v[4 * g + 2] += t.z; v[4 * g + 3] += t.w;
          }
          if (DUAL) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float4 t = pr[(((BN + c) >> 2) + g) * rpc + rl];
              u[4 * g] += t.x; u[4 * g + 1] += t.y; u[4 * g + 2] += t.z; u[4 * g + 3] += t.w;
            }
          }
        }
        if (DUAL) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu(v[j]) * u[j];
        }
        if (ok) epi(p, m0 + row, n0 + c, v);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
}


// ---------------------------------------------------------------------------------------------
// Persistent variant for compute-bound problems: one CTA per SM walks a list of output tiles
// (grouped so that the tiles in flight at any time share A and B panels in L2). The smem ring
// keeps running across tiles, and the accumulator is double-buffered in TMEM (2 x BN columns):
// while the epilogue warps drain tile i, the MMA warp already accumulates tile i+1.
// ---------------------------------------------------------------------------------------------
struct __align__(8) PersistentBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

template <int BN>
__host__ __device__ constexpr size_t persistent_smem_bytes(int stages) {
  return 1024 + (size_t)stages * stage_bytes<BN, false>() + sizeof(PersistentBarriers);
}

__device__ __forceinline__ void tile_of(int t, int m_tiles, int n_tiles, int& mt, int& nt) {
  constexpr int kGroupM = 16;
  const int in_group = kGroupM * n_tiles;
  const int gid = t / in_group;
  const int first_m = gid * kGroupM;
  const int gsm = (m_tiles - first_m) < kGroupM ? (m_tiles - first_m) : kGroupM;
  const int r = t - gid * in_group;
  mt = first_m + r % gsm;
  nt = r / gsm;
}

template <int BN, typename EpiFn>
__device__ __forceinline__ void gemm_persistent_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                                     const Params& p, const EpiFn& epi) {
  static_assert(BN == 128 || BN == 256, "persistent kernel: BN 128 or 256 (2*BN TMEM columns)");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kStage = stage_bytes<BN, false>();
  constexpr int kABytes = kBM * kBK * 2;
  constexpr uint32_t kTmemCols = 2 * BN;
  const int stages = p.stages;
  PersistentBarriers* bars = reinterpret_cast<PersistentBarriers*>(smem + (size_t)stages * kStage);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBM - 1) / kBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total = m_tiles * n_tiles;
  const int k_iters = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&bars->tmem_full[b], 1);
      ptx::mbar_init(&bars->tmem_empty[b], 128);  // every epilogue thread arrives
    }
    bars->failed = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tmap(tma_a);
      ptx::prefetch_tmap(tma_b);
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x) {
        int mt, nt;
        tile_of(t, m_tiles, n_tiles, mt, nt);
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!ptx::mbar_wait(&bars->empty[s], ph ^ 1)) {
            bars->failed = 1;
            if (p.status) atomicExch(p.status, 111);
            t = total;
            break;
          }
          uint8_t* st = smem + (size_t)s * kStage;
          ptx::mbar_arrive_expect_tx(&bars->full[s], kStage);
          ptx::tma_load_2d(st, tma_a, &bars->full[s], k * kBK, mt * kBM);
          ptx::tma_load_2d(st + kABytes, tma_b, &bars->full[s], k * kBK, nt * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16(kBM, BN);
      uint32_t it = 0;
      int i = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
        const int acc = i & 1;
        if (!ptx::mbar_wait(&bars->tmem_empty[acc], (((uint32_t)i >> 1) & 1) ^ 1)) {
          bars->failed = 1;
          if (p.status) atomicExch(p.status, 112);
          break;
        }
        ptx::tc_fence_after();
        bool ok = true;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!ptx::mbar_wait(&bars->full[s], ph)) {
            bars->failed = 1;
            if (p.status) atomicExch(p.status, 113);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(smem + (size_t)s * kStage);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            ptx::umma_bf16_ss(tmem_base + acc * BN, ptx::make_desc_sw128(a_addr + kk * 32),
                              ptx::make_desc_sw128(b_addr + kk * 32), idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          ptx::umma_commit(&bars->empty[s]);
        }
        if (!ok) break;
        ptx::umma_commit(&bars->tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int i = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
      int mt, nt;
      tile_of(t, m_tiles, n_tiles, mt, nt);
      const int acc = i & 1;
      if (!ptx::mbar_wait(&bars->tmem_full[acc], ((uint32_t)i >> 1) & 1)) {
        bars->failed = 1;
        if (p.status) atomicExch(p.status, 114);
        break;
      }
      ptx::tc_fence_after();
#pragma unroll 2
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c, r);
        ptx::tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        epi(p, mt * kBM + row, nt * BN + c, v);
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(&bars->tmem_empty[acc]);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace gemm
}  // namespace ccl
