// Single-token ("decode") attention for a Llama-style decoder, fused with rotary embedding and
// the KV-cache append: one launch per layer reads q/k/v of the new token from the packed QKV
// projection output, rotates q and k, writes k/v into the cache at the sequence's current
// position, and attends over positions [0, pos]. Memory-bound on the KV cache, so the work is
// split over the sequence (flash-decoding): each CTA handles one (sequence, head, KV range) and
// writes an un-normalised partial (running max, sum, output) to a scratch buffer; the last CTA
// to finish a (sequence, head) combines the partials. head_dim is fixed at 128.
//
// The K and V rows of one (sequence, head) are contiguous in the cache, so one elected thread
// streams them with untiled bulk copies (cp.async.bulk, completion on an mbarrier) into a 3-stage
// shared-memory ring of 32-position chunks; with four CTAs per SM that keeps ~190 KB of loads in
// flight per SM without spending registers on them. Thread mapping for the math: 8 lanes share
// one cache position (16 dims = 32 bytes each), so a warp covers 4 positions per step and a
// 4-warp CTA 16.
#include "decode_attention.h"

#include "gemm.h"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

namespace ccl {
namespace {

constexpr int kHD = 128;
constexpr int kThreads = 128;
constexpr int kGroups = kThreads / 8;  // positions per CTA step
constexpr int kChunk = 32;             // positions per pipeline stage
constexpr int kStages = 3;             // 48 KB of ring: four CTAs fit on an SM
constexpr int kRowBytes = kHD * 2;
constexpr int kStageBytes = 2 * kChunk * kRowBytes;  // K chunk followed by V chunk
constexpr size_t kDynSmem = (size_t)kStages * kStageBytes + 128;

__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&f)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    f[2 * i] = __low2float(h);
    f[2 * i + 1] = __high2float(h);
  }
}
__device__ __forceinline__ void load16_smem(const unsigned char* p, float (&f)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    f[2 * i] = __low2float(h);
    f[2 * i + 1] = __high2float(h);
  }
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&f)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Rotary embedding (rotate-half convention) of the 16 dims [16j, 16j+16) of one head vector.
// `own` holds those dims, `partner` the dims 64 away; cos/sin rows have 64 entries.
__device__ __forceinline__ void rope16(float (&own)[16], const float (&partner)[16], const float* cosr,
                                       const float* sinr, int j) {
  const int base = (j & 3) * 16;  // frequency index of own dim i is (16j + i) mod 64
  const float sign = (j < 4) ? -1.f : 1.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float c = cosr[base + i], s = sinr[base + i];
    own[i] = own[i] * c + sign * partner[i] * s;
  }
}

__global__ void __launch_bounds__(kThreads) decode_attention_kernel(const DecodeAttnParams p) {
  ptx::griddep_launch_dependents();
  const int split = blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int nsplit = gridDim.x;
  const int tid = threadIdx.x;
  const int g = tid >> 3;  // position group within the CTA
  const int j = tid & 7;   // dim slice within the head
  const int kvh = h / (p.n_heads / p.n_kv_heads);
  if (tid == 0 && p.prefetch_l2) {
    // While the projection kernel before this one is still running, pull this CTA's range of the
    // cache towards L2. The cached positions were written by earlier steps; the position read here
    // may be one step old (the kernel that advances it is not known to have finished yet), which
    // moves the range by one row at most - it is only a hint, everything is read again below.
    const int pp = *reinterpret_cast<const volatile int*>(p.positions + b);
    if (pp >= 0 && pp < p.max_seq) {
      const int tot = pp + 1;
      const int pr = (tot + nsplit - 1) / nsplit;
      const int a0 = split * pr, a1 = min(tot, a0 + pr);
      if (a1 > a0) {
        const size_t base = (((size_t)b * p.n_kv_heads + kvh) * p.max_seq + a0) * kHD;
        const uint32_t bytes = (uint32_t)(a1 - a0) * kRowBytes;
        ptx::bulk_prefetch_l2(p.k_cache + base, bytes);
        ptx::bulk_prefetch_l2(p.v_cache + base, bytes);
      }
    }
  }
  ptx::griddep_wait();  // q/k/v of the new token come from the projection kernel just before
  const int pos = p.positions[b];  // the new token's position; attends over [0, pos]
  if (pos < 0 || pos >= p.max_seq) {
    // a position outside the cache would index the cache and the rotary tables out of bounds:
    // record it, write nothing to the cache and emit a zero row (uniform for the whole CTA, and
    // every split of this (sequence, head) takes the same exit, so the arrival counter stays 0)
    if (tid == 0 && p.status) atomicExch(p.status, 201);
    if (split == 0) p.out[(size_t)b * p.out_stride + (size_t)h * kHD + tid] = __float2bfloat16(0.f);
    return;
  }
  const int total = pos + 1;
  const int per = (total + nsplit - 1) / nsplit;
  const int t0 = split * per;
  const int t1 = min(total, t0 + per);

  const __nv_bfloat16* qkv = p.qkv + (size_t)b * p.qkv_stride;
  const float* cosr = p.cos + (size_t)pos * (kHD / 2);
  const float* sinr = p.sin + (size_t)pos * (kHD / 2);
  const int pj = j ^ 4;

  // q: rotate and pre-scale
  float q[16];
  {
    float partner[16];
    load16(qkv + (size_t)h * kHD + j * 16, q);
    load16(qkv + (size_t)h * kHD + pj * 16, partner);
    rope16(q, partner, cosr, sinr, j);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] *= p.scale;
  }

  __nv_bfloat16* kc = p.k_cache + (((size_t)b * p.n_kv_heads + kvh) * p.max_seq) * kHD;
  __nv_bfloat16* vc = p.v_cache + (((size_t)b * p.n_kv_heads + kvh) * p.max_seq) * kHD;

  // The CTA whose range contains `pos` handles the new token from the projection output: it
  // rotates k, keeps k/v (rounded like the cache) in shared memory for its own use and, for the
  // first head of a KV group, appends them to the cache. No other CTA reads that position.
  const bool owns_new = (pos >= t0 && pos < t1);
  __shared__ float s_new_k[kHD], s_new_v[kHD];
  if (owns_new && g == 0) {
    float k[16], partner[16], v[16];
    const __nv_bfloat16* kn = qkv + (size_t)(p.n_heads + kvh) * kHD;
    const __nv_bfloat16* vn = qkv + (size_t)(p.n_heads + p.n_kv_heads + kvh) * kHD;
    load16(kn + j * 16, k);
    load16(kn + pj * 16, partner);
    load16(vn + j * 16, v);
    rope16(k, partner, cosr, sinr, j);
    if (h % (p.n_heads / p.n_kv_heads) == 0) {
      store16(kc + (size_t)pos * kHD + j * 16, k);
      store16(vc + (size_t)pos * kHD + j * 16, v);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      s_new_k[j * 16 + i] = __bfloat162float(__float2bfloat16(k[i]));
      s_new_v[j * 16 + i] = __bfloat162float(__float2bfloat16(v[i]));
    }
  }
  __syncthreads();

  const unsigned gmask = 0xffu << (8 * ((tid & 31) >> 3));
  float m = -INFINITY, l = 0.f, o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = 0.f;

  // ---- stream [t0, t1) through the shared-memory ring ---------------------------------------
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(dyn_smem) + 127) & ~uintptr_t(127));
  __shared__ __align__(8) uint64_t s_full[kStages];
  const int n_chunks = (t1 > t0) ? (t1 - t0 + kChunk - 1) / kChunk : 0;
  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) ptx::mbar_init(&s_full[i], 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int c) {  // thread 0 only
    const int st = c % kStages;
    const int start = t0 + c * kChunk;
    const int n = min(kChunk, t1 - start);
    const uint32_t bytes = (uint32_t)n * kRowBytes;
    unsigned char* dst = ring + (size_t)st * kStageBytes;
    ptx::mbar_arrive_expect_tx(&s_full[st], 2 * bytes);
    ptx::bulk_load(dst, kc + (size_t)start * kHD, bytes, &s_full[st]);
    ptx::bulk_load(dst + kChunk * kRowBytes, vc + (size_t)start * kHD, bytes, &s_full[st]);
  };
  if (tid == 0)
    for (int c = 0; c < n_chunks && c < kStages; ++c) issue(c);
  bool ok = true;
  for (int c = 0; c < n_chunks; ++c) {
    const int st = c % kStages;
    if (!ptx::mbar_wait(&s_full[st], (c / kStages) & 1)) ok = false;  // bounded; result is then invalid
    const unsigned char* ks = ring + (size_t)st * kStageBytes;
    const unsigned char* vs = ks + kChunk * kRowBytes;
    const int start = t0 + c * kChunk;
    const int n = min(kChunk, t1 - start);
#pragma unroll
    for (int pass = 0; pass < kChunk / kGroups; ++pass) {
      const int lt = pass * kGroups + g;
      const int t = start + lt;
      float k[16], v[16];
      if (lt < n) {
        if (t == pos) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            k[i] = s_new_k[j * 16 + i];
            v[i] = s_new_v[j * 16 + i];
          }
        } else {
          load16_smem(ks + (size_t)lt * kRowBytes + j * 32, k);
          load16_smem(vs + (size_t)lt * kRowBytes + j * 32, v);
        }
      }
      // all 8 lanes of a group share `lt`, so the branch is uniform within the shuffle mask
      if (lt < n) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) s += q[i] * k[i];
        s += __shfl_xor_sync(gmask, s, 1);
        s += __shfl_xor_sync(gmask, s, 2);
        s += __shfl_xor_sync(gmask, s, 4);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn);
        const float pr = __expf(s - mn);
        l = l * corr + pr;
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = o[i] * corr + pr * v[i];
        m = mn;
      }
    }
    __syncthreads();  // everyone is done with this stage: refill it
    if (tid == 0 && c + kStages < n_chunks) issue(c + kStages);
  }
  if (!ok && p.status && tid == 0) atomicExch(p.status, 201);

  // combine the kGroups position groups of this CTA
  // (the ring is free now — every chunk was consumed before the last barrier — and is reused
  // for the partial outputs)
  __shared__ float s_m[kGroups], s_l[kGroups];
  float (*s_o)[kHD] = reinterpret_cast<float (*)[kHD]>(ring);
  if (j == 0) {
    s_m[g] = m;
    s_l[g] = l;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) s_o[g][j * 16 + i] = o[i];
  __syncthreads();
  float M = -INFINITY;
  for (int i = 0; i < kGroups; ++i) M = fmaxf(M, s_m[i]);
  float L = 0.f, acc = 0.f;  // thread `tid` owns output dim tid
  for (int i = 0; i < kGroups; ++i) {
    const float w = (s_m[i] == -INFINITY) ? 0.f : __expf(s_m[i] - M);
    L += s_l[i] * w;
    acc += s_o[i][tid] * w;
  }

  __nv_bfloat16* out = p.out + (size_t)b * p.out_stride + (size_t)h * kHD;
  if (nsplit == 1) {
    out[tid] = __float2bfloat16(acc / L);
    return;
  }
  // partial of this split: [b][h][split] -> {M, L, o[128]}
  float* part = p.scratch + (((size_t)b * p.n_heads + h) * nsplit + split) * (kHD + 2);
  part[2 + tid] = acc;
  if (tid == 0) {
    part[0] = M;
    part[1] = L;
  }
  __threadfence();
  __shared__ int s_last;
  __syncthreads();
  if (tid == 0) {
    unsigned int* counter = p.counters + (size_t)b * p.n_heads + h;
    const unsigned int prev = atomicAdd(counter, 1u);
    s_last = (prev == (unsigned int)nsplit - 1);
    if (s_last) *counter = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* base = p.scratch + ((size_t)b * p.n_heads + h) * nsplit * (kHD + 2);
  float GM = -INFINITY;
  for (int i = 0; i < nsplit; ++i) GM = fmaxf(GM, __ldcg(base + (size_t)i * (kHD + 2)));
  float GL = 0.f, gacc = 0.f;
  for (int i = 0; i < nsplit; ++i) {
    const float* pi = base + (size_t)i * (kHD + 2);
    const float mi = __ldcg(pi);
    const float w = (mi == -INFINITY) ? 0.f : __expf(mi - GM);
    GL += __ldcg(pi + 1) * w;
    gacc += __ldcg(pi + 2 + tid) * w;
  }
  out[tid] = __float2bfloat16(gacc / GL);
}

}  // namespace

size_t decode_attention_scratch_bytes(int batch, int n_heads, int nsplit) {
  return (size_t)batch * n_heads * nsplit * (kHD + 2) * sizeof(float);
}

int decode_attention_default_splits(int batch, int n_heads, int max_context) {
  const int pairs = batch * n_heads;
  // four CTAs fit on an SM (shared-memory ring): fill them, but stay within one wave. (Measured and
  // rejected for 512 pairs, where the SMs get 3 or 4 equal CTAs: an uneven two-way split, 7/8 heads
  // dispatched before 1/8 tails, was no faster than no split - 52.1 vs 51.6 us.)
  int s = (4 * 148) / pairs;
  const int cap = (max_context + 127) / 128;  // at least 128 positions (four pipeline chunks) per split
  if (s > cap) s = cap;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

// The kernel moves q/k/v, the cache rows and the output with 16-byte accesses and bulk copies:
// every base pointer must be 16-byte aligned, both row strides multiples of 8 elements, and a
// row must not overlap the next one.
bool decode_attention_layout_ok(const DecodeAttnParams& p) {
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!aligned(p.qkv) || !aligned(p.k_cache) || !aligned(p.v_cache) || !aligned(p.out)) return false;
  if (p.qkv_stride % 8 != 0 || p.out_stride % 8 != 0) return false;
  if (p.qkv_stride < (long long)(p.n_heads + 2 * p.n_kv_heads) * kHD) return false;
  if (p.out_stride < (long long)p.n_heads * kHD) return false;
  return true;
}

cudaError_t decode_attention(const DecodeAttnParams& p, int batch, int nsplit, cudaStream_t stream) {
  if (p.head_dim != kHD) return cudaErrorInvalidValue;
  if (nsplit > 1 && (!p.scratch || !p.counters)) return cudaErrorInvalidValue;
  if (!decode_attention_layout_ok(p)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, p.n_heads, batch);
  cfg.blockDim = dim3(kThreads, 1, 1);
  static DeviceOnce configured;  // the shared-memory opt-in is a per-device attribute
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDynSmem);
    if (e != cudaSuccess) return e;
    configured.done();
  }
  cfg.dynamicSmemBytes = kDynSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = pdl_launch_attr(&attr[0]);
  // Early L2 prefetch only when the K/V of the whole launch is well below the 126 MB L2 (a tensor-parallel
  // shard): for a full-size cache (268 MB at batch 16 x 32 heads) the hint would only evict itself and was
  // measured to cost 20 % of the step.
  DecodeAttnParams q = p;
  q.prefetch_l2 = pdl_enabled() && (size_t)batch * p.n_kv_heads * p.max_seq * kRowBytes * 2 <= (48u << 20);
  return cudaLaunchKernelEx(&cfg, decode_attention_kernel, q);
}

}  // namespace ccl

// ------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see decode_attention_noalloc.h for who needs it and the
// rules of use). It lives in this file because the scratch array below has file scope and the
// host can only turn the array's name into a device address from the file that defines it.
// ------------------------------------------------------------------------------------------
#include <mutex>
#include <string>

#include "decode_attention_noalloc.h"

namespace {

// Split-KV partials followed by the arrival counters. In host code `g_noalloc_scratch` is only
// a stand-in for the symbol, not a device address: the address comes from
// cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CCL_NOALLOC_SCRATCH_BYTES];

constexpr size_t kNoallocPartialBytes = (size_t)CCL_NOALLOC_MAX_PARTIALS * 130 * 4;
constexpr int kNoallocMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kNoallocMaxDevices] = {};
thread_local std::string g_noalloc_error;

int noalloc_fail(int code, const std::string& msg) {
  g_noalloc_error = msg;
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char* ccl_noalloc_last_error(void) {
  return g_noalloc_error.c_str();
}

extern "C" __attribute__((visibility("default"))) int ccl_decode_attention_noalloc(
    const void* qkv, long long qkv_stride, void* k_cache, void* v_cache, const int* positions, const float* cos,
    const float* sin, void* out, long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
    int max_seq, int nsplit, void* stream) {
  g_noalloc_error.clear();
  if (!qkv || !k_cache || !v_cache || !positions || !cos || !sin || !out)
    return noalloc_fail(2, "ccl_decode_attention_noalloc: null pointer argument");
  if (batch <= 0 || n_heads <= 0 || n_kv_heads <= 0 || nsplit <= 0 || max_seq <= 0 || n_heads % n_kv_heads != 0)
    return noalloc_fail(2, "ccl_decode_attention_noalloc: batch, heads, max_seq and nsplit must be positive and n_heads a multiple of n_kv_heads");
  if (head_dim != 128) return noalloc_fail(2, "ccl_decode_attention_noalloc: head_dim must be 128");
  const long long partials = (long long)batch * n_heads * nsplit;
  if (partials > CCL_NOALLOC_MAX_PARTIALS)
    return noalloc_fail(1, "ccl_decode_attention_noalloc: batch * n_heads * nsplit = " + std::to_string(partials) +
                               " exceeds the built-in scratch of " + std::to_string(CCL_NOALLOC_MAX_PARTIALS) +
                               " partial results; lower nsplit or use the entry point that takes a caller-provided scratch buffer");
  {
    ccl::DecodeAttnParams chk{};
    chk.qkv = static_cast<const __nv_bfloat16*>(qkv);
    chk.qkv_stride = qkv_stride;
    chk.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    chk.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    chk.out = static_cast<__nv_bfloat16*>(out);
    chk.out_stride = out_stride;
    chk.n_heads = n_heads;
    chk.n_kv_heads = n_kv_heads;
    if (!ccl::decode_attention_layout_ok(chk))
      return noalloc_fail(2, "ccl_decode_attention_noalloc: qkv, k_cache, v_cache and out must be 16-byte aligned, qkv_stride and "
                             "out_stride multiples of 8 elements and at least (n_heads + 2 * n_kv_heads) * 128 and n_heads * 128");
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(3, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kNoallocMaxDevices) return noalloc_fail(2, "ccl_decode_attention_noalloc: device index out of range");
  void* base = nullptr;
  {
    // first call on this device: resolve the device address of the built-in array
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p) return noalloc_fail(3, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
      g_noalloc_ptr[dev] = p;
    }
    base = g_noalloc_ptr[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned int* counters = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(base) + kNoallocPartialBytes);
  // the array keeps the previous call's contents: the counters must start at zero
  e = cudaMemsetAsync(counters, 0, (size_t)batch * n_heads * sizeof(unsigned int), s);
  if (e != cudaSuccess) return noalloc_fail(3, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  ccl::DecodeAttnParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.qkv_stride = qkv_stride;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.positions = positions;
  p.cos = cos;
  p.sin = sin;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.scratch = static_cast<float*>(base);
  p.counters = counters;
  p.n_heads = n_heads;
  p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim;
  p.max_seq = max_seq;
  p.scale = 1.0f / sqrtf((float)head_dim);
  e = ccl::decode_attention(p, batch, nsplit, s);
  if (e != cudaSuccess) return noalloc_fail(3, std::string("decode_attention launch: ") + cudaGetErrorString(e));
  return 0;
}
