// The element loops of this file want the vectoriser at full strength whatever the build's
// global level is (the rest of the host code stays at -O2).
#if defined(__GNUC__) && !defined(__clang__)
#pragma GCC optimize("O3")
#endif
#include "cpu/CpuCollectives.h"

#include <c10/util/BFloat16.h>
#include <c10/util/Half.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>

#include "cuda/kernels/collectives.h"  // DType / ReduceKind numbering shared with the GPU path

namespace ccl {
namespace cpu {

namespace {

constexpr size_t kOneShotBytes = 64 << 10;

template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<c10::Half> { using type = float; };
template <> struct AccOf<c10::BFloat16> { using type = float; };

template <typename A>
inline A combine(int kind, A a, A b) {
  switch (kind) {
    case kSum: return a + b;
    case kProd: return a * b;
    case kMin: return b < a ? b : a;
    case kMax: return b > a ? b : a;
    default:
      if constexpr (std::is_integral<A>::value) {
        if (kind == kBand) return a & b;
        if (kind == kBor) return a | b;
        if (kind == kBxor) return a ^ b;
      }
      return a + b;
  }
}

// dst[i] = scale(op over s of srcs[s][i]); dst may alias one of the sources.
// The reduce kind and the number of sources are resolved outside the element loop (KIND as a
// template argument, common source counts unrolled), so that the loop body is branch-free and the
// compiler can vectorise it.
// MODE: 0 = plain, 1 = multiply the accumulator by `f`, 2 = divide it by `f` (average) - applied
// before the single rounding to T.
template <typename T, int KIND, int NS, int MODE>
void reduce_loop(T* dst, const void* const* srcs, size_t ns_dyn, size_t count, typename AccOf<T>::type f) {
  using A = typename AccOf<T>::type;
  const size_t ns = NS > 0 ? (size_t)NS : ns_dyn;
  for (size_t i = 0; i < count; ++i) {
    A acc = static_cast<A>(static_cast<const T*>(srcs[0])[i]);
    for (size_t s = 1; s < ns; ++s) acc = combine<A>(KIND, acc, static_cast<A>(static_cast<const T*>(srcs[s])[i]));
    if (MODE == 1) acc = static_cast<A>(acc * f);
    if (MODE == 2) acc = static_cast<A>(acc / f);
    dst[i] = static_cast<T>(acc);
  }
}

template <typename T, int KIND, int MODE>
void reduce_kind(T* dst, const void* const* srcs, size_t ns, size_t count, typename AccOf<T>::type f) {
  switch (ns) {
    case 2: return reduce_loop<T, KIND, 2, MODE>(dst, srcs, ns, count, f);
    case 4: return reduce_loop<T, KIND, 4, MODE>(dst, srcs, ns, count, f);
    case 8: return reduce_loop<T, KIND, 8, MODE>(dst, srcs, ns, count, f);
    default: return reduce_loop<T, KIND, 0, MODE>(dst, srcs, ns, count, f);
  }
}

template <typename T, int MODE>
void reduce_mode(T* dst, const void* const* sp, size_t ns, size_t count, int kind, typename AccOf<T>::type f) {
  switch (kind) {
    case kProd: return reduce_kind<T, kProd, MODE>(dst, sp, ns, count, f);
    case kMin: return reduce_kind<T, kMin, MODE>(dst, sp, ns, count, f);
    case kMax: return reduce_kind<T, kMax, MODE>(dst, sp, ns, count, f);
    case kBand: return reduce_kind<T, kBand, MODE>(dst, sp, ns, count, f);
    case kBor: return reduce_kind<T, kBor, MODE>(dst, sp, ns, count, f);
    case kBxor: return reduce_kind<T, kBxor, MODE>(dst, sp, ns, count, f);
    default: return reduce_kind<T, kSum, MODE>(dst, sp, ns, count, f);
  }
}

template <typename T>
void reduce_typed(T* dst, const std::vector<const void*>& srcs, size_t count, const ReduceDesc& rd, int world) {
  using A = typename AccOf<T>::type;
  const void* const* sp = srcs.data();
  const size_t ns = srcs.size();
  if (!rd.has_scale) return reduce_mode<T, 0>(dst, sp, ns, count, rd.kind, A(1));
  if (rd.is_avg) return reduce_mode<T, 2>(dst, sp, ns, count, rd.kind, static_cast<A>(world));
  if constexpr (std::is_integral<A>::value) {
    return reduce_mode<T, 0>(dst, sp, ns, count, rd.kind, A(1));  // integer PREMUL_SUM is scaled by the caller
  } else {
    return reduce_mode<T, 1>(dst, sp, ns, count, rd.kind, static_cast<A>(rd.scale));
  }
}

void reduce_any(void* dst, const std::vector<const void*>& srcs, size_t count, const ReduceDesc& rd, int world) {
  switch (rd.dtype) {
    case kU8: return reduce_typed(static_cast<uint8_t*>(dst), srcs, count, rd, world);
    case kI8: return reduce_typed(static_cast<int8_t*>(dst), srcs, count, rd, world);
    case kI16: return reduce_typed(static_cast<int16_t*>(dst), srcs, count, rd, world);
    case kI32: return reduce_typed(static_cast<int32_t*>(dst), srcs, count, rd, world);
    case kI64: return reduce_typed(static_cast<int64_t*>(dst), srcs, count, rd, world);
    case kF16: return reduce_typed(static_cast<c10::Half*>(dst), srcs, count, rd, world);
    case kBF16: return reduce_typed(static_cast<c10::BFloat16*>(dst), srcs, count, rd, world);
    case kF32: return reduce_typed(static_cast<float*>(dst), srcs, count, rd, world);
    case kF64: return reduce_typed(static_cast<double*>(dst), srcs, count, rd, world);
    default: throw std::runtime_error("ccl: unsupported dtype in CPU reduction");
  }
}

struct Seg { size_t e0, e1; };
inline Seg segment(size_t n, int world, int r) {
  const size_t per = (n + world - 1) / world;
  const size_t e0 = std::min(n, per * (size_t)r);
  return {e0, std::min(n, e0 + per)};
}

// Shared body of allreduce (root < 0) and reduce (root >= 0).
void reduce_impl(ShmComm& c, void* buf, size_t count, const ReduceDesc& rd, int root, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t esz = dtype_size(rd.dtype);
  const size_t cap = c.slot_bytes() / esz;
  char* p = static_cast<char*>(buf);
  const bool want = root < 0 || root == me;
  size_t done = 0;
  do {
    const size_t n = std::min(cap, count - done);
    c.next_step();
    std::memcpy(c.slot(me), p + done * esz, n * esz);
    c.barrier(timeout);
    std::vector<const void*> srcs(W);
    if (n * esz <= kOneShotBytes) {
      if (want) {
        for (int r = 0; r < W; ++r) srcs[r] = c.slot(r);
        reduce_any(p + done * esz, srcs, n, rd, W);
      }
    } else {
      const Seg s = segment(n, W, me);
      for (int r = 0; r < W; ++r) srcs[r] = c.slot(r) + s.e0 * esz;
      reduce_any(c.slot(me) + s.e0 * esz, srcs, s.e1 - s.e0, rd, W);
      c.barrier(timeout);
      if (want)
        for (int r = 0; r < W; ++r) {
          const Seg q = segment(n, W, r);
          std::memcpy(p + (done + q.e0) * esz, c.slot(r) + q.e0 * esz, (q.e1 - q.e0) * esz);
        }
    }
    done += n;
  } while (done < count);
  // Slots alternate between two halves; a rank can reach the step after next only after all
  // ranks passed the barrier of the next step, i.e. finished reading this one.
}

}  // namespace

void allreduce(ShmComm& c, void* buf, size_t count, const ReduceDesc& rd, Ms timeout) {
  reduce_impl(c, buf, count, rd, -1, timeout);
}

void reduce(ShmComm& c, void* buf, size_t count, const ReduceDesc& rd, int root, Ms timeout) {
  reduce_impl(c, buf, count, rd, root, timeout);
  // a rooted op lets non-root ranks run ahead; keep them within one step of the root
  c.next_step();
  c.barrier(timeout);
}

void broadcast(ShmComm& c, void* buf, size_t bytes, int root, Ms timeout) {
  const int me = c.rank();
  const size_t cap = c.slot_bytes();
  char* p = static_cast<char*>(buf);
  size_t done = 0;
  do {
    const size_t n = std::min(cap, bytes - done);
    c.next_step();
    if (me == root) std::memcpy(c.slot(root), p + done, n);
    c.barrier(timeout);
    if (me != root) std::memcpy(p + done, c.slot(root), n);
    done += n;
  } while (done < bytes);
  c.next_step();
  c.barrier(timeout);
}

void allgatherv(ShmComm& c, const void* in, const std::vector<void*>& outs, const std::vector<size_t>& bytes, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t cap = c.slot_bytes();
  const size_t mx = *std::max_element(bytes.begin(), bytes.end());
  size_t done = 0;
  do {
    c.next_step();
    if (done < bytes[me]) std::memcpy(c.slot(me), static_cast<const char*>(in) + done, std::min(cap, bytes[me] - done));
    c.barrier(timeout);
    for (int r = 0; r < W; ++r) {
      if (done >= bytes[r]) continue;
      const size_t n = std::min(cap, bytes[r] - done);
      char* dst = static_cast<char*>(outs[r]) + done;
      if (r == me) {
        if (dst != static_cast<const char*>(in) + done) std::memmove(dst, static_cast<const char*>(in) + done, n);
      } else {
        std::memcpy(dst, c.slot(r), n);
      }
    }
    done += cap;
  } while (done < mx);
}

void gather(ShmComm& c, const void* in, const std::vector<void*>& outs, size_t bytes, int root, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t cap = c.slot_bytes();
  size_t done = 0;
  do {
    const size_t n = std::min(cap, bytes - done);
    c.next_step();
    if (me != root) std::memcpy(c.slot(me), static_cast<const char*>(in) + done, n);
    c.barrier(timeout);
    if (me == root)
      for (int r = 0; r < W; ++r) {
        const char* src = (r == me) ? static_cast<const char*>(in) + done : c.slot(r);
        char* dst = static_cast<char*>(outs[r]) + done;
        if (dst != src) std::memmove(dst, src, n);
      }
    done += n;
  } while (done < bytes);
  c.next_step();
  c.barrier(timeout);
}

void scatter(ShmComm& c, const std::vector<const void*>& ins, void* out, size_t bytes, int root, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t cap = c.slot_bytes() / W / 64 * 64;
  if (cap == 0) throw std::runtime_error("ccl: shared-memory slot too small for scatter");
  size_t done = 0;
  do {
    const size_t n = std::min(cap, bytes - done);
    c.next_step();
    if (me == root)
      for (int r = 0; r < W; ++r)
        if (r != me) std::memcpy(c.slot(root) + (size_t)r * cap, static_cast<const char*>(ins[r]) + done, n);
    c.barrier(timeout);
    if (me == root) {
      const char* src = static_cast<const char*>(ins[me]) + done;
      if (src != static_cast<char*>(out) + done) std::memmove(static_cast<char*>(out) + done, src, n);
    } else {
      std::memcpy(static_cast<char*>(out) + done, c.slot(root) + (size_t)me * cap, n);
    }
    done += n;
  } while (done < bytes);
  c.next_step();
  c.barrier(timeout);
}

void reduce_scatterv(ShmComm& c, const std::vector<const void*>& ins, void* out, const std::vector<size_t>& counts,
                     const ReduceDesc& rd, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t esz = dtype_size(rd.dtype);
  const size_t cap = c.slot_bytes() / W / 64 * 64 / esz;  // elements per piece and step
  if (cap == 0) throw std::runtime_error("ccl: shared-memory slot too small for reduce_scatter");
  const size_t mx = *std::max_element(counts.begin(), counts.end());
  size_t done = 0;
  do {
    c.next_step();
    for (int r = 0; r < W; ++r) {
      if (r == me || done >= counts[r]) continue;
      std::memcpy(c.slot(me) + (size_t)r * cap * esz, static_cast<const char*>(ins[r]) + done * esz,
                  std::min(cap, counts[r] - done) * esz);
    }
    c.barrier(timeout);
    if (done < counts[me]) {
      const size_t n = std::min(cap, counts[me] - done);
      std::vector<const void*> srcs(W);
      for (int r = 0; r < W; ++r)
        srcs[r] = (r == me) ? static_cast<const char*>(ins[me]) + done * esz : c.slot(r) + (size_t)me * cap * esz;
      reduce_any(static_cast<char*>(out) + done * esz, srcs, n, rd, W);
    }
    done += cap;
  } while (done < mx);
}

void alltoallv(ShmComm& c, const std::vector<const void*>& ins, const std::vector<size_t>& send_bytes,
               const std::vector<void*>& outs, const std::vector<size_t>& recv_bytes, Ms timeout) {
  const int W = c.world(), me = c.rank();
  const size_t cap = c.slot_bytes() / W / 64 * 64;
  if (cap == 0) throw std::runtime_error("ccl: shared-memory slot too small for alltoall");
  // agree on the number of steps: the largest pair-wise piece of the whole group
  c.next_step();
  size_t mine = 0;
  for (int r = 0; r < W; ++r) mine = std::max(mine, send_bytes[r]);
  c.scratch()[me] = mine;
  c.barrier(timeout);
  size_t mx = 0;
  for (int r = 0; r < W; ++r) mx = std::max(mx, (size_t)c.scratch()[r]);
  size_t done = 0;
  while (done < mx) {
    c.next_step();
    for (int r = 0; r < W; ++r) {
      if (r == me || done >= send_bytes[r]) continue;
      std::memcpy(c.slot(me) + (size_t)r * cap, static_cast<const char*>(ins[r]) + done, std::min(cap, send_bytes[r] - done));
    }
    c.barrier(timeout);
    for (int r = 0; r < W; ++r) {
      if (done >= recv_bytes[r]) continue;
      const size_t n = std::min(cap, recv_bytes[r] - done);
      char* dst = static_cast<char*>(outs[r]) + done;
      if (r == me) {
        const char* src = static_cast<const char*>(ins[me]) + done;
        if (src != dst) std::memmove(dst, src, n);
      } else {
        std::memcpy(dst, c.slot(r) + (size_t)me * cap, n);
      }
    }
    done += cap;
  }
  c.next_step();
  c.barrier(timeout);
}

void barrier(ShmComm& c, Ms timeout) {
  c.next_step();
  c.barrier(timeout);
}

}  // namespace cpu
}  // namespace ccl
