// Collective algorithms on CPU tensors over a ShmComm: every rank copies its contribution into
// its own staging slot, ranks meet at a sequence barrier, and each rank then reads what it
// needs from the other slots. Large messages are processed in slot-sized steps; reductions
// use a two-shot schedule (each rank reduces one segment, then all copy every segment) above a
// small-message threshold. Reductions of f16/bf16 accumulate in fp32.
//
// Covers the 14 ops of the reference CPU stub (src/cpu/cpu_ccl.cpp:306-1076) plus send/recv,
// reduce_scatter_tensor_coalesced, AVG / PREMUL_SUM and the bitwise ops, which the reference
// CPU path lacks (README.md:24-25; src/utils.cpp:38-44).
#pragma once
#include <chrono>
#include <cstddef>
#include <vector>

#include "cpu/ShmComm.h"

namespace ccl {
namespace cpu {

struct ReduceDesc {
  int dtype;      // ccl::DType numbering
  int kind;       // ccl::ReduceKind numbering
  bool has_scale = false;
  bool is_avg = false;
  double scale = 1.0;
};

using Ms = std::chrono::milliseconds;

void allreduce(ShmComm& c, void* buf, size_t count, const ReduceDesc& rd, Ms timeout);
// In-place on root; other ranks' buffers are left untouched.
void reduce(ShmComm& c, void* buf, size_t count, const ReduceDesc& rd, int root, Ms timeout);
void broadcast(ShmComm& c, void* buf, size_t bytes, int root, Ms timeout);
// Piece p (bytes[p] bytes) of every rank lands in outs[p]; `in` holds bytes[rank] bytes.
void allgatherv(ShmComm& c, const void* in, const std::vector<void*>& outs, const std::vector<size_t>& bytes, Ms timeout);
// Root receives `bytes` from every rank into outs[p]; non-root outs is empty.
void gather(ShmComm& c, const void* in, const std::vector<void*>& outs, size_t bytes, int root, Ms timeout);
void scatter(ShmComm& c, const std::vector<const void*>& ins, void* out, size_t bytes, int root, Ms timeout);
// Rank r receives the reduction of everybody's piece r: ins[p] has counts[p] elements.
void reduce_scatterv(ShmComm& c, const std::vector<const void*>& ins, void* out, const std::vector<size_t>& counts,
                     const ReduceDesc& rd, Ms timeout);
// Piece p of the input (send_bytes[p]) goes to rank p; recv_bytes[p] arrives from rank p.
void alltoallv(ShmComm& c, const std::vector<const void*>& ins, const std::vector<size_t>& send_bytes,
               const std::vector<void*>& outs, const std::vector<size_t>& recv_bytes, Ms timeout);
void barrier(ShmComm& c, Ms timeout);

}  // namespace cpu
}  // namespace ccl
