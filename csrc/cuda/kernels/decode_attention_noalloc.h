// ccl_decode_attention_noalloc: the split-KV decode attention with its scratch memory built in.
//
// This entry point has no counterpart in intel/torch-ccl. It exists for callers that are handed
// raw device pointers and a stream but must not allocate device memory themselves: a custom op
// hosted by an inference server whose memory pool belongs to the host framework, a step that
// runs while another library is capturing a CUDA graph on the device (cudaMalloc would be illegal
// or would synchronise the whole GPU there), or a process that has been given a fixed memory
// slice and is not allowed to grow it. The regular entry point (ccl::decode_attention) needs the
// caller to supply a scratch buffer for the split-KV partial results and a counter array; here
// both live in a file-scope `static __device__` array inside the library, so the call allocates
// nothing: no cudaMalloc / cudaFree, no torch allocator, no allocating library routine.
//
// What to know before using it:
//   * Limit: batch * n_heads * nsplit <= CCL_NOALLOC_MAX_PARTIALS (4096). A larger request is
//     rejected with an error code and a message (ccl_noalloc_last_error); nothing is launched.
//   * The built-in scratch costs CCL_NOALLOC_SCRATCH_BYTES (about 2.1 MiB) of device memory on
//     every GPU that loads this library, from load until the process exits.
//   * The first call on each device looks up the device address of the built-in array
//     (cudaGetSymbolAddress, with that device current) and caches it. Make that first call
//     outside any stream capture.
//   * Every call on a device shares the same array, which still holds whatever the previous call
//     left there. The entry point clears the part that has to start at zero (the arrival
//     counters) on the caller's stream before launching. Two calls that overlap on the same GPU
//     (different streams, or different threads) race on the array: serialise them.
//   * Inputs and outputs are the caller's, exactly as for the regular entry point: qkv, the two
//     caches and out 16-byte aligned, both row strides multiples of 8 elements and no shorter
//     than a row. A call that breaks this returns 2 and launches nothing. A position outside
//     [0, max_seq) gives a zero output row and leaves the caches alone.
//   * Several GPUs in one process: each device resolves the array and configures the kernel on
//     its own first call, with that device current.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CCL_NOALLOC_MAX_PARTIALS 4096
// partials: 4096 * (128 + 2) floats; counters: 4096 uint32, rounded up to 256 bytes
#define CCL_NOALLOC_SCRATCH_BYTES (4096 * 130 * 4 + 4096 * 4)

// qkv:        [batch, qkv_stride] bf16: q heads, then k heads, then v heads of the new token
// k_cache/v_cache: [batch, n_kv_heads, max_seq, 128] bf16
// positions:  [batch] int32, position of the new token; cos/sin: [max_seq, 64] fp32 rotary tables
// out:        [batch, out_stride] bf16, n_heads * 128 values per row
// stream:     a cudaStream_t (0 = default stream)
// Returns 0 on success; 1 = size beyond the built-in scratch, 2 = bad argument, 3 = CUDA error.
int ccl_decode_attention_noalloc(const void* qkv, long long qkv_stride, void* k_cache, void* v_cache,
                                 const int* positions, const float* cos, const float* sin, void* out,
                                 long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                 int max_seq, int nsplit, void* stream);

// Message of the last failing call on this thread ("" if none).
const char* ccl_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
