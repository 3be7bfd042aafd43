// Host interface of the fused RoPE + KV-append + split-KV decode attention kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace ccl {

struct DecodeAttnParams {
  const __nv_bfloat16* qkv;  // [batch, qkv_stride]: q heads, then k heads, then v heads of the new token
  long long qkv_stride;
  __nv_bfloat16* k_cache;    // [batch, n_kv_heads, max_seq, head_dim]
  __nv_bfloat16* v_cache;
  const int* positions;      // [batch] position of the new token (= tokens already cached)
  const float* cos;          // [max_seq, head_dim/2] rotary tables
  const float* sin;
  __nv_bfloat16* out;        // [batch, out_stride]: n_heads * head_dim values per row
  long long out_stride;
  float* scratch;            // split-KV partials: decode_attention_scratch_bytes(); unused if nsplit == 1
  unsigned int* counters;    // [batch * n_heads], zero-initialised once; the kernel re-zeroes them
  int n_heads, n_kv_heads, head_dim, max_seq;
  float scale;               // 1/sqrt(head_dim)
  int* status = nullptr;     // optional device error word (set if a bounded wait expires)
  int prefetch_l2 = 0;       // set by decode_attention(): the launch's whole K/V fits L2 comfortably, so every CTA
                             // pulls its range towards L2 while the kernel before it is still running
};

size_t decode_attention_scratch_bytes(int batch, int n_heads, int nsplit);
int decode_attention_default_splits(int batch, int n_heads, int max_context);
// Pointer alignment (16 bytes) and row-stride rules of the kernel; decode_attention() refuses a
// launch that breaks them with cudaErrorInvalidValue. A position outside [0, max_seq) is caught on
// the device: that sequence's output row is zero, its cache is untouched and `status` (if given)
// is set to 201.
bool decode_attention_layout_ok(const DecodeAttnParams& p);
cudaError_t decode_attention(const DecodeAttnParams& p, int batch, int nsplit, cudaStream_t stream);

}  // namespace ccl
