// C interface of attention_mma.cu that is meant for callers outside this package.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Decode attention without any allocation.  This entry point has no counterpart in
// jtiro232/Alpacca (which has no GPU code and allocates freely in Python); it exists for
// callers of this library that cannot allocate device memory at the time of the call:
// a plug-in that runs inside another program's serving loop with a memory budget that
// was fixed at start-up, a binding from a language that has no allocator of its own for
// the device, a latency-critical loop that must not meet the device-wide
// synchronisation that cudaMalloc and cudaFree imply.
//
// It computes what ab_attention_decode_bf16 computes (one new token per sequence over
// the paged cache, bfloat16) from the same inputs into the same output.  The scratch
// memory that the split over key chunks needs (partial outputs, their running maxima
// and sums, arrival counters) is not passed in: it is a fixed array inside the
// library, AB_DECODE_NOALLOC_SCRATCH_BYTES large, which every GPU that loads the
// library holds until the process ends.  The call itself uses no cudaMalloc, cudaFree
// or allocating library routine.
//
// Limits: n_tokens * H * n_chunks * D <= AB_DECODE_NOALLOC_MAX_PARTIAL floats and
// n_tokens * K * ceil(H / K / 8) <= AB_DECODE_NOALLOC_MAX_COUNTERS; larger problems
// are refused with AB_NOALLOC_TOO_LARGE (the message of ab_attention_decode_bf16_noalloc_error
// names the limit).  Use ab_attention_decode_bf16 with your own scratch for those.
//
// The first call on a device looks up the device address of the scratch array (the
// array's name in host code is only a handle, not an address a kernel could use) and
// remembers it for that device; make that first call with the device current and
// before any stream capture begins.  All calls share the one array: the arrival
// counters are cleared on the stream at the start of every call, the rest is
// overwritten before it is read.  Two calls that overlap on the GPU (different
// streams, or the same call from two threads) race on it: serialise them.
#define AB_DECODE_NOALLOC_MAX_PARTIAL (1u << 20)
#define AB_DECODE_NOALLOC_MAX_COUNTERS (1u << 16)
#define AB_DECODE_NOALLOC_SCRATCH_BYTES \
  (AB_DECODE_NOALLOC_MAX_PARTIAL * 4u + (AB_DECODE_NOALLOC_MAX_PARTIAL / 8u) * 4u + AB_DECODE_NOALLOC_MAX_COUNTERS * 4u)
#define AB_NOALLOC_TOO_LARGE 2

int ab_attention_decode_bf16_noalloc(const void* qkv, int q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* block_table, int table_width,
                                     const int* tok_seq, const int* kv_len, int n_tokens, int H, int K, int D,
                                     float scale, int window, int pages_per_cta, int n_chunks, cudaStream_t stream);

// Text for the last non-zero code that ab_attention_decode_bf16_noalloc returned in this thread.
const char* ab_attention_decode_bf16_noalloc_error(void);

#ifdef __cplusplus
}
#endif
