// hx_paged_attention_no_alloc: paged attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project.  It exists for users of the
// kernel library who have to run attention without handing it scratch memory:
//
//   * a serving process that gave all device memory to weights and the cache pool when it
//     started: there is nothing left to allocate from, and a request must not fail on that;
//   * code on a latency-critical path: cudaMalloc and cudaFree stall the whole device;
//   * callers from C or through a foreign-function interface, who have no caching allocator
//     and would otherwise have to size and keep the scratch buffer themselves.
//
// What it does.  The same computation, by the same kernels, as hx_paged_attention (see
// hx_attention.cu), with the split-K scratch (partial sums and arrival counters) taken from
// one array that is compiled into the library instead of from the caller.  Inputs and the
// output are still the caller's.  It calls no cudaMalloc, no cudaFree and no other routine
// that allocates.
//
// Limits.  The array holds HX_NO_ALLOC_PARTIAL_WORDS floats of partial sums and
// HX_NO_ALLOC_COUNTER_WORDS counters (tokens * heads must fit): 4.5 MiB in all, resident on
// every GPU that loads the library until the process exits.  How many partial sums a call
// needs depends on the kernel that serves it (hx_paged_attention_scratch_floats_for()):
//   * bfloat16, no window, pages of 8, 16 or 32 keys, head sizes in steps of 16 up to 128 and
//     of 32 up to 256 (the streaming kernel): a fixed amount that always fits, whatever the
//     number of tokens, heads and splits;
//   * everything else (float32, a window, other page or head sizes; the CUDA-core kernel):
//     tokens * heads * max_splits * (head_dim + 2) floats when max_splits > 1, which must fit.
//     At 32 heads of 128 that is tokens * max_splits <= 267: eight tokens cut into 32 splits.
// A call that needs more is refused with an error message that says how much it needed;
// nothing is launched then.
//
// Set-up.  The first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first call
// outside of any stream capture.
//
// Sharing.  All calls use the same array and find in it what the previous call left.  The
// partial sums are always written before they are read; the counters have to start at zero
// and are cleared in stream order at the start of every call.  Two calls whose kernels may
// run at the same time on one GPU (different streams, or different threads) would use the
// same scratch at once and corrupt each other's results: keep calls on one GPU in one
// stream, or order them yourself.
//
// Returns 0, or a negative code with a message for hx_last_error().
#pragma once

#include <cuda_runtime.h>

#define HX_NO_ALLOC_PARTIAL_WORDS (17 << 16)
#define HX_NO_ALLOC_COUNTER_WORDS (1 << 16)
#define HX_NO_ALLOC_SCRATCH_WORDS (HX_NO_ALLOC_PARTIAL_WORDS + HX_NO_ALLOC_COUNTER_WORDS)

#ifdef __cplusplus
extern "C" {
#endif

int hx_paged_attention_no_alloc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                int dtype, const int* positions, const int* token_request,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, const int* request_start, int skip_query_len,
                                void* out, int ldo, int tokens, int heads, int kv_heads,
                                int head_dim, int page_size, int num_pages, int window, float scale,
                                int split_keys, int max_splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
