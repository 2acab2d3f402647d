/* helix_b200/kernels.h: the C interface of the sm_100a kernel library.
 *
 * The engine's entry points for users are the Python package (helix_runtime_b200.Engine) and
 * the command line (bin/helix_generate); the reference exposes its engine to C++ through
 * include/helix (README.md:199-209).  What this project offers to C and C++ callers is the
 * layer below: every kernel the engine runs, as a plain C function of the shared library the
 * package builds (helix_runtime_b200/csrc/_build/libhelix_b200_<hash>.so; CUDA runtime linked
 * statically).  The Python side calls exactly these symbols through ctypes.
 *
 * Conventions.  Every function takes raw device pointers, sizes and the stream to launch on;
 * it allocates nothing (scratch is the caller's; see hx_paged_attention_no_alloc for the one
 * exception that brings its own) and never synchronises.  It returns 0, or a negative code
 * (HX_RC_*) and leaves a message for hx_last_error().  Sizes a kernel cannot run are refused
 * on the host, before any launch: never a wrong result.  Kernels that can detect a bad input
 * on the device (a token id outside the vocabulary, a page number outside the pool, a bounded
 * wait that ran out, a non-finite logit, a position beyond the rotary table) OR a bit into the caller's `status` word
 * (HX_STATUS_*), which the host reads after the step.
 *
 * dtype codes: HX_F32 = 0, HX_BF16 = 1.  Matrices are [rows, row stride] row-major; weights
 * are [out_features, in_features] ("K-major").  Epilogues of the products: 0 store in the
 * activation dtype, 1 store float32, 2 add into float32, 3 SwiGLU (tensor cores only).
 *
 * Cache layout of one layer, keys and values alike:
 *   [page][kv_head][head_dim / c][slot][c]   with c = hx_cache_chunk_elements(dtype, head_dim)
 * (16 bytes of elements when the head size allows), so the keys of a (page, head) are one
 * contiguous block.  Block tables are int32 [rows, table_stride], -1 = no page.
 */
#ifndef HELIX_B200_KERNELS_H
#define HELIX_B200_KERNELS_H

#ifdef __CUDACC__
#include <cuda_runtime.h>
#else
typedef struct CUstream_st* cudaStream_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define HX_RC_ARGUMENT (-1)
#define HX_RC_LAUNCH (-2)
#define HX_RC_UNSUPPORTED (-3)

#define HX_DTYPE_F32 0
#define HX_DTYPE_BF16 1

#define HX_STATUS_BAD_TOKEN 1
#define HX_STATUS_BAD_PAGE 2
#define HX_STATUS_WAIT_TIMEOUT 4
#define HX_STATUS_NONFINITE 8
#define HX_STATUS_BAD_POSITION 16

/* ---- library ---------------------------------------------------------------------------- */
int hx_abi_version(void);
int hx_sm_count(void);                     /* multiprocessors of the current device, 0 on error */
const char* hx_last_error(void);          /* message of this thread's last failed call */
long long hx_launch_count(void);          /* kernels launched by this library so far */
void hx_set_dependent_launch(int enabled); /* programmatic dependent launch between kernels */
/* the kernels' bounded mbarrier wait on a barrier of its own, limited to `polls` polls
   (1..1,000,000): with arrive = 0 it runs out, sets HX_STATUS_WAIT_TIMEOUT in *status and the
   kernel returns; *succeeded (may be null) receives 1 or 0 */
int hx_bounded_wait_check(int polls, int arrive, int* status, int* succeeded, cudaStream_t stream);

/* ---- embedding, norm, activation ------------------------------------------------------- */
/* out[t, :] = table[ids[t], :] as float32 (the residual stream) */
int hx_embed(const void* table, int dtype, const int* ids, float* out, int tokens, int hidden,
             int vocab, int* status, cudaStream_t stream);
/* y[r, :] = x[rows ? rows[r] : r, :] * rsqrt(mean(x^2) + eps) * weight, float32 inside */
int hx_rmsnorm(const float* x, const float* weight, void* y, int out_dtype, const int* rows,
               int n_rows, int hidden, float eps, cudaStream_t stream);
/* act[t, f] = silu(gate_up[t, f]) * gate_up[t, intermediate + f]; zero_input clears gate_up */
int hx_swiglu(float* gate_up, void* act, int out_dtype, int tokens, int intermediate, int ld_in,
              int zero_input, cudaStream_t stream);

/* ---- rotary encoding + cache append ---------------------------------------------------- */
/* qkv row = [q heads | k heads | v heads]; pairing 0: pairs (2p, 2p+1), 1: (p, p + rotary/2).
 * accum != NULL: take the row from this float32 accumulator instead and clear it. */
int hx_rope_append(void* qkv, int dtype, int ld, const int* positions, const int* token_request,
                   const int* request_table_row, const int* block_tables, int table_stride,
                   void* k_cache, void* v_cache, int write_cache, const float* cos_table,
                   const float* sin_table, int table_positions, int tokens, int heads, int kv_heads,
                   int head_dim, int rotary_dim, int pairing, int page_size, int num_pages,
                   int* status, float* accum, int ld_accum, cudaStream_t stream);
/* token_ids[i] = max(sampled[rows[i]], 0): a step takes its tokens from the output of the
 * step before it without a round trip to the host */
int hx_feed_tokens(int* token_ids, const int* sampled, const int* rows, int count,
                   int sampled_rows, cudaStream_t stream);

/* ---- matrix products: out[t, f] (+)= sum_k x[t, k] * w[f, k] ---------------------------- */
/* CUDA cores, float32 accumulate in a fixed order; both dtypes; the true 32-bit path */
int hx_gemm_simt(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int dtype,
                 int tokens, int features, int depth, int epilogue, cudaStream_t stream);
/* tcgen05 tensor cores, bfloat16 operands, float32 accumulate in tensor memory.
 * weight_tiles != 0: w holds the matrix as [ceil(rows / 128)][ceil(depth / 64)] tiles of
 * [128][64] elements, zero padded, each tile 16 contiguous kilobytes (ldw is ignored). */
int hx_gemm_tc_supports(int tokens, int features, int depth, int ldx, int ldw);
int hx_gemm_tc_token_tile(int tokens);
int hx_gemm_tc(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
               int weight_rows, void* out, int ldo, int tokens, int features, int depth,
               int epilogue, int up_row_offset, int k_splits, int weight_tiles, int* status,
               cudaStream_t stream);
/* the fused QKV product of a prompt portion (more than 64 tokens) with rotary encoding and
   cache append as its epilogue: rotated queries to `out`, keys and values to their pages */
int hx_gemm_tc_rope_append_min_tokens(void);
int hx_gemm_tc_rope_append(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                           int weight_rows, void* out, int ldo, int tokens, int depth,
                           int weight_tiles, const int* positions, const int* token_request,
                           const int* request_table_row, const int* block_tables,
                           int table_stride, void* k_cache, void* v_cache, const float* cos_table,
                           const float* sin_table, int table_positions, int heads, int kv_heads,
                           int head_dim, int rotary_dim, int page_size, int num_pages, int* status,
                           cudaStream_t stream);

/* ---- attention over the paged cache ----------------------------------------------------- */
int hx_cache_chunk_elements(int dtype, int head_dim);
long long hx_paged_attention_scratch_floats(int tokens, int heads, int head_dim, int max_splits);
/* the same when the caller says which case it has (the streaming kernel needs less) */
long long hx_paged_attention_scratch_floats_for(int dtype, int tokens, int heads, int head_dim,
                                                int page_size, int window, int max_splits);
/* every query token over the keys [position - window + 1 (or 0), position] of its request */
int hx_paged_attention(const void* q, int ldq, const void* k_cache, const void* v_cache, int dtype,
                       const int* positions, const int* token_request,
                       const int* request_table_row, const int* block_tables, int table_stride,
                       const int* request_start, int skip_query_len, void* out, int ldo,
                       float* partial, int* arrivals, int tokens, int heads, int kv_heads,
                       int head_dim, int page_size, int num_pages, int window, float scale,
                       int split_keys, int max_splits, int* status, cudaStream_t stream);
/* the same with scratch built into the library: see hx_no_alloc.h beside the sources */
int hx_paged_attention_no_alloc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                int dtype, const int* positions, const int* token_request,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, const int* request_start, int skip_query_len,
                                void* out, int ldo, int tokens, int heads, int kv_heads,
                                int head_dim, int page_size, int num_pages, int window, float scale,
                                int split_keys, int max_splits, int* status, cudaStream_t stream);
/* prompt portions on the tensor cores (bfloat16, head sizes in steps of 16 up to 128 and of
   32 up to 256) */
int hx_prefill_attention_supports(int head_dim, int page_size);
int hx_prefill_attention(const void* q, int ldq, const void* k_cache, const void* v_cache,
                         const int* request_start, const int* request_context,
                         const int* request_table_row, const int* block_tables, int table_stride,
                         void* out, int ldo, int requests, int tile_bound, int heads, int kv_heads,
                         int head_dim, int page_size, int num_pages, float scale, int min_query_len,
                         int* status, cudaStream_t stream);

/* the same on tcgen05, scores and partial outputs in tensor memory (pages of 16, 32, 64) */
int hx_prefill_attention_tc_supports(int head_dim, int page_size);
int hx_prefill_attention_tc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                            const int* request_start, const int* request_context,
                            const int* request_table_row, const int* block_tables,
                            int table_stride, void* out, int ldo, int requests, int tile_bound,
                            int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                            float scale, int min_query_len, int* status, cudaStream_t stream);

/* ---- sampling --------------------------------------------------------------------------- */
/* lowest id among the maxima; -1 and HX_STATUS_NONFINITE for a row with a non-finite logit */
int hx_argmax(const float* logits, int ld, int rows, int vocab, int* tokens, int* status,
              cudaStream_t stream);
/* inverse-CDF draw from softmax(logits / temperature) with the caller's uniform numbers;
 * temperature 0 is the greedy rule */
int hx_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
              const float* uniform, int* tokens, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HELIX_B200_KERNELS_H */
