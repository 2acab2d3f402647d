// Paged causal attention for prompt portions on the tensor cores (bfloat16 storage).
//
// One CTA takes 64 consecutive query tokens of one request and one head; its four warps own
// 16 query rows each and walk the request's keys in tiles of 64, anchored at key 0, with
// the online softmax of flash attention: S = Q K^T on the tensor cores (bf16 products,
// float32 sums), running maximum, exp and running sum in float32 registers, O += P V on the
// tensor cores.  The probabilities are fed to the second product as TWO bfloat16 terms
// (P = hi + lo), so they keep about 16 bits instead of 8 and the softmax stays a float32
// quantity as far as the result can tell.  The reference materialises a [heads, T, T] score
// tensor for the same computation (src/attention/cuda.cu:31-77, src/model/cuda_llama.cpp:249).
//
// Keys and values come straight from the pages: the keys of a (page, head) are one contiguous
// block of the cache and so are its values, so a 64-key tile is a handful of bulk copies
// (cp.async.bulk counted on an mbarrier) issued by one thread, two tiles in flight, and the
// tensor-core loads (ldmatrix) read the page blocks as they lie.  Value rows beyond the last
// key any query of the CTA may see are cleared in shared memory, so a stale or poisoned page
// cannot leak in through a zero probability.
//
// A query row's result depends on its own position only: key tiles are anchored at key 0
// and rows of a tile do not interact, so it does not matter which tile a token falls into
// or what else is in the batch.
//
// Requests with fewer than `min_query_len` tokens in the step are left to the CUDA-core
// kernel (hx_paged_attention skips the others), so decode tokens beside prompt portions
// are each handled by the kernel that suits them.
#include "hx_mma.cuh"

namespace {

constexpr int BLOCK_M = 64;   // query rows per CTA
constexpr int BLOCK_N = 64;   // keys per tile
constexpr int THREADS = 128;

struct PrefillArgs {
  const __nv_bfloat16* q;
  int ldq;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* request_start;     // [requests + 1] first token of each request in the batch
  const int* request_context;   // [requests] tokens cached before this step
  const int* request_table_row;
  const int* block_tables;
  int table_stride;
  __nv_bfloat16* out;
  int ldo;
  int requests;
  int heads;
  int kv_heads;
  int page_size;
  int num_pages;
  float scale;
  int min_query_len;
  int* status;
};

constexpr int RING = 2;                         // key/value tiles in flight per CTA
constexpr uint32_t WAIT_LIMIT = 20u * 1000u * 1000u;

__device__ __forceinline__ bool tile_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t address = hx_shared_address(bar);
  for (uint32_t spin = 0; spin < WAIT_LIMIT; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(address), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(hx_shared_address(bar))
      : "memory");
}

// Byte offset, inside the key (or value) half of a tile, of the 16-byte piece that holds
// coordinates 8c..8c+7 of key `key`: the half is 64 / page_size page blocks, each laid out
// [D/8][page_size][8] exactly as in the cache.
__device__ __forceinline__ uint32_t piece_offset(int key, int c, int page_size,
                                                 uint32_t page_bytes) {
  return (key / page_size) * page_bytes + ((c * page_size + key % page_size) << 4);
}

// CTAs per SM the register budget is set for: three up to a head size of 128, one above
// (the output accumulator of a thread is D / 2 floats).
template <int D>
__global__ __launch_bounds__(THREADS, D <= 128 ? 3 : 1) void prefill_attention_kernel(PrefillArgs a) {
  constexpr int kHalfBytes = BLOCK_N * D * 2;      // keys (or values) of a 64-key tile
  constexpr int kDSteps = D / 16;                  // k-steps of Q K^T
  constexpr int kOBlocks = D / 8;                  // n-blocks of the output
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[RING];
  __shared__ int tile_state[RING];                 // 1: a page of the tile could not be read
  hx_pdl_prologue();

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (a.heads / a.kv_heads);

  // which request and which 64-row tile of it is this CTA?
  int tile_in_request = 0, tiles_of_request = 0;
  const int request = hx_find_query_tile(a.request_start, a.requests, a.min_query_len, BLOCK_M,
                                         blockIdx.x, tile_in_request, tiles_of_request);
  if (request < 0) return;
  const int q_begin = a.request_start[request];
  const int q_len = a.request_start[request + 1] - q_begin;
  const int context = a.request_context[request];
  const int row0 = tile_in_request * BLOCK_M;                 // first query row of the tile
  const int rows_here = min(BLOCK_M, q_len - row0);
  const int last_key = context + row0 + rows_here - 1;        // last key any row here sees
  const int n_tiles = last_key / BLOCK_N + 1;
  const int* table = a.block_tables +
                     static_cast<size_t>(a.request_table_row[request]) * a.table_stride;
  const int page_size = a.page_size;
  const int pages_per_tile = BLOCK_N / page_size;
  const uint32_t page_bytes = static_cast<uint32_t>(page_size) * D * 2;
  const int last_page = last_key / page_size;

  if (tid == 0) {
    for (int s = 0; s < RING; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(hx_shared_address(&full_bar[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // one thread asks for the pages of a tile: two bulk copies (keys, values) per page
  auto request_tile = [&](int tile) {
    const int stage = tile % RING;
    const uint32_t base = hx_shared_address(smem) + stage * 2 * kHalfBytes;
    int pages[8];
    uint32_t expected = 0;
    int unreadable = 0;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      pages[p] = -1;
      const int index = tile * pages_per_tile + p;
      if (p < pages_per_tile && index <= last_page) {
        const int page = table[index];
        if (page >= 0 && page < a.num_pages) {
          pages[p] = page;
          expected += 2 * page_bytes;
        } else {
          unreadable = 1;
        }
      }
    }
    tile_state[stage] = unreadable;
    if (unreadable && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                     hx_shared_address(&full_bar[stage])), "r"(expected) : "memory");
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      if (pages[p] >= 0) {
        const size_t block = (static_cast<size_t>(pages[p]) * a.kv_heads + kv_head) * page_bytes;
        bulk_copy(base + p * page_bytes, reinterpret_cast<const uint8_t*>(a.k_cache) + block,
                  page_bytes, &full_bar[stage]);
        bulk_copy(base + kHalfBytes + p * page_bytes,
                  reinterpret_cast<const uint8_t*>(a.v_cache) + block, page_bytes, &full_bar[stage]);
      }
    }
  };
  if (tid == 0) {
    for (int t = 0; t < RING && t < n_tiles; ++t) request_tile(t);
  }
  __syncthreads();      // tile_state of the first tiles is visible to every warp

  // ---- the query rows of this warp, straight from global memory into A fragments:
  // this thread owns rows (lane / 4) and (lane / 4 + 8) of its warp's 16
  const int warp_row = warp * 16;
  uint32_t q_frag[kDSteps][4];
  {
    const int r0 = warp_row + (lane >> 2), r1 = r0 + 8;
    const __nv_bfloat16* q0 = a.q + static_cast<size_t>(q_begin + row0 + min(r0, rows_here - 1)) * a.ldq +
                              static_cast<size_t>(head) * D + 2 * (lane & 3);
    const __nv_bfloat16* q1 = a.q + static_cast<size_t>(q_begin + row0 + min(r1, rows_here - 1)) * a.ldq +
                              static_cast<size_t>(head) * D + 2 * (lane & 3);
#pragma unroll
    for (int k = 0; k < kDSteps; ++k) {
      q_frag[k][0] = *reinterpret_cast<const uint32_t*>(q0 + k * 16);
      q_frag[k][1] = *reinterpret_cast<const uint32_t*>(q1 + k * 16);
      q_frag[k][2] = *reinterpret_cast<const uint32_t*>(q0 + k * 16 + 8);
      q_frag[k][3] = *reinterpret_cast<const uint32_t*>(q1 + k * 16 + 8);
    }
  }

  // where this lane's ldmatrix rows sit inside a tile half (the same for every tile)
  const int matrix = lane >> 3;
  const uint32_t piece_step = static_cast<uint32_t>(page_size) * 32;   // two 16-byte pieces on
  uint32_t k_offset[BLOCK_N / 16], v_offset[BLOCK_N / 16];
#pragma unroll
  for (int g = 0; g < BLOCK_N / 16; ++g) {
    // keys: matrices (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
    k_offset[g] = piece_offset(g * 16 + (matrix >> 1) * 8 + (lane & 7), matrix & 1, page_size,
                               page_bytes);
    // values, transposed: (keys 0-7, d lo), (keys 8-15, d lo), (keys 0-7, d hi), (keys 8-15, d hi)
    v_offset[g] = piece_offset(g * 16 + (matrix & 1) * 8 + (lane & 7), matrix >> 1, page_size,
                               page_bytes);
  }

  float o_acc[kOBlocks][4];
#pragma unroll
  for (int n = 0; n < kOBlocks; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[n][e] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0f, 0.0f};
  const int q_pos0 = context + row0 + warp_row + (lane >> 2);   // position of the first row
  const int q_pos1 = q_pos0 + 8;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile % RING;
    bool arrived = true;
    if (lane == 0) arrived = tile_wait(&full_bar[stage], static_cast<uint32_t>(tile / RING) & 1u);
    arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
    if (!arrived) {
      if (lane == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
      return;      // no block-wide barrier follows a failed wait in any warp: all warps fail alike
    }
    const uint32_t k_base = hx_shared_address(smem) + stage * 2 * kHalfBytes;
    const uint32_t v_base = k_base + kHalfBytes;

    // Behind the last key the tile holds whatever the pages (or an earlier tile) left there.
    // Scores of such keys are masked by selection, but a value of NaN would survive a zero
    // probability, so those value rows are cleared; likewise everything of an unreadable tile.
    const int first_stale = tile_state[stage] ? 0 : last_key + 1 - tile * BLOCK_N;
    if (first_stale < BLOCK_N) {
      for (int index = tid; index < BLOCK_N * (D / 8); index += THREADS) {
        const int key = index / (D / 8);
        const int piece = index - key * (D / 8);
        if (key >= first_stale) {
          const uint32_t address = v_base + piece_offset(key, piece, page_size, page_bytes);
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(address), "r"(0u) : "memory");
        }
      }
      __syncthreads();
    }

    // ---- S = Q K^T for 16 rows x 64 keys: 8 n-blocks of 8 keys
    float s[BLOCK_N / 8][4];
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.0f;
#pragma unroll
    for (int k = 0; k < kDSteps; ++k) {
#pragma unroll
      for (int pair = 0; pair < BLOCK_N / 16; ++pair) {
        uint32_t b[4];
        hx_ldmatrix_x4(b, k_base + k_offset[pair] + k * piece_step);
        hx_mma_bf16(s[pair * 2], q_frag[k], b[0], b[1]);
        hx_mma_bf16(s[pair * 2 + 1], q_frag[k], b[2], b[3]);
      }
    }

    // ---- scale, causal mask, running maximum
    const int key0 = tile * BLOCK_N + 2 * (lane & 3);
    const bool needs_mask = tile * BLOCK_N + BLOCK_N - 1 > context + row0 + warp_row;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float value = s[n][e] * a.scale;
        if (needs_mask) {
          const int key = key0 + n * 8 + (e & 1);
          const int q_pos = (e & 2) ? q_pos1 : q_pos0;
          if (key > q_pos) value = -INFINITY;
        }
        s[n][e] = value;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], value);
      }
    }
    float correction[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max[r]);
      // new_max is finite from the first tile on: key 0 is visible to every row
      correction[r] = row_max[r] == -INFINITY ? 0.0f : __expf(row_max[r] - new_max);
      row_max[r] = new_max;
      row_sum[r] *= correction[r];
    }
#pragma unroll
    for (int n = 0; n < kOBlocks; ++n) {
      o_acc[n][0] *= correction[0];
      o_acc[n][1] *= correction[0];
      o_acc[n][2] *= correction[1];
      o_acc[n][3] *= correction[1];
    }

    // ---- P = exp(S - max), O += P V with P = hi + lo in bfloat16
#pragma unroll
    for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
      float p[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float value = __expf(s[kk * 2 + half][e] - row_max[e >> 1]);
          p[half][e] = value;
          row_sum[e >> 1] += value;
        }
      uint32_t p_hi[4], p_lo[4];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int r = 0; r < 2; ++r)
          hx_split_bf16(p[half][r * 2], p[half][r * 2 + 1], p_hi[half * 2 + r], p_lo[half * 2 + r]);
#pragma unroll
      for (int nn = 0; nn < kOBlocks / 2; ++nn) {
        uint32_t b[4];      // V[keys kk*16 .. +15][d nn*16 .. +15], transposed
        hx_ldmatrix_x4_trans(b, v_base + v_offset[kk] + nn * piece_step);
        hx_mma_bf16(o_acc[nn * 2], p_hi, b[0], b[1]);
        hx_mma_bf16(o_acc[nn * 2], p_lo, b[0], b[1]);
        hx_mma_bf16(o_acc[nn * 2 + 1], p_hi, b[2], b[3]);
        hx_mma_bf16(o_acc[nn * 2 + 1], p_lo, b[2], b[3]);
      }
    }
    __syncthreads();      // every warp is done with this stage before it is refilled
    if (tid == 0 && tile + RING < n_tiles) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      request_tile(tile + RING);
    }
  }

  // ---- finish: full row sums, normalise, store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
  const float inverse[2] = {1.0f / row_sum[0], 1.0f / row_sum[1]};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp_row + (lane >> 2) + r * 8;
    if (row >= rows_here) continue;
    __nv_bfloat16* dst = a.out + static_cast<size_t>(q_begin + row0 + row) * a.ldo +
                         static_cast<size_t>(head) * D + 2 * (lane & 3);
#pragma unroll
    for (int n = 0; n < kOBlocks; ++n) {
      const __nv_bfloat162 value = __floats2bfloat162_rn(o_acc[n][r * 2] * inverse[r],
                                                         o_acc[n][r * 2 + 1] * inverse[r]);
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = value;
    }
  }
}

template <int D>
int launch(const PrefillArgs& a, int tiles, cudaStream_t stream) {
  constexpr int kSmem = RING * 2 * BLOCK_N * D * 2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attention_kernel<D>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
      cudaGetLastError();
      hx_set_error("hx_prefill_attention: cannot reserve %d bytes of shared memory", kSmem);
      return HX_ERR_LAUNCH;
    }
    configured = true;
  }
  const dim3 grid(tiles, a.heads);
  hx_launch(prefill_attention_kernel<D>, grid, THREADS, kSmem, stream, a);
  return HX_OK;
}

}  // namespace

// 1 when the tensor-core kernel takes this head size and page size (bfloat16 only).
HX_API int hx_prefill_attention_supports(int head_dim, int page_size) {
  return head_dim >= 16 && head_dim <= 256 && head_dim % (head_dim <= 128 ? 16 : 32) == 0 &&
         (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Attention of every request that brings at least `min_query_len` tokens to this step.
// `tile_bound` is an upper bound of the number of 64-row query tiles over those requests
// (tokens / 64 + requests is always enough).
HX_API int hx_prefill_attention(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* request_start, const int* request_context,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, void* out, int ldo, int requests, int tile_bound,
                                int heads, int kv_heads, int head_dim, int page_size,
                                int num_pages, float scale, int min_query_len, int* status,
                                cudaStream_t stream) {
  HX_REQUIRE(hx_prefill_attention_supports(head_dim, page_size),
             "hx_prefill_attention: head_dim %d with pages of %d is not supported (head sizes in "
             "steps of 16 up to 128 and of 32 up to 256, pages of 8, 16, 32 or 64)", head_dim, page_size);
  HX_REQUIRE(requests >= 0 && tile_bound >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
             "hx_prefill_attention: bad sizes");
  HX_REQUIRE(heads <= 65535, "hx_prefill_attention: too many heads");
  HX_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0,
             "hx_prefill_attention: bad cache geometry");
  HX_REQUIRE(ldq % 8 == 0 && ldo % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 3) == 0,
             "hx_prefill_attention: operands must be 16-byte aligned");
  if (requests == 0 || tile_bound == 0) return HX_OK;
  PrefillArgs a{static_cast<const __nv_bfloat16*>(q), ldq,
                static_cast<const __nv_bfloat16*>(k_cache),
                static_cast<const __nv_bfloat16*>(v_cache), request_start, request_context,
                request_table_row, block_tables, table_stride, static_cast<__nv_bfloat16*>(out),
                ldo, requests, heads, kv_heads, page_size, num_pages, scale, min_query_len, status};
  int rc = HX_ERR_UNSUPPORTED;
  switch (head_dim) {
    case 16: rc = launch<16>(a, tile_bound, stream); break;
    case 32: rc = launch<32>(a, tile_bound, stream); break;
    case 48: rc = launch<48>(a, tile_bound, stream); break;
    case 64: rc = launch<64>(a, tile_bound, stream); break;
    case 80: rc = launch<80>(a, tile_bound, stream); break;
    case 96: rc = launch<96>(a, tile_bound, stream); break;
    case 112: rc = launch<112>(a, tile_bound, stream); break;
    case 128: rc = launch<128>(a, tile_bound, stream); break;
    case 160: rc = launch<160>(a, tile_bound, stream); break;
    case 192: rc = launch<192>(a, tile_bound, stream); break;
    case 224: rc = launch<224>(a, tile_bound, stream); break;
    case 256: rc = launch<256>(a, tile_bound, stream); break;
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_prefill_attention");
  return HX_OK;
}
