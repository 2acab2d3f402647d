// Paged causal attention over block tables for decode tokens and short prompt portions.
//
// Every query token of the flattened batch attends to the keys of its own request at
// absolute positions [lo, position], lo = 0 or position - window + 1; this step's
// own keys are already in the pages (the rotary/append kernel ran first), so prompt
// portions and single decode tokens are the same case.  The reference computes the
// same thing in three stages through a materialised score tensor
// (src/attention/cuda_paged.cu:108-192: scores, softmax, values); here one warp
// walks the keys of one (token, head, key split) with an online softmax and never
// stores a score.
//
// Two kernels share the splitting and merging:
//
//  * the CUDA-core kernel takes every dtype, head size, page size and window: per chunk of
//    32 keys, lane j owns key j for the score and a slice of the head dimension for the
//    weighted value sum, all in float32;
//  * the streaming kernel (bfloat16, head sizes 64 and 128, pages of 8, 16 or 32 keys, no
//    window) is what decoding runs.  The keys of a (page, head) are one contiguous block of
//    the cache and so are its values, so a 32-key chunk is fetched with a few bulk copies
//    (cp.async.bulk counted on an mbarrier) into a ring of shared-memory slots that belongs
//    to the warp, and both products run on the tensor cores straight out of those slots: the
//    query is row 0 of a 16-row tile.  The bytes in flight live in shared memory, not in
//    registers, and the instruction count per byte is a sixth of the CUDA-core kernel's,
//    which is what it takes to stream the cache at memory speed.  Probabilities enter the
//    second product as two bfloat16 terms (hi + lo), so the softmax stays a float32
//    quantity as far as the result can tell.
//
// Key splits.  A long context is cut into splits of `split_keys` keys, one warp each.
// Every split writes its unnormalised sum, maximum and weight to scratch; the warp that
// finishes LAST for a (token, head) combines them in ascending order (a counter per
// (token, head) in scratch tells who is last, and is left at zero again).
//
// Exactness: the running maximum, exp, the running sum and the merge are float32; dot
// products are float32 sums of exact products.  The order of every sum is a function of the
// token's own position and of split_keys only (32-key chunks and splits anchored at lo,
// merged in ascending order), so a token's result does not depend on how the batch was cut,
// what else is in it, or which pages hold the keys.
#include "hx_mma.cuh"

namespace {

constexpr int WARPS_PER_BLOCK = 4;
constexpr int MAX_HEAD_DIM = 256;

struct AttentionArgs {
  const void* q;
  int ldq;
  const void* k_cache;
  const void* v_cache;
  const int* positions;
  const int* token_request;
  const int* request_table_row;
  const int* block_tables;
  int table_stride;
  const int* request_start;   // [requests + 1], needed only when skip_query_len > 0
  int skip_query_len;         // > 0: leave requests with at least this many tokens to the
                              // tensor-core prompt kernel
  void* out;
  int ldo;
  float* partial;   // [tokens * heads][max_splits][head_dim + 2], only when max_splits > 1
  int* arrivals;    // [tokens * heads] counters, zero on entry and on exit
  int tokens;
  int heads;
  int kv_heads;
  int head_dim;
  int page_size;
  int num_pages;
  int window;       // 0: every earlier key
  float scale;
  int split_keys;
  int max_splits;
  int* status;
};

__device__ __forceinline__ bool skipped(const AttentionArgs& a, int token) {
  if (a.skip_query_len <= 0) return false;
  const int request = a.token_request[token];
  return a.request_start[request + 1] - a.request_start[request] >= a.skip_query_len;
}

__device__ __forceinline__ void key_range(const AttentionArgs& a, int token, int& lo, int& hi) {
  const int position = a.positions[token];
  hi = position + 1;
  lo = a.window > 0 ? max(0, hi - a.window) : 0;
}

// Which (token, head, split) is this warp's, and which keys does it walk?  False: nothing to do.
struct Item {
  long long token_head;
  int token, head, split, n_splits, begin, end;
};

__device__ __forceinline__ bool find_item(const AttentionArgs& a, long long index, Item& item) {
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  if (index >= items) return false;
  item.split = static_cast<int>(index % a.max_splits);
  item.token_head = index / a.max_splits;
  item.head = static_cast<int>(item.token_head % a.heads);
  item.token = static_cast<int>(item.token_head / a.heads);
  if (skipped(a, item.token)) return false;
  int lo, hi;
  key_range(a, item.token, lo, hi);
  item.n_splits = (hi - lo + a.split_keys - 1) / a.split_keys;
  if (item.split >= item.n_splits) return false;
  item.begin = lo + item.split * a.split_keys;
  item.end = min(item.begin + a.split_keys, hi);
  return true;
}

// Combine the splits of one (token, head) in ascending order; run by one warp.
template <typename T>
__device__ void merge_splits(const AttentionArgs& a, const Item& item, int lane) {
  const int D = a.head_dim;
  const int stride = D + 2;
  const int n_splits = item.n_splits;
  const float* part = a.partial + static_cast<size_t>(item.token_head) * a.max_splits * stride;
  // maxima of the splits, 32 at a time, read past the L1 (other SMs wrote them)
  float total_max = -INFINITY;
  for (int base = 0; base < n_splits; base += 32) {
    const int s = base + lane;
    float m = s < n_splits ? __ldcg(part + static_cast<size_t>(s) * stride + D) : -INFINITY;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, offset));
    total_max = fmaxf(total_max, m);
  }
  // the total weight, split by split in ascending order
  float total_sum = 0.0f;
  for (int base = 0; base < n_splits; base += 32) {
    const int s = base + lane;
    float weighted = 0.0f;
    if (s < n_splits) {
      const float m = __ldcg(part + static_cast<size_t>(s) * stride + D);
      const float l = __ldcg(part + static_cast<size_t>(s) * stride + D + 1);
      weighted = m == -INFINITY ? 0.0f : l * expf(m - total_max);
    }
    const int here = min(32, n_splits - base);
    for (int j = 0; j < here; ++j) total_sum += __shfl_sync(0xffffffffu, weighted, j);
  }
  const float inverse = 1.0f / total_sum;
  T* out = static_cast<T*>(a.out) + static_cast<size_t>(item.token) * a.ldo +
           static_cast<size_t>(item.head) * D;
  for (int d = lane; d < D; d += 32) {
    float value = 0.0f;
    for (int base = 0; base < n_splits; base += 4) {
      float m[4], o[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = base + u;
        m[u] = s < n_splits ? __ldcg(part + static_cast<size_t>(s) * stride + D) : -INFINITY;
        o[u] = s < n_splits ? __ldcg(part + static_cast<size_t>(s) * stride + d) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        value = fmaf(o[u], m[u] == -INFINITY ? 0.0f : expf(m[u] - total_max), value);
    }
    out[d] = hx_from_float<T>(value * inverse);
  }
}

// What a warp does with its finished item.  The result arrives as `count` consecutive
// coordinates per lane starting at `first_dim` (lanes that hold nothing pass count 0).  With
// one split the output is written, else the partial result goes to scratch and the warp that
// arrives last merges.
template <typename T, int COUNT>
__device__ __forceinline__ void finish_item(const AttentionArgs& a, const Item& item, int lane,
                                            int first_dim, int count, const float (&acc)[COUNT],
                                            float running_max, float running_sum) {
  const int D = a.head_dim;
  if (item.n_splits == 1) {
    const float inverse = 1.0f / running_sum;
    T* out = static_cast<T*>(a.out) + static_cast<size_t>(item.token) * a.ldo +
             static_cast<size_t>(item.head) * D + first_dim;
#pragma unroll
    for (int i = 0; i < COUNT; ++i)
      if (i < count) out[i] = hx_from_float<T>(acc[i] * inverse);
    return;
  }
  float* part = a.partial +
                (static_cast<size_t>(item.token_head) * a.max_splits + item.split) * (D + 2);
#pragma unroll
  for (int i = 0; i < COUNT; ++i)
    if (i < count) part[first_dim + i] = acc[i];
  if (lane == 0) {
    part[D] = running_max;
    part[D + 1] = running_sum;
  }
  __threadfence();
  __syncwarp();
  int arrived = 0;
  if (lane == 0) arrived = atomicAdd(a.arrivals + item.token_head, 1);
  arrived = __shfl_sync(0xffffffffu, arrived, 0);
  if (arrived != item.n_splits - 1) return;
  __threadfence();
  if (lane == 0) a.arrivals[item.token_head] = 0;     // ready for the next call
  merge_splits<T>(a, item, lane);
}

// ------------------------------------------------------------------ CUDA-core kernel

// DPL: value coordinates per lane in the value phase (32 * DPL >= head_dim).  Cache elements
// are read two at a time, which every chunk size and every even head size allows.
template <typename T, int DPL>
__global__ __launch_bounds__(WARPS_PER_BLOCK * 32) void paged_attention_kernel(AttentionArgs a) {
  __shared__ float q_shared[WARPS_PER_BLOCK][MAX_HEAD_DIM];
  hx_pdl_prologue();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Item item;
  if (!find_item(a, static_cast<long long>(blockIdx.x) * WARPS_PER_BLOCK + warp, item)) return;

  const int D = a.head_dim;
  const int chunk_elems = hx_cache_chunk(sizeof(T), D);
  const int kv_head = item.head / (a.heads / a.kv_heads);
  const T* q = static_cast<const T*>(a.q) + static_cast<size_t>(item.token) * a.ldq +
               static_cast<size_t>(item.head) * D;
  float* qs = q_shared[warp];
  for (int d = lane; d < D; d += 32) qs[d] = hx_to_float<T>(q[d]);
  __syncwarp();

  const int table_row = a.request_table_row[a.token_request[item.token]];
  const int* table = a.block_tables + static_cast<size_t>(table_row) * a.table_stride;
  const T* k_cache = static_cast<const T*>(a.k_cache);
  const T* v_cache = static_cast<const T*>(a.v_cache);

  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY;
  float running_sum = 0.0f;
  const int my_dim = lane * DPL;

  for (int chunk = item.begin; chunk < item.end; chunk += 32) {
    const int key = chunk + lane;
    bool valid = key < item.end;
    int page = -1, slot = 0;
    if (valid) {
      page = table[key / a.page_size];
      slot = key % a.page_size;
      if (page < 0 || page >= a.num_pages) {
        if (a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
        valid = false;
        page = -1;
      }
    }
    float score = -INFINITY;
    if (valid) {
      float dot = 0.0f;
      for (int d = 0; d < D; d += 2) {
        const T* k = k_cache + hx_cache_offset(page, kv_head, slot, d, a.kv_heads, a.page_size, D,
                                               chunk_elems);
        dot = fmaf(qs[d], hx_to_float<T>(k[0]), dot);
        dot = fmaf(qs[d + 1], hx_to_float<T>(k[1]), dot);
      }
      score = dot * a.scale;
    }
    float chunk_max = score;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, offset));
    const float new_max = fmaxf(running_max, chunk_max);
    if (new_max == -INFINITY) continue;   // every key of the chunk unreadable
    const float correction = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
    const float probability = valid ? expf(score - new_max) : 0.0f;
    float chunk_sum = probability;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, offset);
    running_sum = running_sum * correction + chunk_sum;
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= correction;
    // values: masked and unreadable keys are skipped, so a stale page is never read
    const int keys_here = min(32, item.end - chunk);
    for (int j = 0; j < keys_here; ++j) {
      const float p = __shfl_sync(0xffffffffu, probability, j);
      const int v_page = __shfl_sync(0xffffffffu, page, j);
      const int v_slot = __shfl_sync(0xffffffffu, slot, j);
      if (v_page >= 0 && my_dim < D) {
#pragma unroll
        for (int i = 0; i < DPL; i += 2) {
          const T* v = v_cache + hx_cache_offset(v_page, kv_head, v_slot, my_dim + i, a.kv_heads,
                                                 a.page_size, D, chunk_elems);
          acc[i] = fmaf(p, hx_to_float<T>(v[0]), acc[i]);
          acc[i + 1] = fmaf(p, hx_to_float<T>(v[1]), acc[i + 1]);
        }
      }
    }
  }
  finish_item<T, DPL>(a, item, lane, my_dim, my_dim < D ? DPL : 0, acc, running_max,
                      running_sum);
}

// ------------------------------------------------------------------ streaming kernel

constexpr int STREAM_WARPS = 2;
constexpr uint32_t STREAM_WAIT_LIMIT = 20u * 1000u * 1000u;

__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t address = hx_shared_address(bar);
  for (uint32_t spin = 0; spin < STREAM_WAIT_LIMIT; ++spin) {
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

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(hx_shared_address(dst)), "l"(src), "r"(bytes), "r"(hx_shared_address(bar))
      : "memory");
}

template <int D>
struct StreamConfig {
  static constexpr int kChunkBytes = 32 * D * 2;     // keys (or values) of a 32-key chunk
  static constexpr int kSlotBytes = 2 * kChunkBytes;
  static constexpr int kRing = 2;     // 64 KB (32 KB) per CTA: three (six) CTAs share an SM
  static constexpr int kSharedBytes = STREAM_WARPS * kRing * kSlotBytes;
};

// Shared-memory address of the 16-byte piece (key `key` of the chunk, coordinates 8c..8c+7)
// inside a slot half that holds `32 / page_size` page blocks of [D/8][page_size][8].
__device__ __forceinline__ uint32_t piece_address(uint32_t half_base, int key, int c,
                                                  int page_size, uint32_t page_bytes) {
  return half_base + (key / page_size) * page_bytes + ((c * page_size + key % page_size) << 4);
}

template <int D>
__global__ __launch_bounds__(STREAM_WARPS * 32) void paged_attention_stream_kernel(
    AttentionArgs a) {
  using T = __nv_bfloat16;
  using Config = StreamConfig<D>;
  constexpr int RING = Config::kRing;
  constexpr int kDSteps = D / 16;     // k-steps of q k^T
  constexpr int kOBlocks = D / 8;     // 8-wide blocks of the output row
  extern __shared__ __align__(128) uint8_t stream_shared[];
  __shared__ uint64_t full_bar[STREAM_WARPS][RING];
  hx_pdl_prologue();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Item item;
  if (!find_item(a, static_cast<long long>(blockIdx.x) * STREAM_WARPS + warp, item)) return;
  const int begin = item.begin;       // no window: a multiple of 32, hence of the page size
  const int end = item.end;
  const int n_chunks = (end - begin + 31) / 32;

  const int kv_head = item.head / (a.heads / a.kv_heads);
  const int page_size = a.page_size;
  const int pages_per_chunk = 32 / page_size;
  const uint32_t page_bytes = static_cast<uint32_t>(page_size) * D * 2;
  const int table_row = a.request_table_row[a.token_request[item.token]];
  const int* table = a.block_tables + static_cast<size_t>(table_row) * a.table_stride;
  const int first_page = begin / page_size;
  const int n_pages = (end - begin + page_size - 1) / page_size;
  const uint8_t* k_cache = static_cast<const uint8_t*>(a.k_cache);
  const uint8_t* v_cache = static_cast<const uint8_t*>(a.v_cache);
  uint8_t* ring = stream_shared + static_cast<size_t>(warp) * RING * Config::kSlotBytes;
  uint64_t* bars = full_bar[warp];

  if (lane == 0) {
    for (int s = 0; s < RING; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(hx_shared_address(&bars[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // request the pages of chunk `c` into its ring slot; `bad` collects unreadable pages
  bool bad = false;
  auto request_chunk = [&](int c) {
    if (lane != 0) return;
    uint8_t* slot = ring + static_cast<size_t>(c % RING) * Config::kSlotBytes;
    uint64_t* bar = &bars[c % RING];
    int pages[4];
    uint32_t expected = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      pages[p] = -1;
      const int index = c * pages_per_chunk + p;
      if (p < pages_per_chunk && index < n_pages) {
        const int page = table[first_page + index];
        if (page >= 0 && page < a.num_pages) {
          pages[p] = page;
          expected += 2 * page_bytes;
        } else {
          bad = true;
        }
      }
    }
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                     hx_shared_address(bar)), "r"(expected) : "memory");
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      if (pages[p] >= 0) {
        const size_t block = (static_cast<size_t>(pages[p]) * a.kv_heads + kv_head) * page_bytes;
        bulk_copy(slot + p * page_bytes, k_cache + block, page_bytes, bar);
        bulk_copy(slot + Config::kChunkBytes + p * page_bytes, v_cache + block, page_bytes, bar);
      }
    }
  };
  const int ahead = n_chunks < RING ? n_chunks : RING;
  for (int c = 0; c < ahead; ++c) request_chunk(c);
  bad = __shfl_sync(0xffffffffu, bad ? 1 : 0, 0) != 0;      // lane 0 looked the pages up

  // the query is row 0 of a 16-row tile: only lanes 0..3 hold non-zero A fragments
  uint32_t q_frag[kDSteps][4];
  {
    const T* q = static_cast<const T*>(a.q) + static_cast<size_t>(item.token) * a.ldq +
                 static_cast<size_t>(item.head) * D;
#pragma unroll
    for (int k = 0; k < kDSteps; ++k) {
      q_frag[k][0] = q_frag[k][1] = q_frag[k][2] = q_frag[k][3] = 0u;
      if (lane < 4) {
        q_frag[k][0] = *reinterpret_cast<const uint32_t*>(q + k * 16 + 2 * lane);
        q_frag[k][2] = *reinterpret_cast<const uint32_t*>(q + k * 16 + 8 + 2 * lane);
      }
    }
  }

  // Where this lane's ldmatrix rows sit inside a slot half never changes from chunk to chunk:
  // work the offsets out once.  Keys: matrices (keys 0-7, d lo), (keys 0-7, d hi),
  // (keys 8-15, d lo), (keys 8-15, d hi) of each 16-key pair; values (transposed load):
  // (keys 0-7, d lo), (keys 8-15, d lo), (keys 0-7, d hi), (keys 8-15, d hi).
  const int matrix = lane >> 3;
  const uint32_t piece_step = static_cast<uint32_t>(page_size) * 32;   // two 16-byte pieces on
  uint32_t k_offset[2], v_offset[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int k_key = half * 16 + (matrix >> 1) * 8 + (lane & 7);
    k_offset[half] = piece_address(0, k_key, matrix & 1, page_size, page_bytes);
    const int v_key = half * 16 + (matrix & 1) * 8 + (lane & 7);
    v_offset[half] = piece_address(0, v_key, matrix >> 1, page_size, page_bytes);
  }

  // row 0 of the output lives in c0, c1 of lanes 0..3: coordinates 8 n + 2 lane + {0, 1}
  float o_acc[kOBlocks][4];
#pragma unroll
  for (int n = 0; n < kOBlocks; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[n][e] = 0.0f;
  float running_max = -INFINITY;
  float running_sum = 0.0f;      // this lane's share of the row sum (lanes 0..3)

  for (int c = 0; c < n_chunks; ++c) {
    bool arrived = true;
    if (lane == 0) arrived = stream_wait(&bars[c % RING], static_cast<uint32_t>(c / RING) & 1u);
    arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
    if (!arrived) {
      if (lane == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
      return;
    }
    const uint32_t k_half = hx_shared_address(ring + static_cast<size_t>(c % RING) * Config::kSlotBytes);
    const uint32_t v_half = k_half + Config::kChunkBytes;
    const int keys_here = min(32, end - (begin + c * 32));

    // Whatever lies behind the last key of the request in its last page, and pages that
    // could not be read, must not reach the second product (0 * NaN is NaN): clear those
    // value rows.  Keys need no clearing: their scores are masked by selection.
    if (keys_here < 32 || bad) {
      for (int index = lane; index < 32 * (D / 8); index += 32) {
        const int key = index / (D / 8);
        const int piece = index - key * (D / 8);
        bool clear = key >= keys_here;
        if (!clear && bad) {
          const int page = table[first_page + c * pages_per_chunk + key / page_size];
          clear = page < 0 || page >= a.num_pages;
        }
        if (clear) {
          const uint32_t address = piece_address(v_half, key, piece, page_size, page_bytes);
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(address), "r"(0u) : "memory");
        }
      }
      __syncwarp();
    }

    // ---- s = q k^T for the 32 keys: 4 blocks of 8 keys
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.0f;
#pragma unroll
    for (int k = 0; k < kDSteps; ++k) {
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        uint32_t b[4];
        hx_ldmatrix_x4(b, k_half + k_offset[pair] + k * piece_step);
        hx_mma_bf16(s[pair * 2], q_frag[k], b[0], b[1]);
        hx_mma_bf16(s[pair * 2 + 1], q_frag[k], b[2], b[3]);
      }
    }

    // ---- scale, mask, online softmax of row 0 (held by lanes 0..3 in c0, c1)
    float chunk_max = -INFINITY;
    if (keys_here == 32 && !bad) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[n][e] *= a.scale;
          chunk_max = fmaxf(chunk_max, s[n][e]);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = n * 8 + 2 * (lane & 3) + e;
          bool visible = key < keys_here;
          if (visible && bad) {
            const int page = table[first_page + c * pages_per_chunk + key / page_size];
            visible = page >= 0 && page < a.num_pages;
          }
          const float value = visible ? s[n][e] * a.scale : -INFINITY;
          s[n][e] = value;
          chunk_max = fmaxf(chunk_max, value);
        }
      }
    }
    chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 1));
    chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 2));
    chunk_max = __shfl_sync(0xffffffffu, chunk_max, 0);      // every lane follows row 0
    const float new_max = fmaxf(running_max, chunk_max);
    if (new_max != -INFINITY) {
      const float correction = running_max == -INFINITY ? 0.0f : __expf(running_max - new_max);
      running_max = new_max;
      running_sum *= correction;
#pragma unroll
      for (int n = 0; n < kOBlocks; ++n) {
        o_acc[n][0] *= correction;
        o_acc[n][1] *= correction;
      }
      // ---- o += p v with p = hi + lo; rows 1..15 of p are zero
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t p_hi[4] = {0u, 0u, 0u, 0u}, p_lo[4] = {0u, 0u, 0u, 0u};
        if (lane < 4) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const float x0 = __expf(s[kk * 2 + half][0] - new_max);
            const float x1 = __expf(s[kk * 2 + half][1] - new_max);
            running_sum += x0 + x1;
            hx_split_bf16(x0, x1, p_hi[half * 2], p_lo[half * 2]);
          }
        }
#pragma unroll
        for (int nn = 0; nn < kOBlocks / 2; ++nn) {
          uint32_t b[4];      // v[keys kk*16 .. +15][d nn*16 .. +15], transposed
          hx_ldmatrix_x4_trans(b, v_half + v_offset[kk] + nn * piece_step);
          hx_mma_bf16(o_acc[nn * 2], p_hi, b[0], b[1]);
          hx_mma_bf16(o_acc[nn * 2], p_lo, b[0], b[1]);
          hx_mma_bf16(o_acc[nn * 2 + 1], p_hi, b[2], b[3]);
          hx_mma_bf16(o_acc[nn * 2 + 1], p_lo, b[2], b[3]);
        }
      }
    }
    __syncwarp();
    if (c + RING < n_chunks) {
      // the slot is free: order this warp's reads before the copy engine's writes
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      request_chunk(c + RING);
      bad = __shfl_sync(0xffffffffu, bad ? 1 : 0, 0) != 0;
    }
  }
  if (lane == 0 && bad && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);

  // the row sum is spread over lanes 0..3; the output row over the same lanes, two
  // coordinates of every 8-wide block each: hand each lane's share to finish_item as
  // kOBlocks pieces of two coordinates
  running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 1);
  running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 2);
  running_sum = __shfl_sync(0xffffffffu, running_sum, 0);

  if (item.n_splits == 1) {
    if (lane < 4) {
      const float inverse = 1.0f / running_sum;
      T* out = static_cast<T*>(a.out) + static_cast<size_t>(item.token) * a.ldo +
               static_cast<size_t>(item.head) * D + 2 * lane;
#pragma unroll
      for (int n = 0; n < kOBlocks; ++n)
        *reinterpret_cast<__nv_bfloat162*>(out + n * 8) =
            __floats2bfloat162_rn(o_acc[n][0] * inverse, o_acc[n][1] * inverse);
    }
    return;
  }
  float* part = a.partial +
                (static_cast<size_t>(item.token_head) * a.max_splits + item.split) * (D + 2);
  if (lane < 4) {
#pragma unroll
    for (int n = 0; n < kOBlocks; ++n) {
      part[n * 8 + 2 * lane] = o_acc[n][0];
      part[n * 8 + 2 * lane + 1] = o_acc[n][1];
    }
  }
  if (lane == 0) {
    part[D] = running_max;
    part[D + 1] = running_sum;
  }
  __threadfence();
  __syncwarp();
  int arrived_count = 0;
  if (lane == 0) arrived_count = atomicAdd(a.arrivals + item.token_head, 1);
  arrived_count = __shfl_sync(0xffffffffu, arrived_count, 0);
  if (arrived_count != item.n_splits - 1) return;
  __threadfence();
  if (lane == 0) a.arrivals[item.token_head] = 0;
  merge_splits<T>(a, item, lane);
}

template <int D>
int launch_stream(const AttentionArgs& a, cudaStream_t stream) {
  using Config = StreamConfig<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(paged_attention_stream_kernel<D>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Config::kSharedBytes) != cudaSuccess) {
      cudaGetLastError();
      hx_set_error("hx_paged_attention: cannot reserve %d bytes of shared memory",
                   Config::kSharedBytes);
      return HX_ERR_LAUNCH;
    }
    configured = true;
  }
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  const int blocks = static_cast<int>((items + STREAM_WARPS - 1) / STREAM_WARPS);
  hx_launch(paged_attention_stream_kernel<D>, blocks, STREAM_WARPS * 32, Config::kSharedBytes,
            stream, a);
  return HX_OK;
}

bool stream_kernel_applies(const AttentionArgs& a, int dtype) {
  return dtype == HX_BF16 && (a.head_dim == 64 || a.head_dim == 128) && a.window == 0 &&
         (a.page_size == 8 || a.page_size == 16 || a.page_size == 32) && a.split_keys % 32 == 0;
}

template <typename T>
int launch_cuda_cores(const AttentionArgs& a, cudaStream_t stream) {
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  const int blocks = static_cast<int>((items + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK);
  if (a.head_dim % 2 != 0 || a.head_dim > MAX_HEAD_DIM) {
    hx_set_error("hx_paged_attention: head_dim %d is not supported (even, at most %d)",
                 a.head_dim, MAX_HEAD_DIM);
    return HX_ERR_UNSUPPORTED;
  }
  if (a.head_dim <= 64) {
    hx_launch(paged_attention_kernel<T, 2>, blocks, WARPS_PER_BLOCK * 32, 0, stream, a);
  } else if (a.head_dim <= 128 && a.head_dim % 4 == 0) {
    hx_launch(paged_attention_kernel<T, 4>, blocks, WARPS_PER_BLOCK * 32, 0, stream, a);
  } else if (a.head_dim % 8 == 0) {
    hx_launch(paged_attention_kernel<T, 8>, blocks, WARPS_PER_BLOCK * 32, 0, stream, a);
  } else {
    hx_set_error("hx_paged_attention: head_dim %d is not supported (above 64 a multiple of 4, "
                 "above 128 a multiple of 8)", a.head_dim);
    return HX_ERR_UNSUPPORTED;
  }
  return HX_OK;
}

}  // namespace

// Elements per chunk of the cache layout for this dtype and head size (see hx_cache_offset).
HX_API int hx_cache_chunk_elements(int dtype, int head_dim) {
  return hx_cache_chunk(dtype == HX_F32 ? 4 : 2, head_dim);
}

// Floats of scratch the call needs in `partial` (0 when max_splits == 1); the same call
// needs tokens * heads ints of zeroed scratch in `arrivals`.
HX_API long long hx_paged_attention_scratch_floats(int tokens, int heads, int head_dim,
                                                   int max_splits) {
  if (max_splits <= 1) return 0;
  return static_cast<long long>(tokens) * heads * max_splits * (head_dim + 2);
}

HX_API int hx_paged_attention(const void* q, int ldq, const void* k_cache, const void* v_cache,
                              int dtype, const int* positions, const int* token_request,
                              const int* request_table_row, const int* block_tables,
                              int table_stride, const int* request_start, int skip_query_len,
                              void* out, int ldo, float* partial, int* arrivals, int tokens,
                              int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                              int window, float scale, int split_keys, int max_splits, int* status,
                              cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
             "hx_paged_attention: heads %d must be a positive multiple of kv_heads %d", heads,
             kv_heads);
  HX_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0,
             "hx_paged_attention: bad cache geometry");
  HX_REQUIRE(split_keys > 0 && max_splits > 0, "hx_paged_attention: bad split sizes");
  HX_REQUIRE(max_splits == 1 || (partial != nullptr && arrivals != nullptr),
             "hx_paged_attention: scratch missing");
  HX_REQUIRE(window >= 0, "hx_paged_attention: window must not be negative");
  HX_REQUIRE(skip_query_len <= 0 || request_start != nullptr,
             "hx_paged_attention: request_start missing");
  HX_REQUIRE(ldq >= heads * head_dim && ldo >= heads * head_dim,
             "hx_paged_attention: row strides too small");
  HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, "hx_paged_attention: unknown dtype %d", dtype);
  if (tokens == 0) return HX_OK;
  AttentionArgs a{q, ldq, k_cache, v_cache, positions, token_request, request_table_row,
                  block_tables, table_stride, request_start, skip_query_len, out, ldo, partial,
                  arrivals, tokens, heads, kv_heads, head_dim, page_size, num_pages, window, scale,
                  split_keys, max_splits, status};
  const long long items = static_cast<long long>(tokens) * heads * max_splits;
  HX_REQUIRE(items / STREAM_WARPS < (1ll << 31) - 1, "hx_paged_attention: grid too large");
  int rc;
  if (stream_kernel_applies(a, dtype)) {
    rc = head_dim == 128 ? launch_stream<128>(a, stream) : launch_stream<64>(a, stream);
  } else if (dtype == HX_F32) {
    rc = launch_cuda_cores<float>(a, stream);
  } else {
    rc = launch_cuda_cores<__nv_bfloat16>(a, stream);
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_paged_attention");
  return HX_OK;
}

// ------------------------------------------------ the same attention, scratch built in
//
// hx_paged_attention() wants two pieces of scratch memory from its caller when a context is
// cut into key splits.  Not every caller can provide them.  A serving process that has
// handed all of its device memory to weights and the cache pool at start-up has nothing
// left to allocate from, and must not find that out in the middle of a request.  A caller on
// a latency-critical path cannot afford cudaMalloc or cudaFree there, because both make the
// whole device wait.  And a caller from plain C, or through a foreign-function interface,
// has no caching allocator to lean on and would have to size and keep such a buffer itself.
// For them the scratch lives in the library: one array in device memory, fixed at
// HX_NO_ALLOC_SCRATCH_WORDS 32-bit words (4.25 MiB), which every GPU that loads the library
// holds until the process ends.  See hx_no_alloc.h for the contract.
#include "hx_no_alloc.h"

#include <mutex>

static __device__ __align__(256) unsigned int hx_static_attention_scratch[HX_NO_ALLOC_SCRATCH_WORDS];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
void* g_static_scratch[kMaxDevices] = {};

// The array's name is only a host-side handle; the kernels need its address on the device
// that is current.  It is looked up once per device and remembered.
int static_scratch_of_current_device(void** address) {
  int device = -1;
  cudaError_t rc = cudaGetDevice(&device);
  if (rc != cudaSuccess) {
    hx_set_error("hx_paged_attention_no_alloc: cudaGetDevice failed: %s", cudaGetErrorString(rc));
    return HX_ERR_LAUNCH;
  }
  if (device < 0 || device >= kMaxDevices) {
    hx_set_error("hx_paged_attention_no_alloc: device %d is outside the supported range", device);
    return HX_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch[device] == nullptr) {
    void* found = nullptr;
    rc = cudaGetSymbolAddress(&found, hx_static_attention_scratch);
    if (rc != cudaSuccess || found == nullptr) {
      hx_set_error("hx_paged_attention_no_alloc: cudaGetSymbolAddress failed on device %d: %s",
                   device, cudaGetErrorString(rc));
      return HX_ERR_LAUNCH;
    }
    g_static_scratch[device] = found;
  }
  *address = g_static_scratch[device];
  return HX_OK;
}

}  // namespace

HX_API int hx_paged_attention_no_alloc(const void* q, int ldq, const void* k_cache,
                                       const void* v_cache, int dtype, const int* positions,
                                       const int* token_request, const int* request_table_row,
                                       const int* block_tables, int table_stride,
                                       const int* request_start, int skip_query_len, void* out,
                                       int ldo, int tokens, int heads, int kv_heads, int head_dim,
                                       int page_size, int num_pages, int window, float scale,
                                       int split_keys, int max_splits, int* status,
                                       cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0 && max_splits > 0,
             "hx_paged_attention_no_alloc: bad sizes");
  const long long floats = hx_paged_attention_scratch_floats(tokens, heads, head_dim, max_splits);
  const long long counters = max_splits > 1 ? static_cast<long long>(tokens) * heads : 0;
  HX_REQUIRE(floats <= HX_NO_ALLOC_PARTIAL_WORDS,
             "hx_paged_attention_no_alloc: %d tokens x %d heads x %d splits of head size %d need "
             "%lld words of scratch, the built-in array holds %d; use fewer splits or tokens, or "
             "call hx_paged_attention with scratch of your own", tokens, heads, max_splits,
             head_dim, floats, HX_NO_ALLOC_PARTIAL_WORDS);
  HX_REQUIRE(counters <= HX_NO_ALLOC_COUNTER_WORDS,
             "hx_paged_attention_no_alloc: %d tokens x %d heads need %lld arrival counters, the "
             "built-in array holds %d", tokens, heads, counters, HX_NO_ALLOC_COUNTER_WORDS);
  void* base = nullptr;
  const int found = static_scratch_of_current_device(&base);
  if (found != HX_OK) return found;
  float* partial = static_cast<float*>(base);
  int* arrivals = reinterpret_cast<int*>(static_cast<unsigned int*>(base) + HX_NO_ALLOC_PARTIAL_WORDS);
  if (counters > 0) {
    // The array keeps whatever the last call left.  Partial results are overwritten before
    // they are read; the arrival counters must start at zero, so they are cleared here, in
    // stream order, in case an earlier call was cut short.
    const cudaError_t rc = cudaMemsetAsync(arrivals, 0, static_cast<size_t>(counters) * sizeof(int),
                                           stream);
    if (rc != cudaSuccess) {
      hx_set_error("hx_paged_attention_no_alloc: clearing the counters failed: %s",
                   cudaGetErrorString(rc));
      return HX_ERR_LAUNCH;
    }
  }
  return hx_paged_attention(q, ldq, k_cache, v_cache, dtype, positions, token_request,
                            request_table_row, block_tables, table_stride, request_start,
                            skip_query_len, out, ldo, partial, arrivals, tokens, heads, kv_heads,
                            head_dim, page_size, num_pages, window, scale, split_keys, max_splits,
                            status, stream);
}
