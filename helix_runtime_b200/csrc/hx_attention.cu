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
//  * the streaming kernel (bfloat16, head sizes in steps of 16 up to 128 and of 32 up to
//    256, pages of 8, 16 or 32 keys, no window) is what decoding runs.  The keys of a (page, head) are one contiguous block of
//    the cache and so are its values, so a 32-key chunk is fetched with a few bulk copies
//    (cp.async.bulk counted on an mbarrier) into a ring of shared-memory slots that belongs
//    to the warp, and both products run on the tensor cores straight out of those slots: the
//    query is row 0 of a 16-row tile.  The bytes in flight live in shared memory, not in
//    registers, and the instruction count per byte is a sixth of the CUDA-core kernel's,
//    which is what it takes to stream the cache at memory speed.  Probabilities enter the
//    second product as two bfloat16 terms (hi + lo), so the softmax stays a float32
//    quantity as far as the result can tell.
//
// Sharing a long context between warps.  The CUDA-core kernel cuts a context into splits of
// `split_keys` keys, one warp each.  The streaming kernel lays all 32-key chunks of all rows
// (token, head) end to end and gives every warp of a grid that fills the GPU once an equal
// run of that list, whatever the mix of context lengths; a run may end one row and begin
// another, and the copies of the chunks ahead stay in flight across that border.  Either
// way a warp that holds only part of a row writes its unnormalised sum, maximum and weight
// to scratch; the warp that finishes LAST for a (token, head) combines the parts in
// ascending order (a counter per (token, head) in scratch tells who is last, and is left at
// zero again).
//
// Exactness: the running maximum, exp, the running sum and the merge are float32; dot
// products are float32 sums of exact products.  Keys are always taken in 32-key chunks
// anchored at the first key and parts are merged in ascending order.  Where a row is cut
// into parts depends on split_keys (CUDA-core kernel) or on what else is in the batch
// (streaming kernel); that changes the grouping of float32 sums, hence the result by
// float32 rounding only, and nothing else about the batch, the cut of the prompt or the
// pages reaches a token's result.
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
  float* partial;   // scratch of hx_paged_attention_scratch_floats() floats
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
  // a caller whose split sizes do not cover the context (split_keys * max_splits keys) gets
  // fewer, longer splits: the last one walks on to the end of the context
  item.n_splits = min((hi - lo + a.split_keys - 1) / a.split_keys, a.max_splits);
  if (item.split >= item.n_splits) return false;
  item.begin = lo + item.split * a.split_keys;
  item.end = item.split == item.n_splits - 1 ? hi : item.begin + a.split_keys;
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

#ifndef HX_MERGE_LOADS
#define HX_MERGE_LOADS 8
#endif
constexpr int STREAM_WARPS = 2;
constexpr int STREAM_RING = 2;      // chunks in flight per warp
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

// KEYS: keys per chunk, the unit a warp fetches and works through at a time (16 or 32).
template <int D, int KEYS>
struct StreamConfig {
  static constexpr int kChunkBytes = KEYS * D * 2;     // keys (or values) of a chunk
  static constexpr int kSlotBytes = 2 * kChunkBytes;
  static constexpr int kRing = STREAM_RING;
  static constexpr int kSharedBytes = STREAM_WARPS * kRing * kSlotBytes;
  static constexpr int kPartStride = D + 4;            // floats; keeps parts 16-byte aligned
  // CTAs that share an SM as far as shared memory goes (the register budget follows it)
  static constexpr int kResident = (227 * 1024 / (kSharedBytes + 1024)) < 8
                                       ? (227 * 1024 / (kSharedBytes + 1024)) : 8;
};

// Shared-memory address of the 16-byte piece (key `key` of the chunk, coordinates 8c..8c+7)
// inside a slot half that holds `KEYS / page_size` page blocks of [D/8][page_size][8].
__device__ __forceinline__ uint32_t piece_address(uint32_t half_base, int key, int c,
                                                  int page_size, uint32_t page_bytes) {
  return half_base + (key / page_size) * page_bytes + ((c * page_size + key % page_size) << 4);
}

// Keys that `token` sees; 0 for tokens another kernel serves and past the end of the batch.
__device__ __forceinline__ int row_keys(const AttentionArgs& a, int token) {
  if (token >= a.tokens || skipped(a, token)) return 0;
  return a.positions[token] + 1;
}

// A place in the flat list of chunks: rows (token, head) in ascending order, the chunks of a
// row in ascending order of their keys.
struct ChunkCursor {
  int token, head, chunk;
  int n;                  // chunks in a row of this token
  int keys;               // keys this token sees
  int table_row;          // row of the block table that holds the token's pages
  long long row_begin;    // flat index of the row's first chunk
};

template <int KEYS>
__device__ __forceinline__ void cursor_next(const AttentionArgs& a, ChunkCursor& c) {
  if (++c.chunk < c.n) return;
  c.chunk = 0;
  c.row_begin += c.n;
  if (++c.head < a.heads) return;
  c.head = 0;
  do {
    ++c.token;
    c.keys = row_keys(a, c.token);
    c.n = (c.keys + KEYS - 1) / KEYS;
  } while (c.n == 0 && c.token < a.tokens);
  if (c.token < a.tokens) {
    c.table_row = a.request_table_row[a.token_request[c.token]];
  } else {
    c.n = 1;      // past the end: never used, but keeps the walk finite
  }
}

// Combine the parts of one row, written by the warps first_warp .. first_warp + n_parts - 1,
// in ascending order; run by one warp.  A warp keeps the part of the row that holds its first
// chunk in its slot 0, that of a row that begins inside its range in slot 1.  All loads of a
// batch of 32 parts are in flight together: the merge is a few round trips to the L2.
template <typename T, int D, int STRIDE>
__device__ void merge_parts(const AttentionArgs& a, int token, int head, long long row_begin,
                            long long per_warp, int first_warp, int n_parts, int lane) {
  // Coordinates per lane: four consecutive ones for a head of 128; otherwise pairs, the
  // i-th pair of a lane at coordinate 2 lane + 64 i (lanes beyond the head hold zeros).
  constexpr int MERGE_LOADS = HX_MERGE_LOADS;      // parts whose loads are in flight together
  constexpr bool QUADS = D == 128;
  constexpr int PER_LANE = QUADS ? 4 : 2 * ((D + 63) / 64);
  auto part_of = [&](int index) {
    const long long w = first_warp + index;
    const int slot = row_begin <= w * per_warp ? 0 : 1;
    return a.partial + static_cast<size_t>(w * 2 + slot) * STRIDE;
  };
  auto load_slice = [&](const float* part, float (&o)[PER_LANE]) {
    if constexpr (QUADS) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(part + 4 * lane));
      o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < PER_LANE; i += 2) {
        const int d = 2 * lane + 32 * i;
        float2 v = make_float2(0.0f, 0.0f);
        if (d < D) v = __ldcg(reinterpret_cast<const float2*>(part + d));
        o[i] = v.x; o[i + 1] = v.y;
      }
    }
  };
  float total_max = -INFINITY;
  float total_sum = 0.0f;
  float acc[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
  for (int base = 0; base < n_parts; base += 32) {
    const int here = min(32, n_parts - base);
    // lane s: maximum and weight of part base + s
    float m = -INFINITY, l = 0.0f;
    if (lane < here) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_of(base + lane) + D));
      m = ml.x;
      l = ml.y;
    }
    float batch_max = m;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      batch_max = fmaxf(batch_max, __shfl_xor_sync(0xffffffffu, batch_max, offset));
    const float new_max = fmaxf(total_max, batch_max);
    const float rescale = total_max == -INFINITY ? 0.0f : __expf(total_max - new_max);
    total_max = new_max;
    total_sum *= rescale;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] *= rescale;
    const float factor = m == -INFINITY ? 0.0f : __expf(m - new_max);
    for (int first = 0; first < here; first += MERGE_LOADS) {
      float o[MERGE_LOADS][PER_LANE];
#pragma unroll
      for (int u = 0; u < MERGE_LOADS; ++u)
        if (first + u < here) load_slice(part_of(base + first + u), o[u]);
#pragma unroll
      for (int u = 0; u < MERGE_LOADS; ++u) {
        if (first + u < here) {
          const float f = __shfl_sync(0xffffffffu, factor, first + u);
          total_sum = fmaf(__shfl_sync(0xffffffffu, l, first + u), f, total_sum);
#pragma unroll
          for (int i = 0; i < PER_LANE; ++i) acc[i] = fmaf(o[u][i], f, acc[i]);
        }
      }
    }
  }
  const float inverse = 1.0f / total_sum;
  T* out = static_cast<T*>(a.out) + static_cast<size_t>(token) * a.ldo +
           static_cast<size_t>(head) * D;
#pragma unroll
  for (int i = 0; i < PER_LANE; i += 2) {
    const int d = QUADS ? 4 * lane + i : 2 * lane + 32 * i;
    if (d < D)
      *reinterpret_cast<__nv_bfloat162*>(out + d) =
          __floats2bfloat162_rn(acc[i] * inverse, acc[i + 1] * inverse);
  }
}

// The flat list of chunks is cut into equal runs, one per warp of the grid, so a warp's run
// may end one row in the middle, cover some rows wholly and begin another: the copies of the
// next chunks are always in flight, across rows too, and every warp has the same amount of
// work whatever the mix of context lengths.  A row that is wholly inside a run is written
// straight to the output; a row cut by run borders is left as parts in scratch (at most two
// per warp) and the warp that finishes last combines them.
template <int D, int KEYS>
__global__ __launch_bounds__(STREAM_WARPS * 32, StreamConfig<D, KEYS>::kResident)
void paged_attention_stream_kernel(
    AttentionArgs a) {
  using T = __nv_bfloat16;
  using Config = StreamConfig<D, KEYS>;
  constexpr int RING = Config::kRing;
  constexpr int kDSteps = D / 16;       // k-steps of the scores
  constexpr int kDTiles = D / 16;       // 16-row tiles of the output
  constexpr int kTiles = KEYS / 16;     // 16-key tiles of a chunk
  constexpr int kMaxPages = KEYS / 8;   // pages of a chunk at the smallest page size
  extern __shared__ __align__(128) uint8_t stream_shared[];
  __shared__ uint64_t full_bar[STREAM_WARPS][RING];
  // The warp first finds its run of chunks from the step's description (positions, requests,
  // table rows: written before the step's first kernel), and only then waits for the kernel
  // before it, which wrote the queries and the newest keys and values.
  hx_pdl_trigger();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = static_cast<long long>(gridDim.x) * STREAM_WARPS;
  const long long me = static_cast<long long>(blockIdx.x) * STREAM_WARPS + warp;

  // ---- this warp's run of the flat chunk list.  Lane t looks at token base + t: its chunk
  // count and, at the same time, the row of the block table its pages are in.
  int first_keys = 0, first_table_row = 0, first_inclusive = 0;      // of the first 32 tokens
  long long total = 0;
  {
    first_keys = row_keys(a, lane);
    if (lane < a.tokens) first_table_row = a.request_table_row[a.token_request[lane]];
    first_inclusive = (first_keys + KEYS - 1) / KEYS;
    // the rest of the tokens (a step that mixes prompt portions with decode tokens brings
    // thousands): every lane adds up its own, with the loads of several rounds in flight
    int mine = first_inclusive;
#pragma unroll 4
    for (int token = 32 + lane; token < a.tokens; token += 32)
      mine += (row_keys(a, token) + KEYS - 1) / KEYS;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, first_inclusive, offset);
      if (lane >= offset) first_inclusive += other;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      mine += __shfl_xor_sync(0xffffffffu, mine, offset);
    total = mine;
  }
  total *= a.heads;
  const long long per_warp = (total + n_warps - 1) / n_warps;
  const long long my_begin = me * per_warp;
  const long long my_end = min(my_begin + per_warp, total);
  if (my_begin >= my_end) {
    hx_pdl_wait();      // a grid must not be seen complete before its predecessor is
    return;
  }

  // the row that holds chunk my_begin: among the first 32 tokens straight from the registers
  ChunkCursor at;
  {
    long long before = 0;      // chunks of one head of all earlier tokens
    int found = -1;
#pragma unroll 1
    for (int base = 0; base < a.tokens && found < 0; base += 32) {
      int keys = first_keys, inclusive = first_inclusive, table_row = first_table_row;
      if (base > 0) {
        keys = row_keys(a, base + lane);
        inclusive = (keys + KEYS - 1) / KEYS;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
          const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
          if (lane >= offset) inclusive += other;
        }
      }
      const unsigned beyond = __ballot_sync(0xffffffffu, (before + inclusive) * a.heads > my_begin);
      if (beyond != 0u) {
        const int source = __ffs(beyond) - 1;
        found = base + source;
        at.keys = __shfl_sync(0xffffffffu, keys, source);
        at.n = (at.keys + KEYS - 1) / KEYS;
        before += __shfl_sync(0xffffffffu, inclusive, source) - at.n;
        at.table_row = base == 0 ? __shfl_sync(0xffffffffu, table_row, source)
                                 : a.request_table_row[a.token_request[found]];
      } else {
        before += __shfl_sync(0xffffffffu, inclusive, 31);
      }
    }
    at.token = found;
    const long long inside = my_begin - before * a.heads;
    at.head = static_cast<int>(inside / at.n);
    at.chunk = static_cast<int>(inside - static_cast<long long>(at.head) * at.n);
    at.row_begin = my_begin - at.chunk;
  }
  ChunkCursor ahead = at;      // the chunk whose copies are requested next

  const int page_size = a.page_size;
  const int pages_per_chunk = KEYS / page_size;
  const uint32_t page_bytes = static_cast<uint32_t>(page_size) * D * 2;
  const int heads_per_kv = a.heads / a.kv_heads;
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

  // Page numbers come 32 at a time, one per lane, from the block table of the token the
  // requests have reached; a chunk's pages never straddle two such windows.
  int window_token = -1, window_base = 0, window_pages = -1;
  unsigned unreadable = 0u;      // per ring slot, one bit per page of the chunk in it
  bool any_unreadable = false;

  // request the copies of the chunk at `ahead` into ring slot `slot`; every lane follows,
  // lane 0 issues
  auto request_chunk = [&](int slot) {
    const int first = ahead.chunk * pages_per_chunk;
    if (ahead.token != window_token || first < window_base || first >= window_base + 32) {
      window_token = ahead.token;
      window_base = first & ~31;
      const int index = window_base + lane;
      window_pages = -1;
      if (index < a.table_stride && index * page_size < ahead.keys)
        window_pages = a.block_tables[static_cast<size_t>(ahead.table_row) * a.table_stride + index];
    }
    uint8_t* slot_base = ring + static_cast<size_t>(slot) * Config::kSlotBytes;
    uint64_t* bar = &bars[slot];
    const int kv_head = ahead.head / heads_per_kv;
    int pages[kMaxPages];
    uint32_t expected = 0;
    unsigned bits = 0u;
#pragma unroll
    for (int p = 0; p < kMaxPages; ++p) {
      pages[p] = -1;
      if (p < pages_per_chunk && (first + p) * page_size < ahead.keys) {
        const int page = __shfl_sync(0xffffffffu, window_pages, first + p - window_base);
        if (page >= 0 && page < a.num_pages) {
          pages[p] = page;
          expected += 2 * page_bytes;
        } else {
          bits |= 1u << p;
        }
      }
    }
    unreadable = (unreadable & ~(0xfu << (4 * slot))) | (bits << (4 * slot));
    any_unreadable = any_unreadable || bits != 0u;
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                       hx_shared_address(bar)), "r"(expected) : "memory");
#pragma unroll
      for (int p = 0; p < kMaxPages; ++p) {
        if (pages[p] >= 0) {
          const size_t block = (static_cast<size_t>(pages[p]) * a.kv_heads + kv_head) * page_bytes;
          bulk_copy(slot_base + p * page_bytes, k_cache + block, page_bytes, bar);
          bulk_copy(slot_base + Config::kChunkBytes + p * page_bytes, v_cache + block, page_bytes,
                    bar);
        }
      }
    }
  };
  const long long run = my_end - my_begin;
  // The kernel before this one writes the keys and values of THIS step's tokens and nothing
  // else of the cache.  A request brings at most a.tokens tokens, so of the keys a token
  // sees only the last a.tokens can be new: a chunk that ends before them holds what
  // earlier steps left, and its copies may start before the wait, while the predecessor
  // still runs.  (Let in early, a warp then finds its first chunks in shared memory when the
  // queries arrive.)
  // (A cursor never steps past the end of the run: behind the last row of a step that mixes
  // decode tokens with prompt portions lie thousands of tokens that are not this kernel's,
  // and walking over them costs a chain of loads each.)
  int requested = 0;
  for (; requested < RING && requested < run; ++requested) {
    if ((ahead.chunk + 1) * KEYS > ahead.keys - a.tokens) break;
    request_chunk(requested);
    if (requested + 1 < run) cursor_next<KEYS>(a, ahead);
  }
  hx_pdl_wait();
  for (; requested < RING && requested < run; ++requested) {
    request_chunk(requested);
    if (requested + 1 < run) cursor_next<KEYS>(a, ahead);
  }

  // Both products put the cache on the 16-row side of the tensor-core tile, where none of it
  // is wasted, and the single query (or probability) vector on the 8-column side:
  //   scores  S[16 keys x 8]  = K[16 keys x 16 d] q[16 d x 8]      (all 8 columns equal)
  //   output  O[16 d x 8]    += V^T[16 d x 16 keys] P[16 keys x 8]  (column 0: hi part of the
  //                                                    probabilities, column 1: lo part)
  // Where this lane's ldmatrix rows sit inside a slot half never changes from chunk to
  // chunk: work the offsets out once.  Keys (plain load): matrices (keys 0-7, d lo),
  // (keys 8-15, d lo), (keys 0-7, d hi), (keys 8-15, d hi) of a 16-key tile; values
  // (transposed load): (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi).
  const int matrix = lane >> 3;
  const int group = lane >> 2;       // row of the tile this lane holds in c0, c1 (and +8 in c2, c3)
  const int quad = lane & 3;
  const uint32_t piece_step = static_cast<uint32_t>(page_size) * 32;   // two 16-byte pieces on
  uint32_t k_offset[kTiles], v_offset[kTiles];
#pragma unroll
  for (int tile = 0; tile < kTiles; ++tile) {
    const int k_key = tile * 16 + (matrix & 1) * 8 + (lane & 7);
    k_offset[tile] = piece_address(0, k_key, matrix >> 1, page_size, page_bytes);
    const int v_key = tile * 16 + (matrix >> 1) * 8 + (lane & 7);
    v_offset[tile] = piece_address(0, v_key, matrix & 1, page_size, page_bytes);
  }

  uint32_t q_frag[kDSteps][2];       // the query as B operand: d 16k + 2 quad (+8), +1
  float o_acc[kDTiles][4];           // lanes with quad 0: d 16m + group (c0 hi, c1 lo), +8 (c2, c3)
  float running_max = -INFINITY;
  float running_sum = 0.0f;          // over this lane's own keys; lanes of a group hold copies
#pragma unroll
  for (int k = 0; k < kDSteps; ++k) q_frag[k][0] = q_frag[k][1] = 0u;

  for (long long i = 0; i < run; ++i) {
    const int slot = static_cast<int>(i % RING);
    if (i == 0 || at.chunk == 0) {
      // a row begins (or goes on from another warp's run): its query, an empty sum
      const T* q = static_cast<const T*>(a.q) + static_cast<size_t>(at.token) * a.ldq +
                   static_cast<size_t>(at.head) * D + 2 * quad;
#pragma unroll
      for (int k = 0; k < kDSteps; ++k) {
        q_frag[k][0] = *reinterpret_cast<const uint32_t*>(q + k * 16);
        q_frag[k][1] = *reinterpret_cast<const uint32_t*>(q + k * 16 + 8);
      }
#pragma unroll
      for (int m = 0; m < kDTiles; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) o_acc[m][e] = 0.0f;
      running_max = -INFINITY;
      running_sum = 0.0f;
    }

    bool arrived = true;
    if (lane == 0)
      arrived = stream_wait(&bars[slot], static_cast<uint32_t>(i / RING) & 1u);
    arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
    if (!arrived) {
      if (lane == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
      return;
    }
    const uint32_t k_half = hx_shared_address(ring + static_cast<size_t>(slot) * Config::kSlotBytes);
    const uint32_t v_half = k_half + Config::kChunkBytes;
    const int keys_here = min(KEYS, at.keys - at.chunk * KEYS);
    const unsigned bad_pages = (unreadable >> (4 * slot)) & 0xfu;

    // Whatever lies behind the last key of the request in its last page, and pages that
    // could not be read, must not reach the second product (0 * NaN is NaN): clear those
    // value rows.  Keys need no clearing: their scores are masked by selection.
    if (keys_here < KEYS || bad_pages != 0u) {
      for (int index = lane; index < KEYS * (D / 8); index += 32) {
        const int key = index / (D / 8);
        const int piece = index - key * (D / 8);
        if (key >= keys_here || ((bad_pages >> (key / page_size)) & 1u)) {
          const uint32_t address = piece_address(v_half, key, piece, page_size, page_bytes);
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(address), "r"(0u) : "memory");
        }
      }
      __syncwarp();
    }

    // ---- scores: this lane ends up with keys group and group + 8 of every tile, each twice
    // (c0 = c1, c2 = c3)
    float s[kTiles][4];
#pragma unroll
    for (int tile = 0; tile < kTiles; ++tile)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[tile][e] = 0.0f;
#pragma unroll
    for (int k = 0; k < kDSteps; ++k) {
#pragma unroll
      for (int tile = 0; tile < kTiles; ++tile) {
        uint32_t keys_a[4];
        hx_ldmatrix_x4(keys_a, k_half + k_offset[tile] + k * piece_step);
        hx_mma_bf16(s[tile], keys_a, q_frag[k][0], q_frag[k][1]);
      }
    }

    // ---- scale, mask, online softmax
    float score[2 * kTiles];      // keys group + 8 j
#pragma unroll
    for (int tile = 0; tile < kTiles; ++tile) {
      score[2 * tile] = s[tile][0];
      score[2 * tile + 1] = s[tile][2];
    }
    float chunk_max = -INFINITY;
    if (keys_here == KEYS && bad_pages == 0u) {
#pragma unroll
      for (int j = 0; j < 2 * kTiles; ++j) {
        score[j] *= a.scale;
        chunk_max = fmaxf(chunk_max, score[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 2 * kTiles; ++j) {
        const int key = group + 8 * j;
        const bool visible = key < keys_here && !((bad_pages >> (key / page_size)) & 1u);
        score[j] = visible ? score[j] * a.scale : -INFINITY;
        chunk_max = fmaxf(chunk_max, score[j]);
      }
    }
    chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 4));
    chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 8));
    chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 16));
    const float new_max = fmaxf(running_max, chunk_max);
    if (new_max != -INFINITY) {
      if (new_max != running_max) {      // the same in every lane
        const float correction = running_max == -INFINITY ? 0.0f : __expf(running_max - new_max);
        running_max = new_max;
        running_sum *= correction;
#pragma unroll
        for (int m = 0; m < kDTiles; ++m)
#pragma unroll
          for (int e = 0; e < 4; ++e) o_acc[m][e] *= correction;
      }
      // probabilities as (hi, lo) bfloat16 pairs, one 32-bit word per key
      uint32_t split[2 * kTiles];
#pragma unroll
      for (int j = 0; j < 2 * kTiles; ++j) {
        const float x = __expf(score[j] - new_max);
        running_sum += x;
        const __nv_bfloat16 hi = __float2bfloat16_rn(x);
        const __nv_bfloat16 lo = __float2bfloat16_rn(x - __bfloat162float(hi));
        split[j] = static_cast<uint32_t>(__bfloat16_as_ushort(hi)) |
                   (static_cast<uint32_t>(__bfloat16_as_ushort(lo)) << 16);
      }
      // ---- o += V^T p.  The B operand wants, in this lane, keys 2 quad, 2 quad + 1 (b0) and
      // 8 more (b1) of each tile: they sit in the lanes of groups 2 quad and 2 quad + 1.
      // Even columns (group even) take the hi parts, odd columns the lo parts; only columns
      // 0 and 1 are read back.
      const int source = 8 * quad;                         // first lane of group 2 quad
      const uint32_t pick = (group & 1) ? 0x7632u : 0x5410u;      // lo halves : hi halves
#pragma unroll
      for (int tile = 0; tile < kTiles; ++tile) {
        const uint32_t e0 = __shfl_sync(0xffffffffu, split[tile * 2], source);
        const uint32_t e1 = __shfl_sync(0xffffffffu, split[tile * 2], source + 4);
        const uint32_t f0 = __shfl_sync(0xffffffffu, split[tile * 2 + 1], source);
        const uint32_t f1 = __shfl_sync(0xffffffffu, split[tile * 2 + 1], source + 4);
        const uint32_t b0 = __byte_perm(e0, e1, pick);
        const uint32_t b1 = __byte_perm(f0, f1, pick);
#pragma unroll
        for (int m = 0; m < kDTiles; ++m) {
          uint32_t values_a[4];      // V^T[d 16m .. +15][keys of the tile]
          hx_ldmatrix_x4_trans(values_a, v_half + v_offset[tile] + m * piece_step);
          hx_mma_bf16(o_acc[m], values_a, b0, b1);
        }
      }
    }
    __syncwarp();
    if (i + RING < run) {
      // the slot is free: order this warp's reads before the copy engine's writes
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      request_chunk(slot);
      if (i + RING + 1 < run) cursor_next<KEYS>(a, ahead);
    }

    if (at.chunk == at.n - 1 || i == run - 1) {
      // ---- the row, or this run's share of it, is done.  Every group of lanes holds the
      // sum over its own keys; the output row sits in the lanes with quad 0.
      float row_sum = running_sum;
      row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 4);
      row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 8);
      row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 16);
      const long long row_end = at.row_begin + at.n;
      if (at.row_begin >= my_begin && row_end <= my_end) {
        if (quad == 0) {
          const float inverse = 1.0f / row_sum;
          T* out = static_cast<T*>(a.out) + static_cast<size_t>(at.token) * a.ldo +
                   static_cast<size_t>(at.head) * D + group;
#pragma unroll
          for (int m = 0; m < kDTiles; ++m) {
            out[m * 16] = __float2bfloat16_rn((o_acc[m][0] + o_acc[m][1]) * inverse);
            out[m * 16 + 8] = __float2bfloat16_rn((o_acc[m][2] + o_acc[m][3]) * inverse);
          }
        }
      } else {
        const int my_slot = at.row_begin <= my_begin ? 0 : 1;
        float* part = a.partial + static_cast<size_t>(me * 2 + my_slot) * Config::kPartStride;
        if (quad == 0) {
#pragma unroll
          for (int m = 0; m < kDTiles; ++m) {
            part[m * 16 + group] = o_acc[m][0] + o_acc[m][1];
            part[m * 16 + group + 8] = o_acc[m][2] + o_acc[m][3];
          }
        }
        if (lane == 0) *reinterpret_cast<float2*>(part + D) = make_float2(running_max, row_sum);
        __threadfence();
        __syncwarp();
        const int first_warp = static_cast<int>(at.row_begin / per_warp);
        const int n_parts = static_cast<int>((row_end - 1) / per_warp) - first_warp + 1;
        const long long counter = static_cast<long long>(at.token) * a.heads + at.head;
        int arrived_count = 0;
        if (lane == 0) arrived_count = atomicAdd(a.arrivals + counter, 1);
        arrived_count = __shfl_sync(0xffffffffu, arrived_count, 0);
        if (arrived_count == n_parts - 1) {
          __threadfence();
          if (lane == 0) a.arrivals[counter] = 0;      // ready for the next call
          merge_parts<T, D, Config::kPartStride>(a, at.token, at.head, at.row_begin, per_warp,
                                                 first_warp, n_parts, lane);
        }
      }
    }
    if (i + 1 < run) cursor_next<KEYS>(a, at);
  }
  if (lane == 0 && any_unreadable && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
}

// Warps the streaming kernel's grid may hold: the scratch keeps two parts per warp.
constexpr int STREAM_MAX_WARPS = 2048;

template <int D, int KEYS>
int launch_stream(const AttentionArgs& a, cudaStream_t stream) {
  using Config = StreamConfig<D, KEYS>;
  static int resident_warps[64] = {};      // per device: warps the whole GPU holds at once
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) device = 0;
  if (resident_warps[device] == 0) {
    int sms = 0, blocks_per_sm = 0;
    if (cudaFuncSetAttribute(paged_attention_stream_kernel<D, KEYS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Config::kSharedBytes) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &blocks_per_sm, paged_attention_stream_kernel<D, KEYS>, STREAM_WARPS * 32,
            Config::kSharedBytes) != cudaSuccess || sms <= 0 || blocks_per_sm <= 0) {
      cudaGetLastError();
      hx_set_error("hx_paged_attention: cannot reserve %d bytes of shared memory",
                   Config::kSharedBytes);
      return HX_ERR_LAUNCH;
    }
    resident_warps[device] = min(STREAM_MAX_WARPS, sms * blocks_per_sm * STREAM_WARPS);
  }
  // one warp per chunk at most (the bound on chunks comes from the caller's split sizes)
  const long long chunk_bound =
      static_cast<long long>(a.tokens) * a.heads *
      ((static_cast<long long>(a.split_keys) * a.max_splits + KEYS - 1) / KEYS);
  const long long warps = min(static_cast<long long>(resident_warps[device]), max(1ll, chunk_bound));
  const int blocks = static_cast<int>((warps + STREAM_WARPS - 1) / STREAM_WARPS);
  hx_launch(paged_attention_stream_kernel<D, KEYS>, blocks, STREAM_WARPS * 32,
            Config::kSharedBytes, stream, a);
  return HX_OK;
}

bool stream_kernel_applies(const AttentionArgs& a, int dtype) {
  return dtype == HX_BF16 && a.head_dim >= 16 && a.head_dim <= 256 &&
         a.head_dim % (a.head_dim <= 128 ? 16 : 32) == 0 && a.window == 0 &&
         (a.page_size == 8 || a.page_size == 16 || a.page_size == 32);
}

int launch_stream_for(const AttentionArgs& a, cudaStream_t stream) {
  // 32-key chunks: the largest page the kernel takes is one block of the cache
  switch (a.head_dim) {
    case 16: return launch_stream<16, 32>(a, stream);
    case 32: return launch_stream<32, 32>(a, stream);
    case 48: return launch_stream<48, 32>(a, stream);
    case 64: return launch_stream<64, 32>(a, stream);
    case 80: return launch_stream<80, 32>(a, stream);
    case 96: return launch_stream<96, 32>(a, stream);
    case 112: return launch_stream<112, 32>(a, stream);
    case 128: return launch_stream<128, 32>(a, stream);
    case 160: return launch_stream<160, 32>(a, stream);
    case 192: return launch_stream<192, 32>(a, stream);
    case 224: return launch_stream<224, 32>(a, stream);
    case 256: return launch_stream<256, 32>(a, stream);
  }
  hx_set_error("hx_paged_attention: no streaming kernel for head_dim %d", a.head_dim);
  return HX_ERR_UNSUPPORTED;
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

// Floats of scratch the call needs in `partial`: room for every key split of every row
// (the CUDA-core kernel) and for two parts per warp of the streaming kernel's grid.  The same
// call needs tokens * heads ints of zeroed scratch in `arrivals`.
HX_API long long hx_paged_attention_scratch_floats(int tokens, int heads, int head_dim,
                                                   int max_splits) {
  const long long by_split =
      max_splits <= 1 ? 0 : static_cast<long long>(tokens) * heads * max_splits * (head_dim + 2);
  const long long by_warp = 2ll * STREAM_MAX_WARPS * (head_dim + 4);
  return by_split > by_warp ? by_split : by_warp;
}

// The same for a caller that says which case it has: the streaming kernel (bfloat16, head
// sizes in steps of 16 up to 128 and of 32 up to 256, pages of 8 to 32 keys, no window) needs its two parts per warp only,
// whatever the number of tokens and splits.
HX_API long long hx_paged_attention_scratch_floats_for(int dtype, int tokens, int heads,
                                                       int head_dim, int page_size, int window,
                                                       int max_splits) {
  AttentionArgs a{};
  a.head_dim = head_dim;
  a.page_size = page_size;
  a.window = window;
  if (stream_kernel_applies(a, dtype)) return 2ll * STREAM_MAX_WARPS * (head_dim + 4);
  return hx_paged_attention_scratch_floats(tokens, heads, head_dim, max_splits);
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
  HX_REQUIRE(partial != nullptr && arrivals != nullptr, "hx_paged_attention: scratch missing");
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
    rc = launch_stream_for(a, stream);
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
// HX_NO_ALLOC_SCRATCH_WORDS 32-bit words (4.5 MiB), which every GPU that loads the library
// holds until the process ends.  See hx_no_alloc.h for the contract.
#include "hx_no_alloc.h"

#include <mutex>

static __device__ __align__(256) unsigned int hx_static_attention_scratch[HX_NO_ALLOC_SCRATCH_WORDS];
// the streaming kernel's area does not depend on the call: every head size it takes must fit
static_assert(HX_NO_ALLOC_PARTIAL_WORDS >= 2ll * STREAM_MAX_WARPS * (MAX_HEAD_DIM + 4),
              "the built-in scratch must hold the streaming kernel's parts at the largest head");

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
  // what the kernel that will run needs: two parts per resident warp for the streaming kernel,
  // a part per key split of every row for the CUDA-core kernel
  const long long floats = hx_paged_attention_scratch_floats_for(dtype, tokens, heads, head_dim,
                                                                 page_size, window, max_splits);
  const long long counters = static_cast<long long>(tokens) * heads;
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
