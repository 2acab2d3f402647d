// Paged causal attention over block tables, float32 arithmetic, any batch shape.
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
// One chunk of 32 keys: lane j owns key j for the score (a whole key row per lane) and
// a slice of the head dimension for the weighted value sum (lane-per-dimension).  For the
// usual head sizes the loads of the key row AND of the 32 value slices are all issued
// before anything is computed, so a chunk costs one trip to memory.
//
// Key splits.  A long context is cut into splits of `split_keys` keys, one warp each.
// Every split writes its unnormalised sum, maximum and weight to scratch; the warp that
// finishes LAST for a (token, head) combines them in ascending order (a counter per
// (token, head) in scratch tells who is last, and is left at zero again).
//
// Exactness: dot products, the running maximum, exp, the running sum and the
// weighted value sum are float32.  The order of every sum is a function of the
// token's own position and of split_keys only (32-key chunks and splits anchored at
// lo, merged in ascending order), so a token's result does not depend on how the
// batch was cut, what else is in it, or which pages hold the keys.
#include "hx_common.cuh"

namespace {

constexpr int WARPS_PER_BLOCK = 4;
constexpr int MAX_HEAD_DIM = 256;

template <typename T, int VEC> struct VecLoad;
template <> struct VecLoad<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
};
template <> struct VecLoad<float, 2> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[2]) {
    const float2 r = *reinterpret_cast<const float2*>(p);
    v[0] = r.x; v[1] = r.y;
  }
};
template <> struct VecLoad<float, 8> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct VecLoad<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[2]) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    v[0] = f.x; v[1] = f.y;
  }
};
template <> struct VecLoad<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
};
template <> struct VecLoad<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.z));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.w));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
};

// A value slice kept as raw bits until it is used, so that 32 of them fit in registers.
template <typename T, int DPL> struct RawSlice;
template <> struct RawSlice<__nv_bfloat16, 2> { using type = uint32_t; };
template <> struct RawSlice<__nv_bfloat16, 4> { using type = uint2; };
template <> struct RawSlice<__nv_bfloat16, 8> { using type = uint4; };
template <> struct RawSlice<float, 2> { using type = float2; };
template <> struct RawSlice<float, 4> { using type = float4; };
template <> struct RawSlice<float, 8> { using type = float4; };   // never used with a known head size

template <typename T, int DPL>
__device__ __forceinline__ void unpack(const typename RawSlice<T, DPL>::type& raw, float (&v)[DPL]) {
  VecLoad<T, DPL>::load(reinterpret_cast<const T*>(&raw), v);
}

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
                              // tensor-core kernel
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

// Combine the splits of one (token, head) in ascending order; run by one warp.
template <typename T>
__device__ void merge_splits(const AttentionArgs& a, long long token_head, int token, int head,
                             int n_splits, int lane) {
  const int D = a.head_dim;
  const int stride = D + 2;
  const float* part = a.partial + static_cast<size_t>(token_head) * a.max_splits * stride;
  // maxima and weights of the splits, 32 at a time, read past the L1 (other SMs wrote them)
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
  T* out = static_cast<T*>(a.out) + static_cast<size_t>(token) * a.ldo +
           static_cast<size_t>(head) * D;
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

// What a warp does with its finished (token, head, split): write the output if it is the only
// split, else leave the partial result in scratch and, if it is the last to arrive, merge.
template <typename T, int DPL>
__device__ __forceinline__ void finish_item(const AttentionArgs& a, long long token_head, int token,
                                            int head, int split, int n_splits, int lane, int D,
                                            const float (&acc)[DPL], float running_max,
                                            float running_sum) {
  const int my_dim = lane * DPL;
  if (n_splits == 1) {
    if (my_dim < D) {
      const float inverse = 1.0f / running_sum;
      T* out = static_cast<T*>(a.out) + static_cast<size_t>(token) * a.ldo +
               static_cast<size_t>(head) * D + my_dim;
#pragma unroll
      for (int i = 0; i < DPL; ++i) out[i] = hx_from_float<T>(acc[i] * inverse);
    }
    return;
  }
  float* part = a.partial + (static_cast<size_t>(token_head) * a.max_splits + split) * (D + 2);
  if (my_dim < D) {
#pragma unroll
    for (int i = 0; i < DPL; ++i) part[my_dim + i] = acc[i];
  }
  if (lane == 0) {
    part[D] = running_max;
    part[D + 1] = running_sum;
  }
  // who finishes last for this (token, head) combines the splits
  __threadfence();
  __syncwarp();
  int arrived = 0;
  if (lane == 0) arrived = atomicAdd(a.arrivals + token_head, 1);
  arrived = __shfl_sync(0xffffffffu, arrived, 0);
  if (arrived != n_splits - 1) return;
  __threadfence();
  if (lane == 0) a.arrivals[token_head] = 0;     // ready for the next call
  merge_splits<T>(a, token_head, token, head, n_splits, lane);
}

// DPL: value coordinates per lane in the value phase (32 * DPL >= head_dim);
// VEC: elements per load in the key phase; HD: the head size when it is known at compile
// time (0: read it from the arguments).
template <typename T, int DPL, int VEC, int HD>
__global__ __launch_bounds__(WARPS_PER_BLOCK * 32, HD > 0 ? 3 : 1) void paged_attention_kernel(
    AttentionArgs a) {
  __shared__ float q_shared[WARPS_PER_BLOCK][MAX_HEAD_DIM];
  hx_pdl_prologue();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * WARPS_PER_BLOCK + warp;
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  if (item >= items) return;
  const int split = static_cast<int>(item % a.max_splits);
  const long long token_head = item / a.max_splits;
  const int head = static_cast<int>(token_head % a.heads);
  const int token = static_cast<int>(token_head / a.heads);
  if (skipped(a, token)) return;

  int lo, hi;
  key_range(a, token, lo, hi);
  const int n_splits = (hi - lo + a.split_keys - 1) / a.split_keys;
  if (split >= n_splits) return;
  const int begin = lo + split * a.split_keys;
  const int end = min(begin + a.split_keys, hi);

  const int D = HD > 0 ? HD : a.head_dim;
  const int kv_head = head / (a.heads / a.kv_heads);
  const T* q = static_cast<const T*>(a.q) + static_cast<size_t>(token) * a.ldq +
               static_cast<size_t>(head) * D;
  float* qs = q_shared[warp];
  for (int d = lane; d < D; d += 32) qs[d] = hx_to_float<T>(q[d]);
  __syncwarp();

  const int table_row = a.request_table_row[a.token_request[token]];
  const int* table = a.block_tables + static_cast<size_t>(table_row) * a.table_stride;
  const T* k_cache = static_cast<const T*>(a.k_cache);
  const T* v_cache = static_cast<const T*>(a.v_cache);

  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY;
  float running_sum = 0.0f;
  const int my_dim = lane * DPL;

  for (int chunk = begin; chunk < end; chunk += 32) {
    const int key = chunk + lane;
    bool valid = key < end;
    int row = -1;            // value row of this lane's key: [page][kv_head][slot]
    size_t key_offset = 0;   // element offset of chunk 0 of this lane's key (see hx_key_offset)
    if (valid) {
      const int page = table[key / a.page_size];
      if (page < 0 || page >= a.num_pages) {
        if (a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
        valid = false;
      } else {
        const int slot = key % a.page_size;
        row = (page * a.kv_heads + kv_head) * a.page_size + slot;
        key_offset = hx_key_offset(page, kv_head, slot, 0, a.kv_heads, a.page_size, D, VEC);
      }
    }
    const size_t chunk_stride = static_cast<size_t>(a.page_size) * VEC;
    const int keys_here = min(32, end - chunk);
    float score = -INFINITY;

    if (HD > 0) {
      // ---- known head size: every load of the chunk goes out before the arithmetic
      using Raw = typename RawSlice<T, DPL>::type;
      using RawKey = typename RawSlice<T, VEC>::type;
      constexpr int kLoads = HD > 0 ? HD / VEC : 1;
      RawKey key_raw[kLoads];
      if (valid) {
        const T* k = k_cache + key_offset;
#pragma unroll
        for (int u = 0; u < kLoads; ++u)
          key_raw[u] = *reinterpret_cast<const RawKey*>(k + u * chunk_stride);
      }
      // value slices of the first 16 keys go out with the key loads, the second 16 once the
      // scores are being reduced: two trips to memory per chunk, half the registers
      Raw values[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int v_row = __shfl_sync(0xffffffffu, row, j);   // -1: masked or unreadable
        if (v_row >= 0 && my_dim < D) {
          values[j] = *reinterpret_cast<const Raw*>(v_cache + static_cast<size_t>(v_row) * D + my_dim);
        } else {
          values[j] = Raw{};
        }
      }
      if (valid) {
        float dot = 0.0f;
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
          float kv[VEC];
          unpack<T, VEC>(key_raw[u], kv);
#pragma unroll
          for (int i = 0; i < VEC; ++i) dot = fmaf(qs[u * VEC + i], kv[i], dot);
        }
        score = dot * a.scale;
      }
      Raw more_values[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int v_row = __shfl_sync(0xffffffffu, row, 16 + j);
        if (v_row >= 0 && my_dim < D) {
          more_values[j] =
              *reinterpret_cast<const Raw*>(v_cache + static_cast<size_t>(v_row) * D + my_dim);
        } else {
          more_values[j] = Raw{};
        }
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
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float p = __shfl_sync(0xffffffffu, probability, j);
        float vv[DPL];
        if (j < 16) {
          unpack<T, DPL>(values[j], vv);
        } else {
          unpack<T, DPL>(more_values[j - 16], vv);
        }
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = fmaf(p, vv[i], acc[i]);
      }
    } else {
      // ---- any head size
      if (valid) {
        const T* k = k_cache + key_offset;
        float dot = 0.0f;
        for (int d = 0; d < D; d += VEC) {
          float kv[VEC];
          VecLoad<T, VEC>::load(k, kv);
          k += chunk_stride;
#pragma unroll
          for (int i = 0; i < VEC; ++i) dot = fmaf(qs[d + i], kv[i], dot);
        }
        score = dot * a.scale;
      }
      float chunk_max = score;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1)
        chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, offset));
      const float new_max = fmaxf(running_max, chunk_max);
      if (new_max == -INFINITY) continue;
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
      // values: eight keys at a time, their loads issued together; masked and unreadable
      // keys are skipped, so a stale page is never read
      for (int j0 = 0; j0 < keys_here; j0 += 8) {
        float p8[8];
        float vv[8][DPL];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          p8[u] = __shfl_sync(0xffffffffu, probability, j0 + u);
          const int v_row = __shfl_sync(0xffffffffu, row, j0 + u);
          if (v_row >= 0 && my_dim < D) {
            VecLoad<T, DPL>::load(v_cache + static_cast<size_t>(v_row) * D + my_dim, vv[u]);
          } else {
#pragma unroll
            for (int i = 0; i < DPL; ++i) vv[u][i] = 0.0f;
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[i] = fmaf(p8[u], vv[u][i], acc[i]);
      }
    }
  }

  finish_item<T, DPL>(a, token_head, token, head, split, n_splits, lane, D, acc, running_max,
                      running_sum);
}

// ------------------------------------------------------------------ streaming variant
//
// bfloat16, head sizes 64 and 128, pages of 8, 16 or 32 keys, no window.  The keys of a
// (page, head) are one contiguous block of the cache and so are its values, so a 32-key
// chunk is fetched with a few bulk copies (cp.async.bulk, completion counted on an
// mbarrier) into a ring of shared-memory slots that belongs to the warp.  The bytes in
// flight no longer live in registers: two warps per CTA keep 96 KB of the cache on its way
// to the SM, which is what it takes to stream the cache at memory speed.  Arithmetic, split
// handling and the order of every sum are those of the kernel above.
constexpr int STREAM_WARPS = 2;
constexpr uint32_t STREAM_WAIT_LIMIT = 20u * 1000u * 1000u;

__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t address = shared_address(bar);
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
      ::"r"(shared_address(dst)), "l"(src), "r"(bytes), "r"(shared_address(bar))
      : "memory");
}

template <int D>
struct StreamConfig {
  static constexpr int kChunkBytes = 32 * D * 2;     // keys (or values) of a 32-key chunk
  static constexpr int kSlotBytes = 2 * kChunkBytes;
  static constexpr int kRing = D == 128 ? 3 : 4;
  static constexpr int kSharedBytes = STREAM_WARPS * kRing * kSlotBytes;
};

template <int D>
__global__ __launch_bounds__(STREAM_WARPS * 32) void paged_attention_stream_kernel(
    AttentionArgs a) {
  using T = __nv_bfloat16;
  using Config = StreamConfig<D>;
  constexpr int DPL = D / 32;
  constexpr int RING = Config::kRing;
  constexpr int kKeyLoads = D / 8;
  extern __shared__ __align__(128) uint8_t stream_shared[];
  __shared__ uint64_t full_bar[STREAM_WARPS][RING];
  __shared__ float q_shared[STREAM_WARPS][D];
  hx_pdl_prologue();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * STREAM_WARPS + warp;
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  if (item >= items) return;
  const int split = static_cast<int>(item % a.max_splits);
  const long long token_head = item / a.max_splits;
  const int head = static_cast<int>(token_head % a.heads);
  const int token = static_cast<int>(token_head / a.heads);
  if (skipped(a, token)) return;

  int lo, hi;
  key_range(a, token, lo, hi);          // no window here: lo == 0
  const int n_splits = (hi - lo + a.split_keys - 1) / a.split_keys;
  if (split >= n_splits) return;
  const int begin = lo + split * a.split_keys;      // a multiple of 32, hence of the page size
  const int end = min(begin + a.split_keys, hi);
  const int n_chunks = (end - begin + 31) / 32;

  const int kv_head = head / (a.heads / a.kv_heads);
  const T* q = static_cast<const T*>(a.q) + static_cast<size_t>(token) * a.ldq +
               static_cast<size_t>(head) * D;
  float* qs = q_shared[warp];
  for (int d = lane; d < D; d += 32) qs[d] = __bfloat162float(q[d]);

  const int page_size = a.page_size;
  const int pages_per_chunk = 32 / page_size;
  const uint32_t page_bytes = static_cast<uint32_t>(page_size) * D * 2;
  const int table_row = a.request_table_row[a.token_request[token]];
  const int* table = a.block_tables + static_cast<size_t>(table_row) * a.table_stride;
  const int first_page = begin / page_size;
  const int n_pages = (end - begin + page_size - 1) / page_size;
  const uint8_t* k_cache = static_cast<const uint8_t*>(a.k_cache);
  const uint8_t* v_cache = static_cast<const uint8_t*>(a.v_cache);
  uint8_t* ring = stream_shared + static_cast<size_t>(warp) * RING * Config::kSlotBytes;
  uint64_t* bars = full_bar[warp];

  if (lane == 0) {
    for (int s = 0; s < RING; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(shared_address(&bars[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // the block table entries of up to 32 pages at a time, one per lane
  int window_first = 0;                 // index (within the split) of the page lane 0 holds
  int my_page = -1;
  auto load_pages = [&](int from) {
    window_first = from;
    const int index = from + lane;
    my_page = index < n_pages ? table[first_page + index] : -1;
    if (my_page >= a.num_pages) my_page = -1;
  };
  load_pages(0);

  // request the pages of chunk `c` into its ring slot (every lane runs this; lane 0 issues)
  auto request_chunk = [&](int c) {
    uint8_t* slot = ring + static_cast<size_t>(c % RING) * Config::kSlotBytes;
    uint64_t* bar = &bars[c % RING];
    int pages[4];
    uint32_t expected = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      pages[p] = -1;
      if (p < pages_per_chunk) {
        const int index = c * pages_per_chunk + p;
        if (index >= window_first + 32) load_pages(index);
        const int page = __shfl_sync(0xffffffffu, my_page, index - window_first);
        if (index < n_pages && page >= 0) {
          pages[p] = page;
          expected += 2 * page_bytes;
        }
      }
    }
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                       shared_address(bar)), "r"(expected) : "memory");
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        if (pages[p] >= 0) {
          const size_t block = (static_cast<size_t>(pages[p]) * a.kv_heads + kv_head) * page_bytes;
          bulk_copy(slot + p * page_bytes, k_cache + block, page_bytes, bar);
          bulk_copy(slot + Config::kChunkBytes + p * page_bytes, v_cache + block, page_bytes, bar);
        }
      }
    }
  };
  const int ahead = n_chunks < RING ? n_chunks : RING;
  for (int c = 0; c < ahead; ++c) request_chunk(c);

  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY;
  float running_sum = 0.0f;
  bool bad_page = false;

  for (int c = 0; c < n_chunks; ++c) {
    // is this lane's key there, and is its page readable?
    const int key = begin + c * 32 + lane;
    const int page_index = c * pages_per_chunk + lane / page_size;
    // the window of table entries may have moved on while requesting ahead: look it up again
    int page = -1;
    if (key < end) {
      page = table[first_page + page_index];
      if (page < 0 || page >= a.num_pages) {
        page = -1;
        bad_page = true;
      }
    }
    const bool valid = page >= 0;

    bool arrived = true;
    if (lane == 0) arrived = stream_wait(&bars[c % RING], static_cast<uint32_t>(c / RING) & 1u);
    arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
    if (!arrived) {
      if (lane == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
      return;
    }
    const uint8_t* slot = ring + static_cast<size_t>(c % RING) * Config::kSlotBytes;

    float score = -INFINITY;
    if (valid) {
      const uint8_t* k = slot + (lane / page_size) * page_bytes + (lane % page_size) * 16;
      float dot = 0.0f;
#pragma unroll
      for (int u = 0; u < kKeyLoads; ++u) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + static_cast<size_t>(u) * page_size * 16);
        float kv[8];
        VecLoad<T, 8>::load(reinterpret_cast<const T*>(&raw), kv);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(qs[u * 8 + i], kv[i], dot);
      }
      score = dot * a.scale;
    }
    float chunk_max = score;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, offset));
    const float new_max = fmaxf(running_max, chunk_max);
    if (new_max != -INFINITY) {
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
      const uint8_t* v = slot + Config::kChunkBytes + lane * DPL * 2;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) {
        const float p = __shfl_sync(0xffffffffu, probability, j);
        if (p != 0.0f) {      // masked and unreadable keys: their slots may hold anything
          float vv[DPL];
          VecLoad<T, DPL>::load(reinterpret_cast<const T*>(v + static_cast<size_t>(j) * D * 2), vv);
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[i] = fmaf(p, vv[i], acc[i]);
        }
      }
    }
    __syncwarp();
    if (c + RING < n_chunks) {
      // the slot is free: order this warp's reads before the copy engine's writes
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      request_chunk(c + RING);
    }
  }
  if (bad_page && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
  finish_item<T, DPL>(a, token_head, token, head, split, n_splits, lane, D, acc, running_max,
                      running_sum);
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

bool stream_variant_applies(const AttentionArgs& a, int dtype) {
  return dtype == HX_BF16 && (a.head_dim == 64 || a.head_dim == 128) && a.window == 0 &&
         (a.page_size == 8 || a.page_size == 16 || a.page_size == 32) && a.split_keys % 32 == 0;
}

template <typename T, int DPL, int VEC, int HD = 0>
void launch_main(const AttentionArgs& a, cudaStream_t stream) {
  const long long items = static_cast<long long>(a.tokens) * a.heads * a.max_splits;
  const int blocks = static_cast<int>((items + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK);
  hx_launch(paged_attention_kernel<T, DPL, VEC, HD>, blocks, WARPS_PER_BLOCK * 32, 0, stream, a);
}

template <typename T, int DPL>
int dispatch_vec(const AttentionArgs& a, cudaStream_t stream) {
  constexpr int kMaxVec = sizeof(T) == 2 ? 8 : 4;
  if (kMaxVec == 8 && a.head_dim % 8 == 0) {
    launch_main<T, DPL, 8>(a, stream);
  } else if (a.head_dim % 4 == 0) {
    launch_main<T, DPL, 4>(a, stream);
  } else {
    launch_main<T, DPL, 2>(a, stream);
  }
  return HX_OK;
}

template <typename T>
int dispatch(const AttentionArgs& a, cudaStream_t stream) {
  constexpr int kMaxVec = sizeof(T) == 2 ? 8 : 4;
  if constexpr (sizeof(T) == 2) {   // float32 rows of 128 would not fit in registers
    if (a.head_dim == 128) {
      launch_main<T, 4, kMaxVec, 128>(a, stream);
      return HX_OK;
    }
  }
  if (a.head_dim == 64) {
    launch_main<T, 2, kMaxVec, 64>(a, stream);
    return HX_OK;
  }
  if (a.head_dim <= 64 && a.head_dim % 2 == 0) return dispatch_vec<T, 2>(a, stream);
  if (a.head_dim <= 128 && a.head_dim % 4 == 0) return dispatch_vec<T, 4>(a, stream);
  if (a.head_dim <= 256 && a.head_dim % 8 == 0) return dispatch_vec<T, 8>(a, stream);
  hx_set_error("hx_paged_attention: head_dim %d is not supported (even up to 64, a multiple of "
               "4 up to 128, a multiple of 8 up to 256)", a.head_dim);
  return HX_ERR_UNSUPPORTED;
}

}  // namespace

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
  HX_REQUIRE(static_cast<long long>(num_pages) * kv_heads * page_size < (1ll << 31),
             "hx_paged_attention: cache rows exceed 32-bit indexing");
  if (tokens == 0) return HX_OK;
  AttentionArgs a{q, ldq, k_cache, v_cache, positions, token_request, request_table_row,
                  block_tables, table_stride, request_start, skip_query_len, out, ldo, partial,
                  arrivals, tokens, heads, kv_heads, head_dim, page_size, num_pages, window, scale,
                  split_keys, max_splits, status};
  const long long items = static_cast<long long>(tokens) * heads * max_splits;
  HX_REQUIRE(items / WARPS_PER_BLOCK < (1ll << 31) - 1, "hx_paged_attention: grid too large");
  int rc;
  if (stream_variant_applies(a, dtype)) {
    rc = a.head_dim == 128 ? launch_stream<128>(a, stream) : launch_stream<64>(a, stream);
  } else if (dtype == HX_F32) {
    rc = dispatch<float>(a, stream);
  } else if (dtype == HX_BF16) {
    rc = dispatch<__nv_bfloat16>(a, stream);
  } else {
    HX_REQUIRE(false, "hx_paged_attention: unknown dtype %d", dtype);
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_paged_attention");
  return HX_OK;
}
