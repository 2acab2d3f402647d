// Embedding gather, RMSNorm, SwiGLU and the rotary-encoding + cache-append kernel.
//
// The residual stream is float32 in both precisions: the embedding widens into
// it, RMSNorm reads it and writes the compute dtype for the next matrix product.
#include "hx_common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstring>

// ------------------------------------------------------------------ error text

static thread_local char g_hx_error[512] = "";

void hx_set_error(const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_hx_error, sizeof(g_hx_error), format, args);
  va_end(args);
}

HX_API const char* hx_last_error() { return g_hx_error; }

static std::atomic<int> g_hx_pdl{1};

bool hx_pdl_enabled() { return g_hx_pdl.load(std::memory_order_relaxed) != 0; }

// 0 launches every kernel fully serialised (for debugging); 1, the default, lets a kernel be
// scheduled while its predecessor drains.
HX_API void hx_set_dependent_launch(int enabled) { g_hx_pdl.store(enabled ? 1 : 0); }

static std::atomic<long long> g_hx_launches{0};

void hx_count_launches(int kernels) { g_hx_launches.fetch_add(kernels, std::memory_order_relaxed); }

// Kernels launched by this library since it was loaded (a launch recorded into a CUDA graph
// counts once, when it is captured).
HX_API long long hx_launch_count() { return g_hx_launches.load(std::memory_order_relaxed); }

HX_API int hx_abi_version() { return 7; }

// Streaming multiprocessors of the current device (asked once per device); 0 with a message
// when the device cannot be asked.  Launch sizes that should fill the GPU come from here.
int hx_device_sm_count() {
  static std::atomic<int> counts[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    cudaGetLastError();
    hx_set_error("hx_sm_count: no current CUDA device");
    return 0;
  }
  int count = counts[device].load(std::memory_order_relaxed);
  if (count == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        count <= 0) {
      cudaGetLastError();
      hx_set_error("hx_sm_count: the device does not report its multiprocessor count");
      return 0;
    }
    counts[device].store(count, std::memory_order_relaxed);
  }
  return count;
}

HX_API int hx_sm_count() { return hx_device_sm_count(); }

// ------------------------------------------------------------------- embedding

// out[t, :] = table[id[t], :] widened to float32.  An id outside the vocabulary
// gives a NaN row and sets a status bit, never an out-of-bounds read
// (the reference's rule, src/kernels/cuda/embedding.cu:21-39).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab, int* status) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int id = ids[token];
  float* row_out = out + static_cast<size_t>(token) * hidden;
  if (id < 0 || id >= vocab) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) row_out[c] = __int_as_float(0x7fc00000);
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, HX_FLAG_BAD_TOKEN);
    return;
  }
  const T* row = table + static_cast<size_t>(id) * hidden;
  if constexpr (sizeof(T) == 2) {
    // rows of whole 16-byte pieces: eight values a load, all of a thread's loads in flight
    // together (one value at a time the row is a chain of sixteen cold loads)
    if (hidden % 8 == 0 && ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
      const uint4* pieces = reinterpret_cast<const uint4*>(row);
      float4* wide = reinterpret_cast<float4*>(row_out);
#pragma unroll 4
      for (int p = threadIdx.x; p < hidden / 8; p += blockDim.x) {
        const uint4 packed = pieces[p];
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&packed);
        const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]);
        const float2 c = __bfloat1622float2(pairs[2]), d = __bfloat1622float2(pairs[3]);
        wide[2 * p] = make_float4(a.x, a.y, b.x, b.y);
        wide[2 * p + 1] = make_float4(c.x, c.y, d.x, d.y);
      }
      return;
    }
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) row_out[c] = hx_to_float<T>(row[c]);
}

HX_API int hx_embed(const void* table, int dtype, const int* ids, float* out, int tokens,
                    int hidden, int vocab, int* status, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "hx_embed: bad sizes");
  if (tokens == 0) return HX_OK;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == HX_F32) {
    hx_launch(embed_kernel<float>, tokens, threads, 0, stream, static_cast<const float*>(table), ids, out, hidden, vocab, status);
  } else if (dtype == HX_BF16) {
    hx_launch(embed_kernel<__nv_bfloat16>, tokens, threads, 0, stream,  static_cast<const __nv_bfloat16*>(table), ids, out, hidden, vocab, status);
  } else {
    HX_REQUIRE(false, "hx_embed: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_embed");
  return HX_OK;
}

// --------------------------------------------------------------------- RMSNorm

// y = x * rsqrt(mean(x^2) + eps) * w, all in float32 (eps inside the root, added to
// the mean; src/kernels/cuda/transformer.cu:32-66).  One block per row; `rows`, when
// given, gathers the rows to normalise (the final norm runs on the wanted rows only).
template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                               TOut* __restrict__ y, const int* __restrict__ rows, int hidden,
                               float eps) {
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const int out_row = blockIdx.x;
  const int in_row = rows != nullptr ? rows[out_row] : out_row;
  const float* xr = x + static_cast<size_t>(in_row) * hidden;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = xr[c];
    sum = fmaf(v, v, sum);
  }
  const float total = hx_block_sum(sum, scratch);
  const float inverse = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
  TOut* yr = y + static_cast<size_t>(out_row) * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    yr[c] = hx_from_float<TOut>(xr[c] * inverse * weight[c]);
}

// The same for widths that are a multiple of four and fit in registers: each thread keeps up
// to RMS_VECTORS float4 of the row (four: widths to 4,096; eight: to 8,192), so the row is
// read once; the weight (which no earlier kernel writes) is fetched before the dependency
// wait.
template <typename TOut, int RMS_VECTORS>
__global__ __launch_bounds__(256) void rmsnorm_vector_kernel(
    const float* __restrict__ x, const float* __restrict__ weight, TOut* __restrict__ y,
    const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  hx_pdl_trigger();
  const int vectors = hidden >> 2;
  float4 w[RMS_VECTORS];
#pragma unroll
  for (int i = 0; i < RMS_VECTORS; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) w[i] = reinterpret_cast<const float4*>(weight)[v];
  }
  hx_pdl_wait();
  const int out_row = blockIdx.x;
  const int in_row = rows != nullptr ? rows[out_row] : out_row;
  const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(in_row) * hidden);
  float4 value[RMS_VECTORS];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < RMS_VECTORS; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) {
      value[i] = xr[v];
      sum = fmaf(value[i].x, value[i].x, sum);
      sum = fmaf(value[i].y, value[i].y, sum);
      sum = fmaf(value[i].z, value[i].z, sum);
      sum = fmaf(value[i].w, value[i].w, sum);
    }
  }
  const float total = hx_block_sum(sum, scratch);
  const float inverse = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
  TOut* yr = y + static_cast<size_t>(out_row) * hidden;
#pragma unroll
  for (int i = 0; i < RMS_VECTORS; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) {
      const float a = value[i].x * inverse * w[i].x;
      const float b = value[i].y * inverse * w[i].y;
      const float c = value[i].z * inverse * w[i].z;
      const float d = value[i].w * inverse * w[i].w;
      if (sizeof(TOut) == 4) {
        reinterpret_cast<float4*>(yr)[v] = make_float4(a, b, c, d);
      } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        reinterpret_cast<uint2*>(yr)[v] = packed;
      }
    }
  }
}

HX_API int hx_rmsnorm(const float* x, const float* weight, void* y, int out_dtype, const int* rows,
                      int n_rows, int hidden, float eps, cudaStream_t stream) {
  HX_REQUIRE(n_rows >= 0 && hidden > 0, "hx_rmsnorm: bad sizes");
  HX_REQUIRE(eps > 0.0f, "hx_rmsnorm: eps must be positive");
  if (n_rows == 0) return HX_OK;
  if (hidden % 4 == 0 && hidden <= 4 * 256 * 8 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
        reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    const bool four = hidden <= 4 * 256 * 4;
    if (out_dtype == HX_F32) {
      float* out = static_cast<float*>(y);
      if (four)
        hx_launch(rmsnorm_vector_kernel<float, 4>, n_rows, 256, 0, stream, x, weight, out, rows,
                  hidden, eps);
      else
        hx_launch(rmsnorm_vector_kernel<float, 8>, n_rows, 256, 0, stream, x, weight, out, rows,
                  hidden, eps);
    } else if (out_dtype == HX_BF16) {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(y);
      if (four)
        hx_launch(rmsnorm_vector_kernel<__nv_bfloat16, 4>, n_rows, 256, 0, stream, x, weight, out,
                  rows, hidden, eps);
      else
        hx_launch(rmsnorm_vector_kernel<__nv_bfloat16, 8>, n_rows, 256, 0, stream, x, weight, out,
                  rows, hidden, eps);
    } else {
      HX_REQUIRE(false, "hx_rmsnorm: unknown dtype %d", out_dtype);
    }
    HX_CHECK_LAUNCH("hx_rmsnorm");
    return HX_OK;
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == HX_F32) {
    hx_launch(rmsnorm_kernel<float>, n_rows, threads, 0, stream, x, weight, static_cast<float*>(y), rows, hidden, eps);
  } else if (out_dtype == HX_BF16) {
    hx_launch(rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream,  x, weight, static_cast<__nv_bfloat16*>(y), rows, hidden, eps);
  } else {
    HX_REQUIRE(false, "hx_rmsnorm: unknown dtype %d", out_dtype);
  }
  HX_CHECK_LAUNCH("hx_rmsnorm");
  return HX_OK;
}

// ---------------------------------------------------------------------- SwiGLU

// act[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]; gate and up arrive as float32
// accumulators, sigmoid and both products are float32, one rounding into the compute dtype
// (src/kernels/cuda/transformer.cu:68-83).  This is the path of the CUDA-core product;
// the tensor-core product applies the same formula in its epilogue.
template <typename TOut>
__global__ void swiglu_kernel(float* __restrict__ gate_up, TOut* __restrict__ act, int tokens,
                              int intermediate, int ld_in, int zero_input) {
  hx_pdl_prologue();
  const size_t total = static_cast<size_t>(tokens) * intermediate;
  for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < total;
       index += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = index / intermediate;
    const int i = static_cast<int>(index - t * intermediate);
    float* row = gate_up + t * ld_in;
    act[index] = hx_from_float<TOut>(hx_silu(row[i]) * row[intermediate + i]);
    if (zero_input) {      // the buffer is a split-K accumulator: leave it clear for its next use
      row[i] = 0.0f;
      row[intermediate + i] = 0.0f;
    }
  }
}

HX_API int hx_swiglu(float* gate_up, void* act, int out_dtype, int tokens, int intermediate,
                     int ld_in, int zero_input, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && intermediate > 0 && ld_in >= 2 * intermediate, "hx_swiglu: bad sizes");
  if (tokens == 0) return HX_OK;
  const size_t total = static_cast<size_t>(tokens) * intermediate;
  const int threads = 256;
  const size_t resident = static_cast<size_t>(hx_device_sm_count() > 0 ? hx_device_sm_count() : 1) * 16;
  const int blocks = static_cast<int>(total / threads + 1 < resident ? total / threads + 1 : resident);
  if (out_dtype == HX_F32) {
    hx_launch(swiglu_kernel<float>, blocks, threads, 0, stream, gate_up, static_cast<float*>(act), tokens, intermediate, ld_in, zero_input);
  } else if (out_dtype == HX_BF16) {
    hx_launch(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream,  gate_up, static_cast<__nv_bfloat16*>(act), tokens, intermediate, ld_in, zero_input);
  } else {
    HX_REQUIRE(false, "hx_swiglu: unknown dtype %d", out_dtype);
  }
  HX_CHECK_LAUNCH("hx_swiglu");
  return HX_OK;
}

// ---------------------------------------------- rotary encoding + cache append

// For token t of the flattened batch: rotate the first `rotary_dim` coordinates of
// every query and key head by the angles of its absolute position, leave values as
// they are, write the query back in place and write key (after rotation) and value
// into the token's slot of its request's page.  Rotation in float32 from a cos/sin
// table built on the host in double (src/model/llama_common.cpp:37-46;
// src/kernels/cuda/transformer.cu:100-119); the reference's separate cache append
// (src/kv_cache/cuda_paged.cpp:561-577) is fused in.
//
// qkv row: [q heads | k heads | v heads], each head `head_dim` wide.
// pairing 0: pairs (2p, 2p+1); pairing 1: pairs (p, p + rotary_dim/2).
// cache layer (keys and values alike): [page][kv_head][head_dim / chunk][slot][chunk],
// see hx_cache_offset.
constexpr int ROPE_HEADS_PER_BLOCK = 4;
// Up to this many tokens the kernel that follows (attention) may be scheduled while the
// rotary kernel still runs.
#ifndef HX_ROPE_RELEASE_TOKENS
#define HX_ROPE_RELEASE_TOKENS 16
#endif

template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                                   const int* __restrict__ token_request,
                                   const int* __restrict__ request_table_row,
                                   const int* __restrict__ block_tables, int table_stride,
                                   T* __restrict__ k_cache, T* __restrict__ v_cache, int write_cache,
                                   const float* __restrict__ cos_table,
                                   const float* __restrict__ sin_table, int table_positions,
                                   int heads, int kv_heads, int head_dim, int rotary_dim,
                                   int pairing, int page_size, int num_pages, int* status,
                                   float* __restrict__ accum, int ld_accum,
                                   int release_successor) {
  // The attention kernel that follows fills the GPU with one resident grid of warps that
  // all start on equal runs of work; let in early, they would all leave the wait in the same
  // instant and stay in step, fetching and computing in bursts (measured: twice the time at
  // batch 64).  So with many tokens it is launched when this kernel is done; with few
  // (release_successor) it may come in early and find its work while this kernel runs.
  if (release_successor) hx_pdl_trigger();
  hx_pdl_wait();
  const int token = blockIdx.x;
  const int position = positions[token];
  T* row = qkv + static_cast<size_t>(token) * ld;
  // When the projection was summed by split-K into a float32 accumulator, the values are
  // taken from there, rounded to the storage type exactly as the projection's own store
  // would have rounded them, and the accumulator is cleared for its next use.
  float* accum_row = accum != nullptr ? accum + static_cast<size_t>(token) * ld_accum : nullptr;
  const int half = rotary_dim / 2;
  // a position the table does not hold: flagged, and rotated with the nearest row so that
  // nothing outside the table is read
  const int table_position = min(max(position, 0), table_positions - 1);
  if (table_position != position && rotary_dim > 0 && threadIdx.x == 0 && status != nullptr)
    atomicOr(status, HX_FLAG_BAD_POSITION);
  const float* cos_row = cos_table + static_cast<size_t>(table_position) * half;
  const float* sin_row = sin_table + static_cast<size_t>(table_position) * half;

  int page = -1;
  int slot = 0;
  if (write_cache) {
    const int request = token_request[token];
    const int table_row = request_table_row[request];
    page = block_tables[static_cast<size_t>(table_row) * table_stride + position / page_size];
    slot = position % page_size;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && status != nullptr) atomicOr(status, HX_FLAG_BAD_PAGE);
      page = -1;
    }
  }

  // blockIdx.y selects a group of HEADS_PER_BLOCK consecutive heads of the row
  // [q heads | k heads | v heads]; one thread per coordinate pair of a q/k head, one per
  // coordinate of a v head.
  const int pairs_per_head = head_dim / 2;
  const int first_head = blockIdx.y * ROPE_HEADS_PER_BLOCK;
  const int total_heads = heads + 2 * kv_heads;
  const int last_head = min(first_head + ROPE_HEADS_PER_BLOCK, total_heads);
  for (int head = first_head; head < last_head; ++head) {
    T* vec = row + static_cast<size_t>(head) * head_dim;
    if (head < heads + kv_heads) {
      for (int pair = threadIdx.x; pair < pairs_per_head; pair += blockDim.x) {
        int i0, i1;
        bool rotate;
        if (pairing == 0) {
          i0 = 2 * pair;
          i1 = i0 + 1;
          rotate = i1 < rotary_dim;
        } else if (pair < half) {
          // half-split pairs inside the rotary part; the rest pass through two by two
          i0 = pair;
          i1 = pair + half;
          rotate = true;
        } else {
          i0 = rotary_dim + 2 * (pair - half);
          i1 = i0 + 1;
          rotate = false;
        }
        float a, b;
        if (accum_row != nullptr) {
          float* source = accum_row + static_cast<size_t>(head) * head_dim;
          a = hx_to_float<T>(hx_from_float<T>(source[i0]));
          b = hx_to_float<T>(hx_from_float<T>(source[i1]));
          source[i0] = 0.0f;
          source[i1] = 0.0f;
        } else {
          a = hx_to_float<T>(vec[i0]);
          b = hx_to_float<T>(vec[i1]);
        }
        if (rotate) {
          const float c = cos_row[pair];
          const float s = sin_row[pair];
          const float ra = a * c - b * s;
          const float rb = a * s + b * c;
          a = ra;
          b = rb;
        }
        const T ta = hx_from_float<T>(a);
        const T tb = hx_from_float<T>(b);
        if (head < heads) {
          vec[i0] = ta;
          vec[i1] = tb;
        } else if (page >= 0) {
          const int kv_head = head - heads;
          // 16-byte chunks, slot-major inside a chunk (see hx_cache_offset)
          const int chunk = hx_cache_chunk(sizeof(T), head_dim);
          k_cache[hx_cache_offset(page, kv_head, slot, i0, kv_heads, page_size, head_dim, chunk)] = ta;
          k_cache[hx_cache_offset(page, kv_head, slot, i1, kv_heads, page_size, head_dim, chunk)] = tb;
        }
      }
    } else {
      const int kv_head = head - heads - kv_heads;
      const int chunk = hx_cache_chunk(sizeof(T), head_dim);
      float* source = accum_row != nullptr ? accum_row + static_cast<size_t>(head) * head_dim
                                           : nullptr;
      for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        T value;
        if (source != nullptr) {
          value = hx_from_float<T>(source[d]);
          source[d] = 0.0f;
        } else {
          value = vec[d];
        }
        if (page >= 0)
          v_cache[hx_cache_offset(page, kv_head, slot, d, kv_heads, page_size, head_dim, chunk)] = value;
      }
    }
  }
}

// The same for bfloat16 rows whose heads are made of whole 16-byte pieces (8 coordinates):
// one thread per piece, every access 16 bytes wide (32 for the float32 accumulator), and a
// piece of a key or value is exactly one 16-byte chunk of the cache layout.  With half-split
// pairs the thread of a piece in the first half of the rotary part also takes the partner
// piece in the second half, whose own thread idles.
__global__ void rope_append_pieces_kernel(
    __nv_bfloat16* __restrict__ qkv, int ld, const int* __restrict__ positions,
    const int* __restrict__ token_request, const int* __restrict__ request_table_row,
    const int* __restrict__ block_tables, int table_stride, __nv_bfloat16* __restrict__ k_cache,
    __nv_bfloat16* __restrict__ v_cache, int write_cache, const float* __restrict__ cos_table,
    const float* __restrict__ sin_table, int table_positions, int heads, int kv_heads,
    int head_dim, int rotary_dim, int pairing, int page_size, int num_pages, int* status,
    float* __restrict__ accum, int ld_accum, int release_successor) {
  // with many tokens the attention kernel that follows is launched when this one is done
  // (see above)
  if (release_successor) hx_pdl_trigger();
  // Where the piece goes and by what it turns are the step's own description and the table
  // of angles, which no kernel of the step writes: all of that is looked up BEFORE the wait
  // for the product, while the product still runs.  What is left after the wait is one load
  // of the sums, the rotation and one store.
  const int token = blockIdx.x;
  const int pieces_per_head = head_dim / 8;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int head = item / pieces_per_head;
  const int piece = item - head * pieces_per_head;
  if (head >= heads + 2 * kv_heads) {
    hx_pdl_wait();      // a grid must not be seen complete before its predecessor is
    return;
  }

  const int position = positions[token];
  int page = -1, slot = 0;
  if (write_cache && head >= heads) {
    const int table_row = request_table_row[token_request[token]];
    page = block_tables[static_cast<size_t>(table_row) * table_stride + position / page_size];
    slot = position % page_size;
    if (page < 0 || page >= num_pages) {
      if (status != nullptr) atomicOr(status, HX_FLAG_BAD_PAGE);
      page = -1;
    }
  }

  // eight coordinates starting at d0, from the accumulator (rounded as the projection's own
  // store would have rounded them; the accumulator is cleared) or from the row
  auto load = [&](int d0, float (&x)[8]) {
    if (accum != nullptr) {
      float4* source = reinterpret_cast<float4*>(accum + static_cast<size_t>(token) * ld_accum +
                                                 static_cast<size_t>(head) * head_dim + d0);
      const float4 lo = source[0], hi = source[1];
      source[0] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      source[1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float raw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(raw[i]));
    } else {
      const uint4 packed = *reinterpret_cast<const uint4*>(
          qkv + static_cast<size_t>(token) * ld + static_cast<size_t>(head) * head_dim + d0);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(pairs[i]);
        x[2 * i] = v.x;
        x[2 * i + 1] = v.y;
      }
    }
  };
  auto store = [&](int d0, const float (&x)[8]) {
    uint4 packed;
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    if (head < heads) {
      *reinterpret_cast<uint4*>(qkv + static_cast<size_t>(token) * ld +
                                static_cast<size_t>(head) * head_dim + d0) = packed;
    } else if (page >= 0) {
      const bool is_key = head < heads + kv_heads;
      const int kv_head = is_key ? head - heads : head - heads - kv_heads;
      __nv_bfloat16* cache = is_key ? k_cache : v_cache;
      *reinterpret_cast<uint4*>(
          cache + hx_cache_offset(page, kv_head, slot, d0, kv_heads, page_size, head_dim, 8)) = packed;
    }
  };

  const int d0 = piece * 8;
  const int half = rotary_dim / 2;
  const bool rotates = head < heads + kv_heads && d0 < rotary_dim;
  if (!rotates) {
    // values, and coordinates behind the rotary part: moved as they are (a query piece that
    // came from the row is already where it belongs)
    hx_pdl_wait();
    if (accum == nullptr && head < heads) return;
    float x[8];
    load(d0, x);
    store(d0, x);
    return;
  }
  // a position the table does not hold: flagged, and rotated with the nearest row so that
  // nothing outside the table is read
  const int table_position = min(max(position, 0), table_positions - 1);
  if (table_position != position && status != nullptr) atomicOr(status, HX_FLAG_BAD_POSITION);
  const float* cos_row = cos_table + static_cast<size_t>(table_position) * half;
  const float* sin_row = sin_table + static_cast<size_t>(table_position) * half;
  if (pairing == 0) {
    // pairs (2p, 2p + 1): this piece holds pairs d0 / 2 .. d0 / 2 + 3
    float cs[4], ss[4];
    if (rotary_dim % 8 == 0) {
      // the table's rows are whole 16-byte runs of four angles
      const float4 c = *reinterpret_cast<const float4*>(cos_row + d0 / 2);
      const float4 sn = *reinterpret_cast<const float4*>(sin_row + d0 / 2);
      cs[0] = c.x; cs[1] = c.y; cs[2] = c.z; cs[3] = c.w;
      ss[0] = sn.x; ss[1] = sn.y; ss[2] = sn.z; ss[3] = sn.w;
    } else {
      // a rotary part that ends inside a piece (100 of 112 coordinates): the pairs behind
      // its end turn by nothing
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool turns = d0 + 2 * i < rotary_dim;
        cs[i] = turns ? cos_row[d0 / 2 + i] : 1.0f;
        ss[i] = turns ? sin_row[d0 / 2 + i] : 0.0f;
      }
    }
    hx_pdl_wait();
    float x[8];
    load(d0, x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = x[2 * i], b = x[2 * i + 1];
      x[2 * i] = a * cs[i] - b * ss[i];
      x[2 * i + 1] = a * ss[i] + b * cs[i];
    }
    store(d0, x);
  } else {
    // pairs (p, p + half): the thread of the first-half piece rotates both pieces
    if (d0 >= half) {
      hx_pdl_wait();
      return;
    }
    const float4 c0 = *reinterpret_cast<const float4*>(cos_row + d0);
    const float4 c1 = *reinterpret_cast<const float4*>(cos_row + d0 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sin_row + d0);
    const float4 s1 = *reinterpret_cast<const float4*>(sin_row + d0 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    hx_pdl_wait();
    float x[8], y[8];
    load(d0, x);
    load(d0 + half, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = x[i], b = y[i];
      x[i] = a * cs[i] - b * ss[i];
      y[i] = a * ss[i] + b * cs[i];
    }
    store(d0, x);
    store(d0 + half, y);
  }
}

HX_API int hx_rope_append(void* qkv, int dtype, int ld, const int* positions,
                          const int* token_request, const int* request_table_row,
                          const int* block_tables, int table_stride, void* k_cache, void* v_cache,
                          int write_cache, const float* cos_table, const float* sin_table,
                          int table_positions, int tokens, int heads, int kv_heads, int head_dim,
                          int rotary_dim, int pairing, int page_size, int num_pages, int* status,
                          float* accum, int ld_accum, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0, "hx_rope_append: bad sizes");
  HX_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "hx_rope_append: head_dim %d must be even", head_dim);
  HX_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
             "hx_rope_append: rotary_dim %d must be even and at most head_dim %d", rotary_dim,
             head_dim);
  HX_REQUIRE(pairing == 0 || pairing == 1, "hx_rope_append: unknown pairing %d", pairing);
  HX_REQUIRE(ld >= (heads + 2 * kv_heads) * head_dim, "hx_rope_append: row stride too small");
  HX_REQUIRE(!write_cache || (page_size > 0 && num_pages > 0 && k_cache && v_cache),
             "hx_rope_append: cache arguments missing");
  HX_REQUIRE(rotary_dim == 0 || table_positions > 0, "hx_rope_append: empty rotary table");
  HX_REQUIRE(accum == nullptr || ld_accum >= (heads + 2 * kv_heads) * head_dim,
             "hx_rope_append: accumulator stride too small");
  if (tokens == 0) return HX_OK;
  const int release_successor = tokens <= HX_ROPE_RELEASE_TOKENS ? 1 : 0;
  const int threads = head_dim / 2 >= 64 ? 64 : 32;
  const dim3 grid(tokens, (heads + 2 * kv_heads + ROPE_HEADS_PER_BLOCK - 1) / ROPE_HEADS_PER_BLOCK);
  HX_REQUIRE(grid.y <= 65535, "hx_rope_append: too many heads");
  const int half = rotary_dim / 2;
  const bool whole_pieces =
      dtype == HX_BF16 && head_dim % 8 == 0 && ld % 8 == 0 && (accum == nullptr || ld_accum % 4 == 0) &&
      (pairing == 0 || half % 8 == 0);
  if (whole_pieces) {
    const int items = (heads + 2 * kv_heads) * (head_dim / 8);
    const int block = items >= 256 ? 256 : ((items + 31) / 32) * 32;
    const dim3 piece_grid(tokens, (items + block - 1) / block);
    HX_REQUIRE(piece_grid.y <= 65535, "hx_rope_append: too many heads");
    hx_launch(rope_append_pieces_kernel, piece_grid, block, 0, stream,
              static_cast<__nv_bfloat16*>(qkv), ld, positions, token_request, request_table_row,
              block_tables, table_stride, static_cast<__nv_bfloat16*>(k_cache),
              static_cast<__nv_bfloat16*>(v_cache), write_cache, cos_table, sin_table,
              table_positions, heads, kv_heads, head_dim, rotary_dim, pairing, page_size, num_pages,
              status, accum, ld_accum, release_successor);
  } else if (dtype == HX_F32) {
    hx_launch(rope_append_kernel<float>, grid, threads, 0, stream,  static_cast<float*>(qkv), ld, positions, token_request, request_table_row, block_tables, table_stride, static_cast<float*>(k_cache), static_cast<float*>(v_cache), write_cache, cos_table, sin_table, table_positions, heads, kv_heads, head_dim, rotary_dim, pairing, page_size, num_pages, status, accum, ld_accum, release_successor);
  } else if (dtype == HX_BF16) {
    hx_launch(rope_append_kernel<__nv_bfloat16>, grid, threads, 0, stream,  static_cast<__nv_bfloat16*>(qkv), ld, positions, token_request, request_table_row, block_tables, table_stride, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), write_cache, cos_table, sin_table, table_positions, heads, kv_heads, head_dim, rotary_dim, pairing, page_size, num_pages, status, accum, ld_accum, release_successor);
  } else {
    HX_REQUIRE(false, "hx_rope_append: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_rope_append");
  return HX_OK;
}

// ------------------------------------------------- tokens of a step queued ahead

// A step that was prepared before the host knew what the step before it sampled takes its
// tokens from that step's output on the device: token_ids[i] = sampled[rows[i]].  A row whose
// logits were not finite (-1) feeds token 0: its request has failed and the host drops the row.
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                   const int* __restrict__ rows, int count, int sampled_rows) {
  hx_pdl_prologue();
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index < count) {
    const int row = rows[index];
    const int token = row >= 0 && row < sampled_rows ? sampled[row] : 0;
    token_ids[index] = token < 0 ? 0 : token;
  }
}

HX_API int hx_feed_tokens(int* token_ids, const int* sampled, const int* rows, int count,
                          int sampled_rows, cudaStream_t stream) {
  HX_REQUIRE(count >= 0 && sampled_rows >= 0, "hx_feed_tokens: bad count");
  if (count == 0) return HX_OK;
  hx_launch(feed_tokens_kernel, (count + 127) / 128, 128, 0, stream, token_ids, sampled, rows,
            count, sampled_rows);
  HX_CHECK_LAUNCH("hx_feed_tokens");
  return HX_OK;
}
