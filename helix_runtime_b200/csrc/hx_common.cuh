// Shared declarations of the sm_100a kernel library.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the
// stream to launch on, allocates nothing and never synchronises; it returns 0 or
// a negative code and leaves a message for hx_last_error().  Sizes a kernel
// cannot run are refused here, on the host, before any launch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define HX_API extern "C" __attribute__((visibility("default")))

enum HxStatus : int {
  HX_OK = 0,
  HX_ERR_ARGUMENT = -1,     // a size or pointer the kernel refuses
  HX_ERR_LAUNCH = -2,       // cudaGetLastError after the launch
  HX_ERR_UNSUPPORTED = -3,  // valid model size, but no kernel instance for it
};

enum HxDType : int { HX_F32 = 0, HX_BF16 = 1 };

// device status word bits, written by kernels that can detect a bad input or a wait
// that ran out; the host reads the word after the step
enum HxDeviceFlag : int {
  HX_FLAG_BAD_TOKEN = 1,      // token id outside the vocabulary
  HX_FLAG_BAD_PAGE = 2,       // block table entry outside the pool
  HX_FLAG_WAIT_TIMEOUT = 4,   // a bounded mbarrier wait gave up
  HX_FLAG_NONFINITE = 8,      // sampling saw a non-finite logit
  HX_FLAG_BAD_POSITION = 16,  // a token's position lies outside the position table
};

void hx_set_error(const char* format, ...);
// Every entry point counts the kernels it launches (read with hx_launch_count()).
void hx_count_launches(int kernels);
// Streaming multiprocessors of the current device (0 and a message when it cannot be asked).
int hx_device_sm_count();

#define HX_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      hx_set_error(__VA_ARGS__);         \
      return HX_ERR_ARGUMENT;            \
    }                                    \
  } while (0)

#define HX_CHECK_LAUNCH(name)                                              \
  do {                                                                     \
    hx_count_launches(1);                                                  \
    cudaError_t hx_err__ = cudaGetLastError();                             \
    if (hx_err__ != cudaSuccess) {                                         \
      hx_set_error("%s: launch failed: %s", name, cudaGetErrorString(hx_err__)); \
      return HX_ERR_LAUNCH;                                                \
    }                                                                      \
  } while (0)

// ---------------------------------------------------------- programmatic dependent launch
//
// A step is a chain of a few hundred short kernels on one stream.  Every kernel is launched
// with programmatic stream serialization: it may be scheduled while its predecessor is still
// running, and calls hx_pdl_wait() before it touches anything a predecessor wrote.  What does
// not depend on the predecessor (the weight tiles of a matrix product) is fetched before the
// wait, so the memory system stays busy across kernel boundaries.  hx_pdl_trigger() lets the
// NEXT kernel be scheduled; the wait of that kernel still holds it until this one has
// completed and its writes are visible.
__device__ __forceinline__ void hx_pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void hx_pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void hx_pdl_prologue() {
  hx_pdl_trigger();
  hx_pdl_wait();
}

bool hx_pdl_enabled();

template <typename... KernelArgs, typename... Args>
inline void hx_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared_bytes,
                      cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = hx_pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

template <typename T> struct HxTraits;
template <> struct HxTraits<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct HxTraits<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float hx_to_float(T v);
template <> __device__ __forceinline__ float hx_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float hx_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T hx_from_float(float v);
template <> __device__ __forceinline__ float hx_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 hx_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Block-wide sum with a fixed reduction tree: the result for a row never depends on
// what else the grid is doing.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float hx_block_sum(float value, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
  __syncthreads();
  if (lane == 0) scratch[warp] = value;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < warps; ++w) total += scratch[w];
  return total;
}

__device__ __forceinline__ float hx_block_max(float value, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
  __syncthreads();
  if (lane == 0) scratch[warp] = value;
  __syncthreads();
  float total = scratch[0];
  for (int w = 1; w < warps; ++w) total = fmaxf(total, scratch[w]);
  return total;
}

// ---------------------------------------------------------------------- cache layout
//
// Keys and values of one layer are stored alike, in chunks of `chunk` elements (16 bytes
// where the head size allows): [page][kv_head][head_dim / chunk][slot][chunk].  All keys
// (or values) of a (page, head) are one contiguous block that a single bulk copy brings to
// shared memory; inside it the 16-byte pieces of consecutive slots are adjacent, which is
// the row order the tensor-core loads (ldmatrix) want and what lets a warp whose lanes each
// own one key read a coalesced stream.
__host__ __device__ __forceinline__ int hx_cache_chunk(int element_bytes, int head_dim) {
  const int widest = 16 / element_bytes;
  if (head_dim % widest == 0) return widest;
  if (widest > 4 && head_dim % 4 == 0) return 4;
  return 2;
}

// Element offset of coordinate `dim` of the key (or value) in (page, kv_head, slot).
__host__ __device__ __forceinline__ size_t hx_cache_offset(int page, int kv_head, int slot,
                                                           int dim, int kv_heads, int page_size,
                                                           int head_dim, int chunk) {
  const size_t page_head = static_cast<size_t>(page) * kv_heads + kv_head;
  return ((page_head * (head_dim / chunk) + dim / chunk) * page_size + slot) * chunk + dim % chunk;
}

// The requests that bring at least `min_len` tokens to a step are cut into tiles of `rows`
// tokens, and the tiles are numbered in the order of the requests.  Which request holds tile
// number `tile`, which of its tiles is it, and how many has it?  Every lane of a (whole,
// converged) warp calls this and gets the same answer; -1: there is no such tile.  Thirty-two
// requests are looked at per round: a step may bring a few prompt portions behind dozens of
// decode tokens, and every CTA of a prompt kernel asks this before anything else.
__device__ __forceinline__ int hx_find_query_tile(const int* request_start, int requests,
                                                  int min_len, int rows, int tile,
                                                  int& tile_in_request, int& tiles_of_request) {
  const int lane = threadIdx.x & 31;
  int before = 0;
  for (int base = 0; base < requests; base += 32) {
    const int r = base + lane;
    int tiles = 0;
    if (r < requests) {
      const int length = request_start[r + 1] - request_start[r];
      if (length >= min_len) tiles = (length + rows - 1) / rows;
    }
    int inclusive = tiles;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= offset) inclusive += other;
    }
    const unsigned beyond = __ballot_sync(0xffffffffu, before + inclusive > tile);
    if (beyond != 0u) {
      const int source = __ffs(beyond) - 1;
      tiles_of_request = __shfl_sync(0xffffffffu, tiles, source);
      tile_in_request =
          tile - (before + __shfl_sync(0xffffffffu, inclusive, source) - tiles_of_request);
      return base + source;
    }
    before += __shfl_sync(0xffffffffu, inclusive, 31);
  }
  return -1;
}

// silu(x) = x * sigmoid(x) with the branch-stable sigmoid of the reference
// (src/kernels/cuda/transformer.cu:68-83).
__device__ __forceinline__ float hx_silu(float x) {
  float sigmoid;
  if (x >= 0.0f) {
    sigmoid = 1.0f / (1.0f + expf(-x));
  } else {
    const float e = expf(x);
    sigmoid = e / (1.0f + e);
  }
  return x * sigmoid;
}

// The same with the hardware exponential (relative error about 2^-21): for results that are
// stored in bfloat16 right away.
__device__ __forceinline__ float hx_silu_fast(float x) {
  return x >= 0.0f ? __fdividef(x, 1.0f + __expf(-x)) : __fdividef(x * __expf(x), 1.0f + __expf(x));
}
