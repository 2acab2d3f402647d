// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   out[t, f] (+)= sum_k x[t, k] * w[f, k]        x: [tokens, K]   w: [features, K]
//
// Both operands are K-major, which is how the checkpoint stores its matrices, so no
// transposed copy is ever made (the reference keeps [in, out] and multiplies with a
// 16x16 shared-memory kernel, src/kernels/cuda/matmul.cu:36-71).
//
// Mapping.  The WEIGHT tile is the MMA's M operand (128 features per CTA) and the
// TOKEN tile its N operand (BN = 16 ... 256 tokens), so one kernel covers decoding
// (a handful of tokens, pure weight streaming) and prompt portions (256-token
// tiles).  The accumulator lives in tensor memory as [128 feature lanes x BN token
// columns] float32.  Warp roles:
//   warp 0      one lane issues the TMA loads of both operand tiles, STAGES deep;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma and commits;
//   warps 2..5  epilogue: tcgen05.ld their 32-lane quarter, apply the epilogue, store.
// Shared-memory tiles are [rows x 64] bfloat16 with the 128-byte swizzle that both
// TMA and the MMA descriptors understand.
//
// Epilogues: store bf16, store f32 (logits), add into f32 (the residual stream; with
// split-K through float32 atomics), and SwiGLU, where the CTA multiplies the same
// token tile with a gate tile and an up tile of the fused [2I, K] matrix into two
// accumulators and writes silu(gate) * up.  For prompt portions the fused QKV product can
// also rotate queries and keys and put keys and values into the cache pages in its epilogue
// (hx_gemm_tc_rope_append), which saves the separate pass over the projected rows.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets a status bit, the
// CTA skips its remaining work, frees its tensor memory and returns.
#include "hx_tcgen05.cuh"

#include <cuda.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

namespace {

constexpr int BM = 128;        // features per CTA (MMA M)
constexpr int BK = 64;         // k elements per stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;     // k elements per tcgen05.mma of kind::f16
constexpr int THREADS = 192;

enum Epilogue : int {
  EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3,
  EPI_ROPE_APPEND = 4      // persistent kernel only, see RopeArgs
};

// Where the [128 rows x 64 k] box of the weights that begins at row `row`, k-block `kb`, is.
// Row-major weights: a box is 128 row segments of 128 bytes, one per row of the matrix.  Tiled
// weights (k_tiles > 0) store every such box as 16 contiguous kilobytes, box after box along
// k, then along the rows: a product that streams its weights once then reads DRAM in long
// runs instead of 128-byte pieces (measured: 4 % less time for the decode products).
__device__ __forceinline__ void load_weight_box(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                int row, int kb, int k_tiles) {
  if (k_tiles > 0) {
    tma_load_2d(dst, map, bar, 0, ((row / BM) * k_tiles + kb) * BM);
  } else {
    tma_load_2d(dst, map, bar, kb * BK, row);
  }
}

// One epilogue warp's share of a finished tile: its 32 features (tensor-memory lanes) for all
// BN token columns, 16 columns at a time.  With SwiGLU the up accumulator sits BN columns on.
template <int BN, int EPI>
__device__ __forceinline__ void write_tile(void* out, int ldo, int tokens, int features,
                                           uint32_t lane_address, int feature, int token0) {
  const bool feature_ok = feature < features;
#pragma unroll 1
  for (int column = 0; column < BN; column += 16) {
    if (token0 + column >= tokens) break;   // uniform over the warp
    float acc[16];
    tmem_load16(lane_address + column, acc);
    if (EPI == EPI_SWIGLU) {
      float up[16];
      tmem_load16(lane_address + BN + column, up);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = hx_silu_fast(acc[j]) * up[j];
    }
    if (feature_ok) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int token = token0 + column + j;
        if (token < tokens) {
          const size_t index = static_cast<size_t>(token) * ldo + feature;
          if (EPI == EPI_STORE_BF16 || EPI == EPI_SWIGLU) {
            static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(acc[j]);
          } else if (EPI == EPI_STORE_F32) {
            static_cast<float*>(out)[index] = acc[j];
          } else {
            // a reduction at the memory side: nothing to wait for.  With one writer per
            // element the sum is still deterministic.
            atomicAdd(static_cast<float*>(out) + index, acc[j]);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------- kernel

template <int BN, bool DUAL>
struct TileConfig {
  static constexpr int kWeightBytes = BM * BK * 2 * (DUAL ? 2 : 1);
  static constexpr int kTokenBytes = BN * BK * 2;
  static constexpr int kStageBytes = kWeightBytes + kTokenBytes;
  // Token tiles up to 128 are the weight-streaming case (decoding, short prompt portions):
  // two CTAs share an SM so that one CTA's pipeline fill and epilogue overlap the other's
  // loads (with 128 tokens that leaves three stages of 32 KB each, and still wins: steps of
  // 65 to 128 tokens take 9 % less time than with one CTA of six stages).  Larger tiles take
  // the SM.
  static constexpr int kBudget = (BN <= 128 && !DUAL) ? 100 * 1024 : 200 * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
  static constexpr int kAccumulatorColumns = BN * (DUAL ? 2 : 1);
  static constexpr int kTmemColumns =
      kAccumulatorColumns <= 32 ? 32
      : kAccumulatorColumns <= 64 ? 64
      : kAccumulatorColumns <= 128 ? 128
      : kAccumulatorColumns <= 256 ? 256 : 512;
};

struct GemmArgs {
  void* out;
  int ldo;
  int tokens;
  int features;     // rows of the output the epilogue may write
  int depth;        // K
  int up_row_offset;  // SwiGLU: row of the first up-projection feature in the weight matrix
  int k_blocks_per_split;
  int k_tiles;        // > 0: the weights are stored as tiles, this many along k
  int* status;
};

template <int BN, int EPI>
__global__ __launch_bounds__(THREADS) void gemm_tc_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const GemmArgs args) {
  constexpr bool DUAL = EPI == EPI_SWIGLU;
  using Config = TileConfig<BN, DUAL>;
  constexpr int STAGES = Config::kStages;

  hx_pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Config::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // token tiles vary fastest: the CTAs that run side by side share a weight tile, which then
  // comes from DRAM once and from the L2 for the rest; the token tiles are L2-resident anyway
  const int feature0 = blockIdx.y * BM;
  const int token0 = blockIdx.x * BN;
  const int total_k_blocks = (args.depth + BK - 1) / BK;
  const int kb_begin = blockIdx.z * args.k_blocks_per_split;
  const int kb_end = min(kb_begin + args.k_blocks_per_split, total_k_blocks);
  const int n_k_blocks = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_holder, Config::kTmemColumns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (n_k_blocks > 0) {
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        // The weight tiles do not depend on the kernel before this one: the first STAGES of
        // them are requested at once, before the dependency wait, so that weights stream
        // across the kernel boundary.  The token tiles follow after the wait.
        const int eager = n_k_blocks < STAGES ? n_k_blocks : STAGES;
        for (int i = 0; i < eager; ++i) {
          uint8_t* stage = smem + i * Config::kStageBytes;
          mbar_expect_tx(&full_bar[i], Config::kStageBytes);
          load_weight_box(stage, &map_w, &full_bar[i], feature0, kb_begin + i, args.k_tiles);
          if (DUAL)
            load_weight_box(stage + BM * BK * 2, &map_w, &full_bar[i],
                            args.up_row_offset + feature0, kb_begin + i, args.k_tiles);
        }
        hx_pdl_wait();
        for (int i = 0; i < eager; ++i) {
          uint8_t* stage = smem + i * Config::kStageBytes;
          tma_load_2d(stage + Config::kWeightBytes, &map_x, &full_bar[i], (kb_begin + i) * BK,
                      token0);
        }
        for (int i = eager; i < n_k_blocks; ++i) {
          const int s = i % STAGES;
          const uint32_t round = static_cast<uint32_t>(i / STAGES);
          if (!mbar_wait(&empty_bar[s], (round & 1u) ^ 1u)) {
            atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
            break;
          }
          uint8_t* stage = smem + s * Config::kStageBytes;
          mbar_expect_tx(&full_bar[s], Config::kStageBytes);
          const int k = (kb_begin + i) * BK;
          load_weight_box(stage, &map_w, &full_bar[s], feature0, kb_begin + i, args.k_tiles);
          if (DUAL)
            load_weight_box(stage + BM * BK * 2, &map_w, &full_bar[s],
                            args.up_row_offset + feature0, kb_begin + i, args.k_tiles);
          tma_load_2d(stage + Config::kWeightBytes, &map_x, &full_bar[s], k, token0);
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc(BM, BN);
        bool ok = true;
        for (int i = 0; i < n_k_blocks && ok; ++i) {
          const int s = i % STAGES;
          const uint32_t round = static_cast<uint32_t>(i / STAGES);
          if (!mbar_wait(&full_bar[s], round & 1u)) {
            atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t stage = smem_u32(smem + s * Config::kStageBytes);
          const uint64_t desc_w = make_smem_desc(stage);
          const uint64_t desc_w2 = make_smem_desc(stage + BM * BK * 2);
          const uint64_t desc_x = make_smem_desc(stage + Config::kWeightBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // stepping 16 k-elements = 32 bytes inside the swizzle span: +2 in 16-byte units
            const uint64_t step = static_cast<uint64_t>(k * UMMA_K * 2 >> 4);
            const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
            umma_bf16(tmem_base, desc_w + step, desc_x + step, idesc, accumulate);
            if (DUAL) umma_bf16(tmem_base + BN, desc_w2 + step, desc_x + step, idesc, accumulate);
          }
          umma_commit(&empty_bar[s]);   // the stage may be refilled once these MMAs have read it
        }
        umma_commit(accum_bar);         // the accumulator is complete
      }
    } else {
      // ---------------------------------------------------------------- epilogue
      hx_pdl_wait();                    // the output may be something the last kernel read
      const int quarter = warp & 3;     // tensor-memory lanes [32 * quarter, 32 * quarter + 32)
      const int feature = feature0 + quarter * 32 + lane;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(accum_bar, 0);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
      } else {
        tc_fence_after();
        const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        write_tile<BN, EPI>(args.out, args.ldo, args.tokens, args.features, lane_address, feature,
                            token0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Config::kTmemColumns);
  }
}

// ------------------------------------------------- persistent kernel for prompt portions
//
// With hundreds of tokens the product is compute bound, and the tile's epilogue (reading a
// 128 x 256 accumulator back, converting, storing) takes a good part of the time of its main
// loop.  Here one CTA per SM walks a list of work units: all of shared memory is one ring of
// operand stages that runs on across units, tensor memory holds TWO accumulators of 256
// columns, and the epilogue warps drain one while the MMA warp fills the other.
//
// The tile is turned round with respect to the kernel above: 128 TOKENS are the MMA's M
// side and 256 weight rows its N side, so a thread of the epilogue owns one token and finds
// 256 consecutive features of it in its lane of tensor memory: it writes them 16 at a time
// with 16-byte stores (or 16-byte reductions into the float32 residual), which the memory
// system takes several times faster than the two-byte stores of a feature-per-thread layout.
// For SwiGLU the N side is 128 gate rows followed by the matching 128 up rows of the fused
// matrix: gate and up of a feature sit side by side in the thread's own lane.
//
// The add epilogue does not add at the memory side here (float32 reductions reach only about
// 1.8 TB/s in the L2, a quarter of what this product would need): while the MMA warp works on
// one accumulator, the epilogue warps load the output tile of the unit after it INTO the other
// accumulator (tcgen05.st), the products then accumulate on top of it, and the epilogue
// stores the sum.  One writer per element: the result is deterministic.
//
// Tiles are dealt round-robin with the token tile varying fastest, so the CTAs that run side
// by side read the same weight tiles at the same time, once from DRAM.

struct PersistentConfig {
  static constexpr int kRowsA = BM;              // tokens
  static constexpr int kRowsB = 2 * BM;          // weight rows: the accumulator's columns
  static constexpr int kBytesA = kRowsA * BK * 2;
  static constexpr int kBytesB = kRowsB * BK * 2;
  static constexpr int kStageBytes = kBytesA + kBytesB;
  static constexpr int kStages = 200 * 1024 / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
  static constexpr int kBufferColumns = 256;     // one accumulator per half of tensor memory
  static constexpr int kTmemColumns = 512;
};

// What the rotary/append epilogue needs beyond the product: the output row is
// [q heads | k heads | v heads], each head `head_dim` wide (a multiple of 16, so the 16
// features a thread handles at a time lie in one head).  Queries are rotated and stored to
// `out`; keys are rotated and, like the values, written into the token's slot of its page
// (k_cache == nullptr: the caller owns no cache, keys and values are dropped).  Pairs are
// adjacent coordinates (2p, 2p + 1); the first `rotary_dim` coordinates of a head rotate.
struct RopeArgs {
  const int* positions;
  const int* token_request;
  const int* request_table_row;
  const int* block_tables;
  int table_stride;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const float* cos_table;      // [table_positions][rotary_dim / 2]
  const float* sin_table;
  int table_positions;
  int heads, kv_heads, head_dim, rotary_dim, page_size, num_pages;
};

#ifndef HX_GEMM_STREAM_K
#define HX_GEMM_STREAM_K 1      // 0: every unit of the persistent kernel is a whole tile
#endif

struct PersistentArgs {
  void* out;
  int ldo;
  int tokens;
  int features;
  int depth;
  int up_row_offset;
  int k_tiles;                // > 0: the weights are stored as tiles, this many along k
  int token_tiles;            // tiles along the tokens
  int units;                  // token_tiles * feature tiles
  int k_blocks;               // per tile
  int* status;
  RopeArgs rope;              // EPI_ROPE_APPEND only
  int whole_rounds;           // >= 0: the tiles behind this many whole rounds are shared out by
                              // k-blocks (add epilogue only); -1: every unit is a whole tile
};

// What a CTA works on at a time: a tile, or (`partial`) a run of k-blocks of a tile that
// other CTAs hold the rest of.
struct Unit {
  int token_tile, feature_tile, kb_begin, kb_end;
  bool partial;
};

// The grid walks the tiles round by round.  The last round seldom fills the grid: 256 tiles
// on 148 CTAs are 1.73 rounds that cost 2.  Where the epilogue ADDS into a float32 output the
// order of the sum is free, so the tiles of that last round are laid end to end as one list
// of k-blocks and every CTA takes an equal run of it (one or two pieces of tiles), which it
// adds to the output with atomic adds; whole tiles keep the plain read-add-store.
__device__ __forceinline__ bool unit_at(const PersistentArgs& a, int iteration, Unit& u) {
  const int grid = static_cast<int>(gridDim.x);
  int index;
  if (a.whole_rounds < 0 || iteration < a.whole_rounds) {
    index = static_cast<int>(blockIdx.x) + iteration * grid;
    if (index >= a.units) return false;
    u.kb_begin = 0;
    u.kb_end = a.k_blocks;
    u.partial = false;
  } else {
    const int first = a.whole_rounds * grid;
    const long long blocks = static_cast<long long>(a.units - first) * a.k_blocks;
    const long long begin = blocks * blockIdx.x / grid;
    const long long end = blocks * (blockIdx.x + 1) / grid;
    const long long tile = begin / a.k_blocks + (iteration - a.whole_rounds);
    const long long from = max(begin, tile * a.k_blocks);
    const long long to = min(end, (tile + 1) * a.k_blocks);
    if (from >= to) return false;
    index = first + static_cast<int>(tile);
    u.kb_begin = static_cast<int>(from - tile * a.k_blocks);
    u.kb_end = static_cast<int>(to - tile * a.k_blocks);
    u.partial = u.kb_begin != 0 || u.kb_end != a.k_blocks;
  }
  u.token_tile = index % a.token_tiles;
  u.feature_tile = index / a.token_tiles;
  return true;
}

// The add epilogue's preparation: this thread's token, 256 columns of the float32 output
// into its lane of the accumulator (zeros where the tile hangs over the output's edge).
__device__ __forceinline__ void load_row_into_accumulator(const float* out, int ldo, int features,
                                                          uint32_t lane_address, int token,
                                                          int tokens, int feature0) {
  const bool wide = (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  const float* row = out + static_cast<size_t>(token < tokens ? token : 0) * ldo + feature0;
#pragma unroll 1
  for (int group = 0; group < 2 * BM; group += 64) {
    float v[4][16];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int column = group + c * 16;
      if (token < tokens && wide && feature0 + column + 16 <= features) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 x = *reinterpret_cast<const float4*>(row + column + 4 * j);
          v[c][4 * j] = x.x;
          v[c][4 * j + 1] = x.y;
          v[c][4 * j + 2] = x.z;
          v[c][4 * j + 3] = x.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          v[c][j] = (token < tokens && feature0 + column + j < features) ? row[column + j] : 0.0f;
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_store16(lane_address + group + c * 16, v[c]);
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// This thread's token: `columns` features starting at feature0, 16 at a time, from its lane of
// the accumulator.  With SwiGLU the accumulator holds 128 gate columns, then 128 up columns.
template <int EPI>
__device__ __forceinline__ void write_row(void* out, int ldo, int features, uint32_t lane_address,
                                          int token, int tokens, int feature0) {
  using Element = typename std::conditional<EPI == EPI_STORE_BF16 || EPI == EPI_SWIGLU,
                                            __nv_bfloat16, float>::type;
  constexpr int kColumns = EPI == EPI_SWIGLU ? BM : 2 * BM;
  const bool wide = (ldo % (16 / static_cast<int>(sizeof(Element))) == 0) &&
                    ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll 1
  for (int column = 0; column < kColumns; column += 16) {
    if (feature0 + column >= features) break;      // uniform over the warp
    float acc[16];
    tmem_load16(lane_address + column, acc);
    if (EPI == EPI_SWIGLU) {
      float up[16];
      tmem_load16(lane_address + BM + column, up);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = hx_silu_fast(acc[j]) * up[j];
    }
    if (token >= tokens) continue;
    Element* row = static_cast<Element*>(out) + static_cast<size_t>(token) * ldo + feature0 + column;
    if (wide && feature0 + column + 16 <= features) {
      if constexpr (std::is_same<Element, __nv_bfloat16>::value) {
        uint4 packed[2];
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) pairs[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        reinterpret_cast<uint4*>(row)[0] = packed[0];
        reinterpret_cast<uint4*>(row)[1] = packed[1];
      } else {
        // the add epilogue too: the accumulator began as the output's old value
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<float4*>(row)[j] =
              make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (feature0 + column + j < features) {
          if constexpr (std::is_same<Element, __nv_bfloat16>::value) {
            row[j] = __float2bfloat16_rn(acc[j]);
          } else {
            row[j] = acc[j];
          }
        }
      }
    }
  }
}

// The rotary/append epilogue for this thread's token: the same arithmetic as the separate
// kernel (hx_rope_append) applied to the product rounded to bfloat16, as the plain store
// would have rounded it: rotation in float32 from the cos/sin table, one more rounding.
__device__ __forceinline__ void write_row_rope(const PersistentArgs& a, uint32_t lane_address,
                                               int token, int feature0) {
  const RopeArgs& r = a.rope;
  const bool live = token < a.tokens;
  const int half = r.rotary_dim / 2;
  const float* cos_row = r.cos_table;
  const float* sin_row = r.sin_table;
  int page = -1, slot = 0;
  if (live) {
    const int position = r.positions[token];
    const int table_position = min(max(position, 0), r.table_positions - 1);
    if (table_position != position && r.rotary_dim > 0 && feature0 == 0 && a.status != nullptr)
      atomicOr(a.status, HX_FLAG_BAD_POSITION);
    cos_row += static_cast<size_t>(table_position) * half;
    sin_row += static_cast<size_t>(table_position) * half;
    if (r.k_cache != nullptr) {
      const int table_row = r.request_table_row[r.token_request[token]];
      page = r.block_tables[static_cast<size_t>(table_row) * r.table_stride + position / r.page_size];
      slot = position % r.page_size;
      if (page < 0 || page >= r.num_pages) {
        atomicOr(a.status, HX_FLAG_BAD_PAGE);
        page = -1;
      }
    }
  }
  const int q_features = r.heads * r.head_dim;
  const int k_end = q_features + r.kv_heads * r.head_dim;
  const bool wide_table = half % 4 == 0 &&
                          ((reinterpret_cast<uintptr_t>(r.cos_table) |
                            reinterpret_cast<uintptr_t>(r.sin_table)) & 15) == 0;
#pragma unroll 1
  for (int column = 0; column < 2 * BM; column += 16) {
    const int feature = feature0 + column;
    if (feature >= a.features) break;      // uniform over the warp
    float x[16];
    tmem_load16(lane_address + column, x);
    if (!live) continue;
    const bool is_query = feature < q_features;
    const bool is_key = !is_query && feature < k_end;
    const int inside = feature - (is_query ? 0 : (is_key ? q_features : k_end));
    const int head = inside / r.head_dim;
    const int d0 = inside - head * r.head_dim;
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = __bfloat162float(__float2bfloat16_rn(x[j]));
    if ((is_query || is_key) && d0 < r.rotary_dim) {
      // the eight angles of this piece: four 16-byte loads where the table's rows allow it
      // (every lane reads another row of the table, so the number of loads is what counts)
      float c[8], sn[8];
      if (wide_table && d0 + 16 <= r.rotary_dim) {
        const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_row + d0 / 2));
        const float4 c1 = __ldg(reinterpret_cast<const float4*>(cos_row + d0 / 2 + 4));
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_row + d0 / 2));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(sin_row + d0 / 2 + 4));
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
        c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w;
        sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool rotates = d0 + 2 * i + 1 < r.rotary_dim;
          c[i] = rotates ? __ldg(cos_row + d0 / 2 + i) : 1.0f;
          sn[i] = rotates ? __ldg(sin_row + d0 / 2 + i) : 0.0f;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float u = x[2 * i], v = x[2 * i + 1];
        x[2 * i] = u * c[i] - v * sn[i];
        x[2 * i + 1] = u * sn[i] + v * c[i];
      }
    }
    uint4 packed[2];
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
    for (int j = 0; j < 8; ++j) pairs[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
    if (is_query) {
      uint4* row = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) +
                                            static_cast<size_t>(token) * a.ldo + feature);
      row[0] = packed[0];
      row[1] = packed[1];
    } else if (page >= 0) {
      __nv_bfloat16* cache = is_key ? r.k_cache : r.v_cache;
      *reinterpret_cast<uint4*>(cache + hx_cache_offset(page, head, slot, d0, r.kv_heads,
                                                        r.page_size, r.head_dim, 8)) = packed[0];
      *reinterpret_cast<uint4*>(cache + hx_cache_offset(page, head, slot, d0 + 8, r.kv_heads,
                                                        r.page_size, r.head_dim, 8)) = packed[1];
    }
  }
}

// The piece of a tile that a partial unit computed: added to the float32 output with atomic
// adds (four values at a time where the row allows).
__device__ __forceinline__ void add_row_atomically(float* out, int ldo, int features,
                                                   uint32_t lane_address, int token, int tokens,
                                                   int feature0) {
  const bool wide = (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll 1
  for (int column = 0; column < 2 * BM; column += 16) {
    if (feature0 + column >= features) break;      // uniform over the warp
    float acc[16];
    tmem_load16(lane_address + column, acc);
    if (token >= tokens) continue;
    float* row = out + static_cast<size_t>(token) * ldo + feature0 + column;
    if (wide && feature0 + column + 16 <= features) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(row + 4 * j),
                     "f"(acc[4 * j]), "f"(acc[4 * j + 1]), "f"(acc[4 * j + 2]),
                     "f"(acc[4 * j + 3]) : "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (feature0 + column + j < features) atomicAdd(row + j, acc[j]);
    }
  }
}

template <int EPI>
__global__ __launch_bounds__(THREADS) void gemm_tc_persistent_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const PersistentArgs args) {
  using Config = PersistentConfig;
  constexpr int STAGES = Config::kStages;
  // features of the output per tile, and where the second half of the N operand comes from
  constexpr int FEATURES = EPI == EPI_SWIGLU ? BM : 2 * BM;

  hx_pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Config::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;      // [2]: the accumulator is complete
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;      // [2]: the epilogue has read it
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 4);      // one arrival per epilogue warp
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_holder, Config::kTmemColumns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  hx_pdl_wait();

  if (warp == 0) {
    // -------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t fill = 0;      // stages filled so far, over all units
      Unit unit;
      for (int iteration = 0; unit_at(args, iteration, unit) && !*failed; ++iteration) {
        const int feature0 = unit.feature_tile * FEATURES;
        const int second_half = EPI == EPI_SWIGLU ? args.up_row_offset + feature0 : feature0 + BM;
        const int token0 = unit.token_tile * BM;
        for (int kb = unit.kb_begin; kb < unit.kb_end; ++kb, ++fill) {
          const int s = fill % STAGES;
          const uint32_t round = fill / STAGES;
          if (!mbar_wait(&empty_bar[s], (round & 1u) ^ 1u)) {
            atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
            *failed = 1;
            break;
          }
          uint8_t* stage = smem + s * Config::kStageBytes;
          mbar_expect_tx(&full_bar[s], Config::kStageBytes);
          const int k = kb * BK;
          tma_load_2d(stage, &map_x, &full_bar[s], k, token0);
          load_weight_box(stage + Config::kBytesA, &map_w, &full_bar[s], feature0, kb, args.k_tiles);
          load_weight_box(stage + Config::kBytesA + BM * BK * 2, &map_w, &full_bar[s], second_half,
                          kb, args.k_tiles);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, Config::kRowsB);
      uint32_t drained = 0;      // stages consumed so far, over all units
      Unit unit;
      for (int iteration = 0; unit_at(args, iteration, unit) && !*failed; ++iteration) {
        const int buffer = iteration & 1;
        const uint32_t use = static_cast<uint32_t>(iteration >> 1);
        // the epilogue must have read this accumulator's previous unit (and, for the add
        // epilogue, have loaded this unit's old output into it: one more arrival)
        if (!mbar_wait(&tmem_empty_bar[buffer], EPI == EPI_ADD_F32 ? (use & 1u) : (use & 1u) ^ 1u)) {
          atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
          break;
        }
        tc_fence_after();
        const uint32_t accumulator = tmem_base + buffer * Config::kBufferColumns;
        for (int kb = unit.kb_begin; kb < unit.kb_end; ++kb, ++drained) {
          const int s = drained % STAGES;
          const uint32_t round = drained / STAGES;
          if (!mbar_wait(&full_bar[s], round & 1u)) {
            atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
            *failed = 1;
            break;
          }
          tc_fence_after();
          const uint32_t stage = smem_u32(smem + s * Config::kStageBytes);
          const uint64_t desc_a = make_smem_desc(stage);
          const uint64_t desc_b = make_smem_desc(stage + Config::kBytesA);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t step = static_cast<uint64_t>(k * UMMA_K * 2 >> 4);
            // a whole tile of the add epilogue starts from the old output in the accumulator
            const uint32_t accumulate =
                ((EPI == EPI_ADD_F32 && !unit.partial) || kb > unit.kb_begin || k > 0) ? 1u : 0u;
            umma_bf16(accumulator, desc_a + step, desc_b + step, idesc, accumulate);
          }
          umma_commit(&empty_bar[s]);
        }
        if (*failed) break;
        umma_commit(&tmem_full_bar[buffer]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;     // tensor-memory lanes [32 * quarter, 32 * quarter + 32)
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    Unit unit;
    // add epilogue: the old output of unit `iteration` goes into its accumulator, which is
    // then handed to the MMA warp
    auto prepare = [&](int iteration) {
      if (EPI != EPI_ADD_F32 || !unit_at(args, iteration, unit)) return;
      const int buffer = iteration & 1;
      if (!unit.partial)      // a piece starts from zero and is added to the output afterwards
        load_row_into_accumulator(static_cast<const float*>(args.out), args.ldo, args.features,
                                  lane_base + buffer * Config::kBufferColumns,
                                  unit.token_tile * BM + quarter * 32 + lane, args.tokens,
                                  unit.feature_tile * FEATURES);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buffer]);
    };
    prepare(0);
    prepare(1);
    for (int iteration = 0; unit_at(args, iteration, unit) && !*failed; ++iteration) {
      const int buffer = iteration & 1;
      const uint32_t use = static_cast<uint32_t>(iteration >> 1);
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&tmem_full_bar[buffer], use & 1u);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) {
          atomicOr(args.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
        }
        break;
      }
      tc_fence_after();
      if constexpr (EPI == EPI_ROPE_APPEND) {
        write_row_rope(args, lane_base + buffer * Config::kBufferColumns,
                       unit.token_tile * BM + quarter * 32 + lane, unit.feature_tile * FEATURES);
      } else if (EPI == EPI_ADD_F32 && unit.partial) {
        add_row_atomically(static_cast<float*>(args.out), args.ldo, args.features,
                           lane_base + buffer * Config::kBufferColumns,
                           unit.token_tile * BM + quarter * 32 + lane, args.tokens,
                           unit.feature_tile * FEATURES);
      } else {
        write_row<EPI>(args.out, args.ldo, args.features,
                       lane_base + buffer * Config::kBufferColumns,
                       unit.token_tile * BM + quarter * 32 + lane, args.tokens,
                       unit.feature_tile * FEATURES);
      }
      // every lane's tcgen05.ld has completed (the loads are waited for where they are
      // issued): hand the accumulator back
      if (EPI == EPI_ADD_F32) {
        prepare(iteration + 2);
      } else {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[buffer]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Config::kTmemColumns);
  }
}

// ----------------------------------------------------------------- host side

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(symbol);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t rows;
  uint64_t depth;
  uint64_t ld;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && depth == o.depth && ld == o.ld &&
           box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1315423911u ^ k.rows;
    h = h * 1315423911u ^ k.depth;
    h = h * 1315423911u ^ k.ld;
    h = h * 1315423911u ^ k.box_rows;
    return h;
  }
};

// Tensor maps are pure functions of (address, shape, box); encoding one costs a few
// microseconds, so they are cached for the life of the process.
int get_tensor_map(const void* base, uint64_t rows, uint64_t depth, uint64_t ld, uint32_t box_rows,
                   CUtensorMap* out) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, depth, ld, box_rows};
  std::lock_guard<std::mutex> lock(mutex);
  auto found = cache.find(key);
  if (found != cache.end()) {
    *out = found->second;
    return HX_OK;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) {
    hx_set_error("hx_gemm_tc: the driver does not export cuTensorMapEncodeTiled");
    return HX_ERR_UNSUPPORTED;
  }
  const cuuint64_t dims[2] = {depth, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                             dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    hx_set_error("hx_gemm_tc: cuTensorMapEncodeTiled failed with %d (base %p rows %llu depth %llu "
                 "ld %llu box %u)", static_cast<int>(rc), base,
                 static_cast<unsigned long long>(rows), static_cast<unsigned long long>(depth),
                 static_cast<unsigned long long>(ld), box_rows);
    return HX_ERR_ARGUMENT;
  }
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return HX_OK;
}

template <int BN, int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmArgs& args, dim3 grid,
           cudaStream_t stream) {
  using Config = TileConfig<BN, EPI == EPI_SWIGLU>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Config::kSmemBytes) != cudaSuccess) {
      hx_set_error("hx_gemm_tc: cannot reserve %d bytes of shared memory", Config::kSmemBytes);
      cudaGetLastError();
      return HX_ERR_LAUNCH;
    }
    configured = true;
  }
  hx_launch(gemm_tc_kernel<BN, EPI>, grid, THREADS, Config::kSmemBytes, stream, map_w, map_x, args);
  return HX_OK;
}

template <int BN>
int launch_epilogue(int epilogue, const CUtensorMap& map_w, const CUtensorMap& map_x,
                    const GemmArgs& args, dim3 grid, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_BF16: return launch<BN, EPI_STORE_BF16>(map_w, map_x, args, grid, stream);
    case EPI_STORE_F32: return launch<BN, EPI_STORE_F32>(map_w, map_x, args, grid, stream);
    case EPI_ADD_F32: return launch<BN, EPI_ADD_F32>(map_w, map_x, args, grid, stream);
    case EPI_SWIGLU: return launch<BN, EPI_SWIGLU>(map_w, map_x, args, grid, stream);
    default:
      hx_set_error("hx_gemm_tc: unknown epilogue %d", epilogue);
      return HX_ERR_ARGUMENT;
  }
}

template <int EPI>
int launch_persistent(const CUtensorMap& map_w, const CUtensorMap& map_x, PersistentArgs args,
                      cudaStream_t stream) {
  using Config = PersistentConfig;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    int device = 0;
    if (cudaFuncSetAttribute(gemm_tc_persistent_kernel<EPI>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Config::kSmemBytes) != cudaSuccess ||
        cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        sms <= 0) {
      hx_set_error("hx_gemm_tc: cannot reserve %d bytes of shared memory", Config::kSmemBytes);
      cudaGetLastError();
      return HX_ERR_LAUNCH;
    }
    configured = true;
  }
  constexpr int kFeatures = EPI == EPI_SWIGLU ? BM : 2 * BM;
  const int feature_tiles = (args.features + kFeatures - 1) / kFeatures;
  args.token_tiles = (args.tokens + BM - 1) / BM;
  const long long tiles = static_cast<long long>(args.token_tiles) * feature_tiles;
  HX_REQUIRE(tiles < (1ll << 30), "hx_gemm_tc: too many tiles");
  args.units = static_cast<int>(tiles);
  // The add epilogue shares the last, partly filled round out by k-blocks (see unit_at) when
  // that pays.  Every piece costs an epilogue of atomic adds (128 KB of them, all CTAs at the
  // same time), which measured about as much as 30 k-blocks of products: with 2,048 tokens
  // (108 tiles left for 148 SMs) sharing out gains nothing, with 512 tokens (64 tiles, less
  // than half the grid) the output and down projections take 20 % and 23 % less time.
  args.whole_rounds = -1;
  int ctas = args.units < sms ? args.units : sms;
  if (EPI == EPI_ADD_F32 && HX_GEMM_STREAM_K) {
    const int rest = args.units % sms;
    const long long run = static_cast<long long>(rest) * args.k_blocks / sms;
    if (rest > 0 && rest * 2 <= sms && run >= 8 && args.k_blocks - run >= 32) {
      args.whole_rounds = args.units / sms;
      ctas = sms;
    }
  }
  hx_launch(gemm_tc_persistent_kernel<EPI>, ctas, THREADS, Config::kSmemBytes, stream, map_w,
            map_x, args);
  return HX_OK;
}

int launch_persistent_epilogue(int epilogue, const CUtensorMap& map_w, const CUtensorMap& map_x,
                               const PersistentArgs& args, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_BF16: return launch_persistent<EPI_STORE_BF16>(map_w, map_x, args, stream);
    case EPI_STORE_F32: return launch_persistent<EPI_STORE_F32>(map_w, map_x, args, stream);
    case EPI_ADD_F32: return launch_persistent<EPI_ADD_F32>(map_w, map_x, args, stream);
    case EPI_SWIGLU: return launch_persistent<EPI_SWIGLU>(map_w, map_x, args, stream);
    case EPI_ROPE_APPEND: return launch_persistent<EPI_ROPE_APPEND>(map_w, map_x, args, stream);
    default:
      hx_set_error("hx_gemm_tc: unknown epilogue %d", epilogue);
      return HX_ERR_ARGUMENT;
  }
}

}  // namespace

// Token tile the kernel would use for this many tokens (for tests and the bench's records).
HX_API int hx_gemm_tc_token_tile(int tokens) {
  if (tokens <= 16) return 16;
  if (tokens <= 32) return 32;
  if (tokens <= 64) return 64;
  if (tokens <= 128) return 128;
  return 256;
}

// 1 when the tensor-core kernel takes this shape; 0 when the caller must use hx_gemm_simt.
HX_API int hx_gemm_tc_supports(int tokens, int features, int depth, int ldx, int ldw) {
  return tokens > 0 && features > 0 && depth > 0 && depth % 8 == 0 && ldx % 8 == 0 &&
         ldw % 8 == 0;
}

// x: [tokens, depth] bf16 (row stride ldx), w: [weight_rows, depth] bf16 (row stride ldw).
// epilogue 0/1/2: `features` = weight_rows outputs per token.  epilogue 3 (SwiGLU): w is the
// fused [gate; up] matrix, `features` = intermediate size, gate rows [0, features), up rows
// [up_row_offset, up_row_offset + features).  k_splits > 1 only with epilogue 2.
// weight_tiles != 0: w holds the matrix as [ceil(weight_rows / 128)][ceil(depth / 64)] tiles of
// [128][64] elements, zero padded (ldw is ignored; up_row_offset is then a multiple of 128).
// x_capacity_rows: rows of the buffer behind x (the tensor map is made for the buffer, so it
// can be reused for every batch size).
HX_API int hx_gemm_tc(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                      int weight_rows, void* out, int ldo, int tokens, int features, int depth,
                      int epilogue, int up_row_offset, int k_splits, int weight_tiles, int* status,
                      cudaStream_t stream) {
  if (weight_tiles) ldw = 8;      // not a stride of anything here
  HX_REQUIRE(!weight_tiles || epilogue != EPI_SWIGLU || up_row_offset % BM == 0,
             "hx_gemm_tc: with tiled weights the up rows must start on a multiple of %d", BM);
  HX_REQUIRE(hx_gemm_tc_supports(tokens, features, depth, ldx, ldw),
             "hx_gemm_tc: shape tokens=%d features=%d depth=%d ldx=%d ldw=%d is not supported "
             "(depth and strides must be multiples of 8)", tokens, features, depth, ldx, ldw);
  HX_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
             "hx_gemm_tc: operands must be 16-byte aligned");
  HX_REQUIRE(x_capacity_rows >= tokens, "hx_gemm_tc: buffer rows %d < tokens %d", x_capacity_rows,
             tokens);
  HX_REQUIRE(status != nullptr, "hx_gemm_tc: status word missing");
  HX_REQUIRE(epilogue >= EPI_STORE_BF16 && epilogue <= EPI_SWIGLU,
             "hx_gemm_tc: unknown epilogue %d", epilogue);
  HX_REQUIRE(k_splits >= 1 && (k_splits == 1 || epilogue == EPI_ADD_F32),
             "hx_gemm_tc: split-K needs the add epilogue");
  HX_REQUIRE(epilogue != EPI_SWIGLU || up_row_offset + features <= weight_rows,
             "hx_gemm_tc: up rows exceed the weight matrix");
  HX_REQUIRE(epilogue == EPI_SWIGLU || features <= weight_rows,
             "hx_gemm_tc: features exceed the weight matrix");
  HX_REQUIRE(ldo >= features, "hx_gemm_tc: output stride too small");

  const int bn = hx_gemm_tc_token_tile(tokens);
  // prompt portions: the persistent kernel, whose tiles have 128 tokens on the M side.  A sum
  // into a float32 output over at most 128 tokens is a weight stream even when it is not cut
  // along the reduction (the fused gate/up matrix has tiles enough as it is) and stays with
  // the streaming kernel: 128 weight rows per CTA, two CTAs an SM (measured: steps of 65 to
  // 128 tokens take 6 to 8 % less time than with that one product on the persistent kernel).
  const bool persistent = bn >= 128 && k_splits == 1 && !(epilogue == EPI_ADD_F32 && tokens <= 128);
  CUtensorMap map_w, map_x;
  const int total_k_blocks = (depth + BK - 1) / BK;
  const int k_tiles = weight_tiles ? total_k_blocks : 0;
  int rc = weight_tiles
               ? get_tensor_map(w, static_cast<uint64_t>((weight_rows + BM - 1) / BM) * k_tiles * BM,
                                BK, BK, BM, &map_w)
               : get_tensor_map(w, weight_rows, depth, ldw, BM, &map_w);
  if (rc != HX_OK) return rc;
  rc = get_tensor_map(x, x_capacity_rows, depth, ldx, persistent ? BM : bn, &map_x);
  if (rc != HX_OK) return rc;

  if (persistent) {
    PersistentArgs args{out, ldo, tokens, features, depth, up_row_offset, k_tiles, 0, 0,
                        total_k_blocks, status, RopeArgs{}};
    rc = launch_persistent_epilogue(epilogue, map_w, map_x, args, stream);
    if (rc != HX_OK) return rc;
    HX_CHECK_LAUNCH("hx_gemm_tc");
    return HX_OK;
  }
  if (k_splits > total_k_blocks) k_splits = total_k_blocks;
  const int per_split = (total_k_blocks + k_splits - 1) / k_splits;
  k_splits = (total_k_blocks + per_split - 1) / per_split;
  GemmArgs args{out, ldo, tokens, features, depth, up_row_offset, per_split, k_tiles, status};
  const dim3 grid((tokens + bn - 1) / bn, (features + BM - 1) / BM, k_splits);
  HX_REQUIRE(grid.y <= 65535, "hx_gemm_tc: too many features (%d)", features);

  switch (bn) {
    case 16: rc = launch_epilogue<16>(epilogue, map_w, map_x, args, grid, stream); break;
    case 32: rc = launch_epilogue<32>(epilogue, map_w, map_x, args, grid, stream); break;
    case 64: rc = launch_epilogue<64>(epilogue, map_w, map_x, args, grid, stream); break;
    case 128: rc = launch_epilogue<128>(epilogue, map_w, map_x, args, grid, stream); break;
    default: rc = launch_epilogue<256>(epilogue, map_w, map_x, args, grid, stream); break;
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_gemm_tc");
  return HX_OK;
}

// Fewest tokens hx_gemm_tc_rope_append takes: it exists for the persistent kernel only.
HX_API int hx_gemm_tc_rope_append_min_tokens() { return 65; }

// The fused QKV product of a prompt portion with the rotary encoding and the cache append as
// its epilogue: qkv[t] = x[t] @ w.T with w = [q heads | k heads | v heads] x head_dim rows;
// the queries are rotated and stored to `out` (row stride ldo; the key and value parts of an
// out row are NOT written), the keys are rotated and, like the values, written to the
// token's slot of its page in k_cache / v_cache (both nullptr: dropped).  The arguments from
// `positions` on mean what they mean to hx_rope_append, with adjacent pairs; x, w, ldx, ldw,
// x_capacity_rows, weight_rows and weight_tiles what they mean to hx_gemm_tc.  Needs more
// than 64 tokens, bfloat16, head_dim a multiple of 16 and 16-byte aligned out and caches.
HX_API int hx_gemm_tc_rope_append(const void* x, int ldx, int x_capacity_rows, const void* w,
                                  int ldw, int weight_rows, void* out, int ldo, int tokens,
                                  int depth, int weight_tiles, const int* positions,
                                  const int* token_request, const int* request_table_row,
                                  const int* block_tables, int table_stride, void* k_cache,
                                  void* v_cache, const float* cos_table, const float* sin_table,
                                  int table_positions, int heads, int kv_heads, int head_dim,
                                  int rotary_dim, int page_size, int num_pages, int* status,
                                  cudaStream_t stream) {
  if (weight_tiles) ldw = 8;      // not a stride of anything here
  HX_REQUIRE(heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 16 == 0,
             "hx_gemm_tc_rope_append: head_dim %d must be a multiple of 16", head_dim);
  HX_REQUIRE(static_cast<long long>(heads + 2 * kv_heads) * head_dim <= weight_rows,
             "hx_gemm_tc_rope_append: %d + 2 x %d heads of %d exceed the %d weight rows", heads,
             kv_heads, head_dim, weight_rows);
  const int features = (heads + 2 * kv_heads) * head_dim;
  HX_REQUIRE(tokens >= hx_gemm_tc_rope_append_min_tokens(),
             "hx_gemm_tc_rope_append: %d tokens; it takes prompt portions of at least %d", tokens,
             hx_gemm_tc_rope_append_min_tokens());
  HX_REQUIRE(hx_gemm_tc_supports(tokens, features, depth, ldx, ldw),
             "hx_gemm_tc_rope_append: shape tokens=%d features=%d depth=%d ldx=%d ldw=%d is not "
             "supported (depth and strides must be multiples of 8)", tokens, features, depth, ldx,
             ldw);
  HX_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
             "hx_gemm_tc_rope_append: rotary_dim %d must be even and at most head_dim %d",
             rotary_dim, head_dim);
  HX_REQUIRE(rotary_dim == 0 || (table_positions > 0 && cos_table && sin_table),
             "hx_gemm_tc_rope_append: rotary table missing");
  HX_REQUIRE((k_cache == nullptr) == (v_cache == nullptr),
             "hx_gemm_tc_rope_append: key and value cache come together");
  HX_REQUIRE(k_cache == nullptr || (page_size > 0 && num_pages > 0 && table_stride > 0 &&
                                    token_request && request_table_row && block_tables),
             "hx_gemm_tc_rope_append: cache arguments missing");
  HX_REQUIRE(positions != nullptr && status != nullptr,
             "hx_gemm_tc_rope_append: positions or status word missing");
  HX_REQUIRE(ldo >= heads * head_dim && ldo % 8 == 0,
             "hx_gemm_tc_rope_append: output stride %d must hold the queries and be a multiple "
             "of 8", ldo);
  HX_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
             "hx_gemm_tc_rope_append: operands must be 16-byte aligned");
  HX_REQUIRE(x_capacity_rows >= tokens, "hx_gemm_tc_rope_append: buffer rows %d < tokens %d",
             x_capacity_rows, tokens);

  CUtensorMap map_w, map_x;
  const int total_k_blocks = (depth + BK - 1) / BK;
  const int k_tiles = weight_tiles ? total_k_blocks : 0;
  int rc = weight_tiles
               ? get_tensor_map(w, static_cast<uint64_t>((weight_rows + BM - 1) / BM) * k_tiles * BM,
                                BK, BK, BM, &map_w)
               : get_tensor_map(w, weight_rows, depth, ldw, BM, &map_w);
  if (rc != HX_OK) return rc;
  rc = get_tensor_map(x, x_capacity_rows, depth, ldx, BM, &map_x);
  if (rc != HX_OK) return rc;
  PersistentArgs args{out, ldo, tokens, features, depth, 0, k_tiles, 0, 0, total_k_blocks, status,
                      RopeArgs{positions, token_request, request_table_row, block_tables,
                               table_stride, static_cast<__nv_bfloat16*>(k_cache),
                               static_cast<__nv_bfloat16*>(v_cache), cos_table, sin_table,
                               table_positions, heads, kv_heads, head_dim, rotary_dim, page_size,
                               num_pages}};
  rc = launch_persistent_epilogue(EPI_ROPE_APPEND, map_w, map_x, args, stream);
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_gemm_tc_rope_append");
  return HX_OK;
}

// ------------------------------------------------------------ the bounded wait, by itself
//
// What a kernel of this library does when an mbarrier it waits for never completes: the wait
// gives up after its limit, the thread sets HX_FLAG_WAIT_TIMEOUT in the status word and the
// kernel returns; the host then fails the step.  This entry point runs exactly that path on a
// barrier of its own, with a limit of `polls` polls instead of the kernels' forty million, so
// that the path can be exercised in a fraction of a millisecond: with `arrive` = 0 nobody
// ever arrives at the barrier and the wait must run out; with `arrive` = 1 the waiting
// thread's own arrival completes the phase first and the wait must succeed.  `succeeded`
// (device, one int, may be null) receives 1 when the wait succeeded and 0 when it ran out.
namespace {

__global__ void bounded_wait_kernel(uint32_t polls, int arrive, int* status, int* succeeded) {
  __shared__ __align__(8) uint64_t barrier;
  hx_pdl_prologue();
  if (threadIdx.x == 0) {
    mbar_init(&barrier, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (arrive) mbar_arrive(&barrier);
    const bool ok = mbar_wait(&barrier, 0, polls);
    if (!ok && status != nullptr) atomicOr(status, HX_FLAG_WAIT_TIMEOUT);
    if (succeeded != nullptr) *succeeded = ok ? 1 : 0;
  }
}

}  // namespace

HX_API int hx_bounded_wait_check(int polls, int arrive, int* status, int* succeeded,
                                 cudaStream_t stream) {
  HX_REQUIRE(polls > 0 && polls <= 1000000, "hx_bounded_wait_check: 1 to 1,000,000 polls");
  HX_REQUIRE(status != nullptr, "hx_bounded_wait_check: status word missing");
  hx_launch(bounded_wait_kernel, 1, 32, 0, stream, static_cast<uint32_t>(polls), arrive, status,
            succeeded);
  HX_CHECK_LAUNCH("hx_bounded_wait_check");
  return HX_OK;
}
