// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05),
// bfloat16 storage.  The same computation as hx_attention_mma.cu (the reference materialises
// a [heads, T, T] score tensor for it, src/attention/cuda.cu:31-77), with both products as
// tcgen05.mma and the scores, the probabilities and the output in tensor memory.
//
// One CTA takes 256 consecutive query tokens of one request and one head, as two lanes of 128
// rows (the M of a product), and walks the request's keys in tiles of 64, anchored at key 0.
// The lanes share the keys and values in shared memory and nothing else: each has its own
// thread issuing score products, its own four softmax warps, its own thread issuing output
// products and its own accumulators in tensor memory.  The second lane's rows see up to two
// key tiles more than the first's; a short request may leave it empty.  Warp roles:
//   warps 0, 1  one lane of each asks for the pages of each tile, warp 0 for the keys and
//               warp 1 for the values: the keys of a (page, head) are one contiguous block of
//               the cache and so are its values, so a tile is a handful of bulk copies
//               (cp.async.bulk counted on an mbarrier) into a ring of stages;
//   warp 2      rewrites the keys of a landed tile piece-major over all 64 keys (see below);
//   warps 3, 4  one lane each issues S_l = Q_l K^T for lane l into one of the lane's two score
//               buffers in tensor memory, a tile ahead of the softmax;
//   warps 5, 6  one lane each issues O_l += P_l V;
//   warp 7      idles (the softmax groups start at a multiple of four warps, which is what
//               selects their rows of tensor memory);
//   warps 8-11, 12-15  softmax of lane 0 / lane 1: thread r owns query row r of its lane.  It
//               reads its row of S from tensor memory, keeps the running maximum and sum in
//               float32 registers and writes the probabilities back over the scores it has
//               read, as TWO bfloat16 terms (P = hi + lo, so the softmax stays a float32
//               quantity as far as the result can tell).  P is the A operand of O += P V
//               straight from tensor memory, and O stays in tensor memory over all tiles.  The
//               maximum a row's exponentials are taken against is only raised when a tile
//               exceeds it by more than 2^8 (any fixed reference gives the same quotient;
//               float32 has the range), so the pass over O that a new maximum costs is rare.
//
// Why two lanes and four issuing threads: a thread needs 55 ns and more to issue one
// tcgen05.mma, whatever its size, while the tensor pipe finishes a product of 64 or 128
// columns in 30 to 35 ns (measured: one to four threads issuing side by side each keep their
// own rate until the pipe is full); one softmax group alone leaves its four schedulers waiting
// on the latencies of tensor-memory loads and stores and on the exponential unit; and what a
// CTA spends before its first and after its last tile (about 12 us: some 3 us until its first
// loads from global memory are back, queries and page table alike, then first pages, rewrite,
// the chain of first products; at the end the last product and the output) is spent once for
// 256 rows, and every key tile is fetched and rewritten once for them.
//
// Operand layouts.  Nothing is swizzled: every operand is made of "core matrices" of 8 rows
// x 16 bytes (128 contiguous bytes), which is exactly what a page block of the cache is made
// of ([head_dim / 8][slot][8 elements]: eight consecutive slots of one 16-byte piece).  For
// O = P V a page block is used as it lies: 16 keys are the K dimension of an MN-major operand
// (a row of a core matrix is 8 consecutive coordinates of one key, its 8 rows are 8 keys).
// For S = Q K^T the keys are the N operand (K-major), and one product should cover all 64
// keys of the tile, which needs one stride from 8 keys to the next across pages: a warp
// rewrites the tile as [piece][64 keys][16 bytes] (products of one page each are four times
// as many).  Q is written to shared memory by the CTA itself in the same core-matrix form.
//
// A query row's result depends on its own position only (tiles are anchored at key 0, rows do
// not interact).  Requests with fewer than `min_query_len` tokens are left to
// hx_paged_attention.  Every wait is bounded; a wait that runs out sets a status bit, and
// the CTA frees its tensor memory and returns.
#include "hx_tcgen05.cuh"

namespace {

constexpr int BLOCK_M = 128;   // query rows per lane (the MMA's M)
constexpr int LANES = 2;       // lanes per CTA: 256 query rows
constexpr int BLOCK_N = 64;    // keys per tile
constexpr int K_STAGES = 2;    // key tiles in shared memory as they land (rewritten at once)
constexpr int V_STAGES = 4;    // value tiles in shared memory (held until both products are done)
constexpr int KEY_BUFFERS = 3; // rewritten key tiles in shared memory
constexpr int S_BUFFERS = 2;   // score tiles in tensor memory per lane
constexpr int THREADS = 512;
constexpr int WARP_KEYS = 0, WARP_VALUES = 1, WARP_REWRITE = 2, WARP_SCORES = 3, WARP_OUTPUT = 5,
              WARP_SOFTMAX = 8;
constexpr int GROUP_STRIDE = 128;             // bytes from one 8-row core matrix to the next row group
constexpr int CHUNK_STRIDE = BLOCK_M * 16;    // bytes from one 16-byte column of Q to the next
constexpr float RAISE_MAXIMUM_BY = 8.0f;      // log2 units a tile must exceed a row's reference by

struct TcPrefillArgs {
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

template <int D>
struct TcConfig {
  static constexpr int kQBytes = BLOCK_M * D * 2;              // per lane
  static constexpr int kHalfBytes = BLOCK_N * D * 2;          // keys (or values) of a tile
  static constexpr int kSmemBytes =
      LANES * kQBytes + (K_STAGES + V_STAGES + KEY_BUFFERS) * kHalfBytes + 1024 + 512;
  static constexpr int kScoreColumns = BLOCK_N;               // per score buffer
  static constexpr int kLowTermColumn = BLOCK_N / 2;          // P: hi in columns [0, 32), lo after
  static constexpr int kOutputColumn = LANES * S_BUFFERS * BLOCK_N;   // lane 0's O; lane 1's follows
  static constexpr int kTmemColumns = 512;
  static_assert(LANES * (S_BUFFERS * BLOCK_N + D) <= 512, "tensor memory has 512 columns");
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <int D>
__global__ __launch_bounds__(THREADS, 1) void prefill_attention_tc_kernel(TcPrefillArgs a) {
  using Config = TcConfig<D>;
  constexpr int kDSteps = D / 16;      // k-steps of Q K^T
  hx_pdl_trigger();

  // which request and which 256-row tile of it is this CTA?  The last rows of a request see
  // the most keys: their CTAs are started first (the grid is walked heads first, then tiles),
  // so the short ones fill the gaps at the end.
  int tile_in_request = 0, tiles_of_request = 0;
  const int request = hx_find_query_tile(a.request_start, a.requests, a.min_query_len,
                                         LANES * BLOCK_M, blockIdx.y, tile_in_request,
                                         tiles_of_request);
  tile_in_request = tiles_of_request - 1 - tile_in_request;
  if (request < 0) return;      // before any barrier or allocation: the whole CTA leaves

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_tile = smem;
  uint8_t* k_stages = q_tile + LANES * Config::kQBytes;
  uint8_t* v_stages = k_stages + K_STAGES * Config::kHalfBytes;
  uint8_t* keys_by_piece = v_stages + V_STAGES * Config::kHalfBytes;      // [KEY_BUFFERS]
  uint64_t* k_full = reinterpret_cast<uint64_t*>(keys_by_piece + KEY_BUFFERS * Config::kHalfBytes);
  uint64_t* k_empty = k_full + K_STAGES;
  uint64_t* v_full = k_empty + K_STAGES;
  uint64_t* v_empty = v_full + V_STAGES;              // [LANES][V_STAGES]: a lane's product has read it
  uint64_t* s_full = v_empty + LANES * V_STAGES;      // [LANES][S_BUFFERS] scores of tile t in buffer t % 2
  uint64_t* p_full = s_full + LANES * S_BUFFERS;      // [LANES][S_BUFFERS] its probabilities are in place
  uint64_t* o_full = p_full + LANES * S_BUFFERS;      // [LANES][S_BUFFERS] its output product is done
  uint64_t* k_ready = o_full + LANES * S_BUFFERS;     // [KEY_BUFFERS] the tile's keys are rewritten
  uint64_t* k_done = k_ready + KEY_BUFFERS;           // [LANES][KEY_BUFFERS] a lane's scores have read them
  uint64_t* q_ready = k_done + LANES * KEY_BUFFERS;   // the query tiles are in shared memory
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(q_ready + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x;
  const int kv_head = head / (a.heads / a.kv_heads);
  const int q_begin = a.request_start[request];
  const int q_len = a.request_start[request + 1] - q_begin;
  const int context = a.request_context[request];
  const int row0 = tile_in_request * LANES * BLOCK_M;         // first query row of the CTA
  const int rows_here = min(LANES * BLOCK_M, q_len - row0);
  const int last_key = context + row0 + rows_here - 1;        // last key any row here sees
  const int n_tiles = last_key / BLOCK_N + 1;                 // key tiles somebody here sees
  // lane l has rows [row0 + 128 l, ...) and sees the tiles before lane_tiles(l); lane 1 may be empty
  auto lane_rows = [&](int l) { return max(0, min(BLOCK_M, rows_here - l * BLOCK_M)); };
  auto lane_tiles = [&](int l) {
    const int rows = lane_rows(l);
    return rows > 0 ? (context + row0 + l * BLOCK_M + rows - 1) / BLOCK_N + 1 : 0;
  };
  const int page_size = a.page_size;
  const int pages_per_tile = BLOCK_N / page_size;
  const uint32_t page_bytes = static_cast<uint32_t>(page_size) * D * 2;
  const uint32_t piece_stride = static_cast<uint32_t>(page_size) * 16;   // next 16-byte piece of a key

  if (threadIdx.x == 0) {
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) mbar_init(&v_full[s], 1);
    for (int s = 0; s < LANES * V_STAGES; ++s) mbar_init(&v_empty[s], 1);
    for (int b = 0; b < LANES * S_BUFFERS; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4);   // one arrival per softmax warp of the lane
      mbar_init(&o_full[b], 1);
    }
    for (int b = 0; b < KEY_BUFFERS; ++b) mbar_init(&k_ready[b], 1);
    for (int b = 0; b < LANES * KEY_BUFFERS; ++b) mbar_init(&k_done[b], 1);
    mbar_init(q_ready, THREADS / 32 - WARP_SCORES);      // one arrival per warp that loads queries
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == WARP_SCORES) tmem_alloc(tmem_holder, Config::kTmemColumns);
  hx_pdl_wait();

  tc_fence_before();
  __syncthreads();      // barriers and tensor memory are there; nothing else is waited for here
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // ---- the query tiles: per lane [D / 8 pieces][16 row groups][8 rows][16 bytes], written by
  // the warps from WARP_SCORES on while the first pages are on their way.  All of a thread's
  // loads are in flight together (one after the other they cost the CTA 6 us).
  if (warp >= WARP_SCORES) {
    constexpr int kLoaders = THREADS - WARP_SCORES * 32;
    constexpr int kPieces = LANES * BLOCK_M * (D / 8);
    constexpr int kPerThread = (kPieces + kLoaders - 1) / kLoaders;
    const int loader = threadIdx.x - WARP_SCORES * 32;
    uint4 values[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int index = loader + i * kLoaders;
      const int row = index / (D / 8);      // among the CTA's 256
      const int piece = index - row * (D / 8);
      values[i] = make_uint4(0u, 0u, 0u, 0u);
      if (index < kPieces && row < rows_here)
        values[i] = *reinterpret_cast<const uint4*>(
            a.q + static_cast<size_t>(q_begin + row0 + row) * a.ldq + static_cast<size_t>(head) * D +
            piece * 8);
    }
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int index = loader + i * kLoaders;
      const int row = index / (D / 8);
      const int piece = index - row * (D / 8);
      const int in_lane = row & (BLOCK_M - 1);
      if (index < kPieces)
        *reinterpret_cast<uint4*>(q_tile + (row / BLOCK_M) * Config::kQBytes + piece * CHUNK_STRIDE +
                                  (in_lane >> 3) * GROUP_STRIDE + (in_lane & 7) * 16) = values[i];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(q_ready);
  }

  if (warp == WARP_KEYS || warp == WARP_VALUES) {
    // ------------------------------------------------------------ page requests
    // Each as far ahead as its own ring allows: the keys of a tile are wanted well before
    // its values (they are rewritten, then multiplied, then the softmax runs), and one ring
    // must not hold up the other.
    if (lane == 0) {
      const bool values = warp == WARP_VALUES;
      const int stages = values ? V_STAGES : K_STAGES;
      uint64_t* full = values ? v_full : k_full;
      uint8_t* ring = values ? v_stages : k_stages;
      const uint8_t* cache = reinterpret_cast<const uint8_t*>(values ? a.v_cache : a.k_cache);
      const int* table = a.block_tables +
                         static_cast<size_t>(a.request_table_row[request]) * a.table_stride;
      const int last_page = last_key / page_size;
      auto pages_of = [&](int tile, int (&pages)[4]) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int index = tile * pages_per_tile + p;
          pages[p] = (p < pages_per_tile && index <= last_page) ? table[index] : -2;   // -2: none
        }
      };
      int pages[4], next_pages[4];
      pages_of(0, pages);
      for (int tile = 0; tile < n_tiles && !*failed; ++tile) {
        if (tile + 1 < n_tiles) pages_of(tile + 1, next_pages);      // in flight during the wait
        const int stage = tile % stages;
        bool free = true;
        if (!values) {
          free = mbar_wait(&k_empty[stage], (static_cast<uint32_t>(tile / stages) & 1u) ^ 1u);
        } else if (tile >= V_STAGES) {
          // the stage held tile - V_STAGES: every lane that saw that tile has multiplied by it
          const int before = tile - V_STAGES;
          for (int l = 0; l < LANES && free; ++l)
            if (before < lane_tiles(l))
              free = mbar_wait(&v_empty[l * V_STAGES + stage],
                               static_cast<uint32_t>(before / V_STAGES) & 1u);
        }
        if (!free) {
          atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
          break;
        }
        uint32_t expected = 0;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          if (pages[p] >= a.num_pages || pages[p] == -1) {
            atomicOr(a.status, HX_FLAG_BAD_PAGE);
            pages[p] = -2;
          }
          if (pages[p] >= 0) expected += page_bytes;
        }
        mbar_expect_tx(&full[stage], expected);
        const uint32_t base = smem_u32(ring + stage * Config::kHalfBytes);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          if (pages[p] >= 0) {
            const size_t block = (static_cast<size_t>(pages[p]) * a.kv_heads + kv_head) * page_bytes;
            bulk_copy(base + p * page_bytes, cache + block, page_bytes, &full[stage]);
          }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) pages[p] = next_pages[p];
      }
    }
  } else if (warp == WARP_REWRITE) {
    // ------------------------------------------------------ keys, piece by piece
    // The score product wants all 64 keys of the tile at one stride, but every page block
    // holds its own keys piece-major: this warp rewrites a landed tile as
    // [piece][64 keys][16 bytes] into buffer tile % KEY_BUFFERS.
    bool ok = true;
    // where keys `lane` and `lane + 32` of a tile sit inside the landed page blocks
    const uint32_t source_low = (lane / page_size) * page_bytes + (lane % page_size) * 16;
    const uint32_t source_high =
        ((lane + 32) / page_size) * page_bytes + ((lane + 32) % page_size) * 16;
    for (int tile = 0; tile < n_tiles && ok && !*failed; ++tile) {
      if (lane == 0) {
        ok = mbar_wait(&k_full[tile % K_STAGES], static_cast<uint32_t>(tile / K_STAGES) & 1u);
        // the score products that read this buffer KEY_BUFFERS tiles ago are done (one per
        // lane that saw that tile; a barrier of its own per lane and buffer, whose next phase
        // needs this very rewrite, so that no phase can be mistaken for another)
        if (tile >= KEY_BUFFERS) {
          const int before = tile - KEY_BUFFERS;
          for (int l = 0; l < LANES && ok; ++l)
            if (before < lane_tiles(l))
              ok = mbar_wait(&k_done[l * KEY_BUFFERS + tile % KEY_BUFFERS],
                             static_cast<uint32_t>(before / KEY_BUFFERS) & 1u);
        }
        if (!ok) {
          atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const uint32_t source = smem_u32(k_stages + (tile % K_STAGES) * Config::kHalfBytes);
      const uint32_t target =
          smem_u32(keys_by_piece + (tile % KEY_BUFFERS) * Config::kHalfBytes) + lane * 16;
      // eight pieces at a time: all their loads are in flight before the first store
#pragma unroll
      for (int piece0 = 0; piece0 < D / 8; piece0 += 8) {
        uint4 low[8], high[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (piece0 + i >= D / 8) continue;      // (a head of 112: fourteen pieces)
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(low[i].x), "=r"(low[i].y), "=r"(low[i].z), "=r"(low[i].w)
                       : "r"(source + source_low + (piece0 + i) * piece_stride));
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(high[i].x), "=r"(high[i].y), "=r"(high[i].z), "=r"(high[i].w)
                       : "r"(source + source_high + (piece0 + i) * piece_stride));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (piece0 + i >= D / 8) continue;
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(
                           target + (piece0 + i) * (BLOCK_N * 16)),
                       "r"(low[i].x), "r"(low[i].y), "r"(low[i].z), "r"(low[i].w) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(
                           target + (piece0 + i) * (BLOCK_N * 16) + 512),
                       "r"(high[i].x), "r"(high[i].y), "r"(high[i].z), "r"(high[i].w) : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&k_ready[tile % KEY_BUFFERS]);
        mbar_arrive(&k_empty[tile % K_STAGES]);      // the landed copy may be overwritten
      }
    }
  } else if (warp == WARP_SCORES || warp == WARP_SCORES + 1) {
    // ------------------------------------------------------------ score products
    if (lane == 0) {
      constexpr uint32_t idesc_scores = make_idesc(BLOCK_M, BLOCK_N);
      // Descriptors differ from product to product only in their start address (the low 14
      // bits, in units of 16 bytes): build one of each kind and add offsets.
      const uint64_t desc_q0 = make_smem_desc_plain(smem_u32(q_tile), CHUNK_STRIDE, GROUP_STRIDE);
      const uint64_t desc_k0 =
          make_smem_desc_plain(smem_u32(keys_by_piece), BLOCK_N * 16, GROUP_STRIDE);
      constexpr uint32_t kKeyBufferStep = Config::kHalfBytes >> 4;
      constexpr uint32_t kChunkPairStep = (2 * CHUNK_STRIDE) >> 4;      // 16 coordinates of Q on
      constexpr uint32_t kKeyPiecePairStep = (2 * BLOCK_N * 16) >> 4;   // 16 coordinates of the keys on
      // S_l[tile % 2] = Q_l K_tile^T: one product of 64 keys per 16 coordinates.  The buffer
      // held the probabilities of tile - 2, which the lane's output product must have read.
      const int l = warp - WARP_SCORES;
      const int my_tiles = lane_tiles(l);
      const uint64_t desc_q = desc_q0 + l * (Config::kQBytes >> 4);
      if (!mbar_wait(q_ready, 0)) {
        atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
        *failed = 1;
      }
      for (int tile = 0; tile < my_tiles && !*failed; ++tile) {
        const int b = l * S_BUFFERS + tile % S_BUFFERS;
        if (!mbar_wait(&k_ready[tile % KEY_BUFFERS], static_cast<uint32_t>(tile / KEY_BUFFERS) & 1u) ||
            (tile >= S_BUFFERS &&
             !mbar_wait(&o_full[b], static_cast<uint32_t>((tile - S_BUFFERS) / S_BUFFERS) & 1u))) {
          atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
          break;
        }
        tc_fence_after();
        const uint64_t desc_k = desc_k0 + (tile % KEY_BUFFERS) * kKeyBufferStep;
        const uint32_t target = tmem_base + b * Config::kScoreColumns;
#pragma unroll
        for (int k = 0; k < kDSteps; ++k)
          umma_bf16(target, desc_q + k * kChunkPairStep, desc_k + k * kKeyPiecePairStep,
                    idesc_scores, k > 0 ? 1u : 0u);
        umma_commit(&s_full[b]);
        umma_commit(&k_done[l * KEY_BUFFERS + tile % KEY_BUFFERS]);
      }
    }
  } else if (warp == WARP_OUTPUT || warp == WARP_OUTPUT + 1) {
    // ----------------------------------------------------------- output products
    if (lane == 0) {
      const int l = warp - WARP_OUTPUT;
      const int my_tiles = lane_tiles(l);
      constexpr uint32_t idesc_output = make_idesc_b_mn_major(BLOCK_M, D);
      // values: MN-major, the next 8 keys are 128 bytes on, the next 8 coordinates one piece on
      const uint64_t desc_v0 = make_smem_desc_plain(smem_u32(v_stages), GROUP_STRIDE, piece_stride);
      constexpr uint32_t kStageStep = Config::kHalfBytes >> 4;
      // where the 16 keys of each product of P V start inside a stage's value half
      uint32_t value_step[BLOCK_N / 16];
#pragma unroll
      for (int g = 0; g < BLOCK_N / 16; ++g) {
        const int key = g * 16;
        value_step[g] = ((key / page_size) * page_bytes + (key % page_size) * 16) >> 4;
      }
      const uint32_t target = tmem_base + Config::kOutputColumn + l * D;
      for (int tile = 0; tile < my_tiles && !*failed; ++tile) {
        // the probabilities of this tile lie where its scores were
        const int s = tile % V_STAGES;
        const int b = l * S_BUFFERS + tile % S_BUFFERS;
        if (!mbar_wait(&p_full[b], static_cast<uint32_t>(tile / S_BUFFERS) & 1u) ||
            !mbar_wait(&v_full[s], static_cast<uint32_t>(tile / V_STAGES) & 1u)) {
          atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
          *failed = 1;
          break;
        }
        tc_fence_after();
        const uint64_t desc_v = desc_v0 + s * kStageStep;
        const uint32_t p_hi = tmem_base + b * Config::kScoreColumns;
        const uint32_t p_lo = p_hi + Config::kLowTermColumn;
        // O_l += P V_tile: 16 keys (8 columns of P) per product, the hi and the lo term of P
#pragma unroll
        for (int g = 0; g < BLOCK_N / 16; ++g) {
          umma_bf16_a_tmem(target, p_hi + g * 8, desc_v + value_step[g], idesc_output,
                           (tile > 0 || g > 0) ? 1u : 0u);
          umma_bf16_a_tmem(target, p_lo + g * 8, desc_v + value_step[g], idesc_output, 1u);
        }
        umma_commit(&v_empty[l * V_STAGES + s]);     // this lane is done with the stage
        umma_commit(&o_full[b]);                     // O holds this tile; its P has been read
      }
    }
  } else if (warp >= WARP_SOFTMAX) {
    // ------------------------------------------------------------------ softmax
    const int l = (warp - WARP_SOFTMAX) >> 2;      // the lane this group serves
    const int my_tiles = lane_tiles(l);
    const int my_rows = lane_rows(l);
    const int quarter = warp & 3;      // tensor-memory lanes [32 * quarter, 32 * quarter + 32)
    const int row = quarter * 32 + lane;
    const int group_thread = threadIdx.x - (WARP_SOFTMAX + 4 * l) * 32;      // 0..127
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t output_base = lane_base + Config::kOutputColumn + l * D;
    const int q_position = context + row0 + l * BLOCK_M + row;      // the last key this row sees
    float row_max = -INFINITY;      // the reference of this row's exponentials, in log2 units
    float row_sum = 0.0f;
    const float scale_log2 = a.scale * 1.4426950408889634f;
    bool ok = true;

    // One lane waits and looks at the failure flag, all lanes get the same answer (what
    // follows a wait is warp-wide: tensor-memory loads and stores need the warp together).
    auto wait_for = [&](uint64_t* bar, uint32_t parity_bit) {
      int state = 0;      // 0: go on, 1: this wait ran out, 2: somebody else failed
      if (lane == 0) state = *failed ? 2 : (mbar_wait(bar, parity_bit) ? 0 : 1);
      state = __shfl_sync(0xffffffffu, state, 0);
      if (state == 1 && lane == 0) {
        atomicOr(a.status, HX_FLAG_WAIT_TIMEOUT);
        *failed = 1;
      }
      return state == 0;
    };

    for (int tile = 0; tile < my_tiles && ok; ++tile) {
      const int b = l * S_BUFFERS + tile % S_BUFFERS;
      ok = wait_for(&s_full[b], static_cast<uint32_t>(tile / S_BUFFERS) & 1u);
      if (!ok) break;
      tc_fence_after();
      const uint32_t score_base = lane_base + b * Config::kScoreColumns;
      // ---- this row's scores of the tile, in units of log2(e) so that exp is one ex2
      float p[BLOCK_N];
      {
        uint32_t r[4][16];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_load16_issue(score_base + c * 16, r[c]);
        tmem_load_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) p[c * 16 + i] = __uint_as_float(r[c][i]) * scale_log2;
      }
      const int key0 = tile * BLOCK_N;
      if (key0 + BLOCK_N - 1 > q_position) {
#pragma unroll
        for (int i = 0; i < BLOCK_N; ++i)
          if (key0 + i > q_position) p[i] = -INFINITY;
      }
      float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 4)
#pragma unroll
        for (int u = 0; u < 4; ++u) part_max[u] = fmaxf(part_max[u], p[i + u]);
      const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
      // key 0 is visible to every row, so the reference is finite from the first tile on
      if (tile == 0) {
        row_max = tile_max;
      } else if (__any_sync(0xffffffffu, tile_max > row_max + RAISE_MAXIMUM_BY)) {
        // ---- a new reference: what O and the sum hold was taken against the old one.  The
        // product of the previous tile must have landed; the product of this tile waits for
        // this warp's arrival below.  (o_full[b] completes a phase for every other tile; its
        // previous phase was complete before the scores of this tile were started.)
        const float new_max = fmaxf(row_max, tile_max);
        const float correction = fast_exp2(row_max - new_max);
        row_max = new_max;
        row_sum *= correction;
        ok = wait_for(&o_full[l * S_BUFFERS + (tile - 1) % S_BUFFERS],
                      static_cast<uint32_t>((tile - 1) / S_BUFFERS) & 1u);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int d0 = 0; d0 < D; d0 += 32) {
          const bool both = d0 + 16 < D;      // (compile time: D is a multiple of 16)
          uint32_t r0[16], r1[16];
          tmem_load16_issue(output_base + d0, r0);
          if (both) tmem_load16_issue(output_base + d0 + 16, r1);
          tmem_load_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            r0[i] = __float_as_uint(__uint_as_float(r0[i]) * correction);
            if (both) r1[i] = __float_as_uint(__uint_as_float(r1[i]) * correction);
          }
          tmem_store16_raw(output_base + d0, r0);
          if (both) tmem_store16_raw(output_base + d0 + 16, r1);
        }
      }
      float part_sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 4)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          p[i + u] = fast_exp2(p[i + u] - row_max);
          part_sum[u] += p[i + u];
        }
      row_sum += (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);

      // ---- P = hi + lo over the scores just read: hi is p cut to its upper 16 bits (a
      // bfloat16 exactly), lo is p - hi (exact in float32) cut the same way: together 16
      // bits of p.  Two keys per column, the earlier key in the lower half.
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = p[c * 32 + 2 * i], p1 = p[c * 32 + 2 * i + 1];
          const uint32_t x0 = __float_as_uint(p0), x1 = __float_as_uint(p1);
          const float rest0 = p0 - __uint_as_float(x0 & 0xffff0000u);
          const float rest1 = p1 - __uint_as_float(x1 & 0xffff0000u);
          hi[i] = __byte_perm(x0, x1, 0x7632);
          lo[i] = __byte_perm(__float_as_uint(rest0), __float_as_uint(rest1), 0x7632);
        }
        tmem_store16_raw(score_base + c * 16, hi);
        tmem_store16_raw(score_base + Config::kLowTermColumn + c * 16, lo);
      }
      tmem_store_wait();

      // ---- value rows behind the last key hold whatever the pages (or an earlier tile)
      // left there; a NaN would survive a zero probability, so they are cleared (by the group
      // that is first to need the tile: the other waits for its own arrival barrier only, but
      // the tile with the last key is seen by the last lane alone, or by lane 0 alone)
      const int first_stale = last_key + 1 - key0;
      if (first_stale < BLOCK_N) {
        ok = wait_for(&v_full[tile % V_STAGES], static_cast<uint32_t>(tile / V_STAGES) & 1u);
        if (!ok) break;
        uint8_t* v_half = v_stages + (tile % V_STAGES) * Config::kHalfBytes;
        for (int index = group_thread; index < BLOCK_N * (D / 8); index += 128) {
          const int key = index / (D / 8);
          const int piece = index - key * (D / 8);
          if (key >= first_stale)
            *reinterpret_cast<uint4*>(v_half + (key / page_size) * page_bytes +
                                      (piece * page_size + key % page_size) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }

    // ---- a commit covers every product its thread issued before it: the lane's last tile
    // says all of them are done
    if (ok && my_tiles > 0) {
      ok = wait_for(&o_full[l * S_BUFFERS + (my_tiles - 1) % S_BUFFERS],
                    static_cast<uint32_t>((my_tiles - 1) / S_BUFFERS) & 1u);
      if (ok) {
        tc_fence_after();
        const float inverse = 1.0f / row_sum;
        __nv_bfloat16* out = a.out +
                             static_cast<size_t>(q_begin + row0 + l * BLOCK_M + row) * a.ldo +
                             static_cast<size_t>(head) * D;
#pragma unroll
        for (int d0 = 0; d0 < D; d0 += 32) {
          const bool both = d0 + 16 < D;
          uint32_t r[2][16];
          tmem_load16_issue(output_base + d0, r[0]);
          if (both) tmem_load16_issue(output_base + d0 + 16, r[1]);
          tmem_load_wait();
          if (row < my_rows) {
#pragma unroll
            for (int h = 0; h < (both ? 2 : 1); ++h)
#pragma unroll
              for (int d = 0; d < 16; d += 8) {
                uint4 packed;
                __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  pairs[i] = __floats2bfloat162_rn(__uint_as_float(r[h][d + 2 * i]) * inverse,
                                                   __uint_as_float(r[h][d + 2 * i + 1]) * inverse);
                *reinterpret_cast<uint4*>(out + d0 + h * 16 + d) = packed;
              }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == WARP_SCORES) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Config::kTmemColumns);
  }
}

template <int D>
int launch(const TcPrefillArgs& a, int tiles, cudaStream_t stream) {
  using Config = TcConfig<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attention_tc_kernel<D>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Config::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      hx_set_error("hx_prefill_attention_tc: cannot reserve %d bytes of shared memory",
                   Config::kSmemBytes);
      return HX_ERR_LAUNCH;
    }
    configured = true;
  }
  hx_launch(prefill_attention_tc_kernel<D>, dim3(a.heads, tiles), THREADS, Config::kSmemBytes,
            stream, a);
  return HX_OK;
}

}  // namespace

// 1 when the tcgen05 kernel takes this head size and page size: a page is the N operand of a
// product, so it has at least 16 keys.
HX_API int hx_prefill_attention_tc_supports(int head_dim, int page_size) {
  return head_dim >= 64 && head_dim <= 128 && head_dim % 16 == 0 &&
         (page_size == 16 || page_size == 32 || page_size == 64);
}

// The arguments of hx_prefill_attention; tile_bound bounds the number of 256-token query tiles
// (a larger bound only launches CTAs that leave at once).
HX_API int hx_prefill_attention_tc(const void* q, int ldq, const void* k_cache,
                                   const void* v_cache, const int* request_start,
                                   const int* request_context, const int* request_table_row,
                                   const int* block_tables, int table_stride, void* out, int ldo,
                                   int requests, int tile_bound, int heads, int kv_heads,
                                   int head_dim, int page_size, int num_pages, float scale,
                                   int min_query_len, int* status, cudaStream_t stream) {
  HX_REQUIRE(hx_prefill_attention_tc_supports(head_dim, page_size),
             "hx_prefill_attention_tc: head_dim %d with pages of %d is not supported (head sizes "
             "64 to 128 in steps of 16, pages of 16, 32 or 64)", head_dim, page_size);
  HX_REQUIRE(requests >= 0 && tile_bound >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
             "hx_prefill_attention_tc: bad sizes");
  HX_REQUIRE(tile_bound <= 65535, "hx_prefill_attention_tc: too many query tiles");
  HX_REQUIRE(num_pages > 0 && table_stride > 0, "hx_prefill_attention_tc: bad cache geometry");
  HX_REQUIRE(status != nullptr, "hx_prefill_attention_tc: status word missing");
  HX_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "hx_prefill_attention_tc: operands must be 16-byte aligned, row strides multiples of 8");
  if (requests == 0 || tile_bound == 0) return HX_OK;
  TcPrefillArgs a{static_cast<const __nv_bfloat16*>(q), ldq,
                  static_cast<const __nv_bfloat16*>(k_cache),
                  static_cast<const __nv_bfloat16*>(v_cache), request_start, request_context,
                  request_table_row, block_tables, table_stride, static_cast<__nv_bfloat16*>(out),
                  ldo, requests, heads, kv_heads, page_size, num_pages, scale, min_query_len, status};
  int rc;
  switch (head_dim) {
    case 64: rc = launch<64>(a, tile_bound, stream); break;
    case 80: rc = launch<80>(a, tile_bound, stream); break;
    case 96: rc = launch<96>(a, tile_bound, stream); break;
    case 112: rc = launch<112>(a, tile_bound, stream); break;
    default: rc = launch<128>(a, tile_bound, stream); break;
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_prefill_attention_tc");
  return HX_OK;
}
