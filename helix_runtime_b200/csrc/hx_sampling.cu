// Token selection on the device: greedy and temperature sampling.
//
// Greedy follows the reference's rule (src/model/cpu_generation.cpp:82-97): the
// lowest id among the maxima wins and a non-finite logit is an error (here: token
// -1 and a status bit, so one bad request does not stop the step).  The reference
// has no other sampler; temperature sampling is this engine's own: probabilities
// softmax(logits / T) in float32, then the inverse of the cumulative distribution
// at a uniform number the caller supplies per row, so the draw depends only on the
// request's own random stream, never on the rest of the batch.
#include "hx_common.cuh"

namespace {

constexpr int THREADS = 256;

__global__ __launch_bounds__(THREADS) void argmax_kernel(const float* __restrict__ logits, int ld,
                                                         int vocab, int* __restrict__ tokens,
                                                         int* status) {
  __shared__ float best_value[THREADS];
  __shared__ int best_index[THREADS];
  __shared__ int bad;
  hx_pdl_prologue();
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  float value = -INFINITY;
  int index = 0x7fffffff;
  bool nonfinite = false;
  auto take = [&](float v, int c) {
    nonfinite |= !isfinite(v);
    if (v > value) {  // strict: within a thread ids ascend, so the lowest id stays
      value = v;
      index = c;
    }
  };
  int done = 0;
  if (ld % 4 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // four logits a load, several loads in flight: the row is 128 KB that nobody has read yet
    const float4* wide = reinterpret_cast<const float4*>(row);
#pragma unroll 4
    for (int q = threadIdx.x; q < vocab / 4; q += THREADS) {
      const float4 v = wide[q];
      take(v.x, 4 * q);
      take(v.y, 4 * q + 1);
      take(v.z, 4 * q + 2);
      take(v.w, 4 * q + 3);
    }
    done = vocab / 4 * 4;
  }
  for (int c = done + threadIdx.x; c < vocab; c += THREADS) take(row[c], c);
  if (nonfinite) bad = 1;
  best_value[threadIdx.x] = value;
  best_index[threadIdx.x] = index;
  __syncthreads();
  for (int stride = THREADS / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) {
      const float other = best_value[threadIdx.x + stride];
      const int other_index = best_index[threadIdx.x + stride];
      if (other > best_value[threadIdx.x] ||
          (other == best_value[threadIdx.x] && other_index < best_index[threadIdx.x])) {
        best_value[threadIdx.x] = other;
        best_index[threadIdx.x] = other_index;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (bad) {
      tokens[blockIdx.x] = -1;
      if (status != nullptr) atomicOr(status, HX_FLAG_NONFINITE);
    } else {
      tokens[blockIdx.x] = best_index[0];
    }
  }
}

// One block per row.  temperature[row] <= 0 selects greedily.  Each thread owns one
// contiguous segment of the vocabulary, so the cumulative sum has a fixed order.
__global__ __launch_bounds__(THREADS) void sample_kernel(const float* __restrict__ logits, int ld,
                                                         int vocab,
                                                         const float* __restrict__ temperature,
                                                         const float* __restrict__ uniform,
                                                         int* __restrict__ tokens, int* status) {
  __shared__ float scratch[32];
  __shared__ float segment_sum[THREADS];
  __shared__ float best_value[THREADS];
  __shared__ int best_index[THREADS];
  __shared__ int bad;
  __shared__ int chosen;
  hx_pdl_prologue();
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  const float temp = temperature[blockIdx.x];
  if (threadIdx.x == 0) {
    bad = 0;
    chosen = -1;
  }
  __syncthreads();

  const int per_thread = (vocab + THREADS - 1) / THREADS;
  const int begin = min(threadIdx.x * per_thread, vocab);
  const int end = min(begin + per_thread, vocab);

  float value = -INFINITY;
  int index = 0x7fffffff;
  bool nonfinite = false;
  for (int c = begin; c < end; ++c) {
    const float v = row[c];
    nonfinite |= !isfinite(v);
    if (v > value) {
      value = v;
      index = c;
    }
  }
  if (nonfinite) bad = 1;
  best_value[threadIdx.x] = value;
  best_index[threadIdx.x] = index;
  __syncthreads();
  for (int stride = THREADS / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) {
      const float other = best_value[threadIdx.x + stride];
      const int other_index = best_index[threadIdx.x + stride];
      if (other > best_value[threadIdx.x] ||
          (other == best_value[threadIdx.x] && other_index < best_index[threadIdx.x])) {
        best_value[threadIdx.x] = other;
        best_index[threadIdx.x] = other_index;
      }
    }
    __syncthreads();
  }
  if (bad) {
    if (threadIdx.x == 0) {
      tokens[blockIdx.x] = -1;
      if (status != nullptr) atomicOr(status, HX_FLAG_NONFINITE);
    }
    return;
  }
  const float maximum = best_value[0];
  if (!(temp > 0.0f)) {
    if (threadIdx.x == 0) tokens[blockIdx.x] = best_index[0];
    return;
  }

  const float inverse_temp = 1.0f / temp;
  float local = 0.0f;
  for (int c = begin; c < end; ++c) local += expf((row[c] - maximum) * inverse_temp);
  segment_sum[threadIdx.x] = local;
  __syncthreads();
  // exclusive prefix over the segments, in order, by one thread: 256 adds
  if (threadIdx.x == 0) {
    float running = 0.0f;
    for (int t = 0; t < THREADS; ++t) {
      const float s = segment_sum[t];
      segment_sum[t] = running;
      running += s;
    }
    scratch[0] = running;
  }
  __syncthreads();
  const float total = scratch[0];
  const float target = uniform[blockIdx.x] * total;
  const float my_start = segment_sum[threadIdx.x];
  const float my_end = threadIdx.x + 1 < THREADS ? segment_sum[threadIdx.x + 1] : total;
  if (begin < end && target >= my_start && target < my_end) {
    float running = my_start;
    int pick = end - 1;
    for (int c = begin; c < end; ++c) {
      running += expf((row[c] - maximum) * inverse_temp);
      if (target < running) {
        pick = c;
        break;
      }
    }
    chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // target == total can only happen through rounding: fall back to the last token with
    // non-zero probability, which is the last id of the vocabulary at worst
    tokens[blockIdx.x] = chosen >= 0 ? chosen : vocab - 1;
  }
}

}  // namespace

HX_API int hx_argmax(const float* logits, int ld, int rows, int vocab, int* tokens, int* status,
                     cudaStream_t stream) {
  HX_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "hx_argmax: bad sizes");
  if (rows == 0) return HX_OK;
  hx_launch(argmax_kernel, rows, THREADS, 0, stream, logits, ld, vocab, tokens, status);
  HX_CHECK_LAUNCH("hx_argmax");
  return HX_OK;
}

HX_API int hx_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                     const float* uniform, int* tokens, int* status, cudaStream_t stream) {
  HX_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "hx_sample: bad sizes");
  HX_REQUIRE(temperature != nullptr && uniform != nullptr, "hx_sample: missing arguments");
  if (rows == 0) return HX_OK;
  hx_launch(sample_kernel, rows, THREADS, 0, stream, logits, ld, vocab, temperature, uniform, tokens, status);
  HX_CHECK_LAUNCH("hx_sample");
  return HX_OK;
}
