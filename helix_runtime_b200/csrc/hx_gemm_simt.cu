// Plain tiled matrix product on the CUDA cores: out[t, o] (+)= sum_k x[t, k] * w[o, k].
//
// This is the true 32-bit path (float32 storage, float32 fused multiply-adds, no
// reduced-precision matrix mode) and also the bfloat16 path for shapes the tensor
// core kernel refuses.  Each output element is one sequential sum over k in
// ascending order, so its value never depends on how many rows the call has or on
// which tile it falls into.  The reference's counterpart is its 16x16 tiled kernel
// (src/kernels/cuda/matmul.cu:36-71); this one keeps a 64x64 tile with 4x4 outputs
// per thread.
#include "hx_common.cuh"

namespace {

constexpr int BM = 64;   // tokens per tile
constexpr int BN = 64;   // output features per tile
constexpr int BK = 16;

enum Epilogue : int { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2 };

template <typename T, int EPI>
__global__ __launch_bounds__(256) void gemm_simt_kernel(const T* __restrict__ x, int ldx,
                                                        const T* __restrict__ w, int ldw,
                                                        void* __restrict__ out, int ldo, int tokens,
                                                        int features, int depth) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  hx_pdl_prologue();
  const int tile_t = blockIdx.y * BM;
  const int tile_f = blockIdx.x * BN;
  const int tx = threadIdx.x & 15;   // feature group
  const int ty = threadIdx.x >> 4;   // token group
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // each thread loads 4 elements of each operand tile per step: row = id / 4, 4 k's
  const int load_row = threadIdx.x >> 2;        // 0..63
  const int load_k = (threadIdx.x & 3) * 4;     // 0,4,8,12
  for (int k0 = 0; k0 < depth; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + load_k + i;
      const int t = tile_t + load_row;
      const int f = tile_f + load_row;
      xs[load_k + i][load_row] =
          (t < tokens && k < depth) ? hx_to_float<T>(x[static_cast<size_t>(t) * ldx + k]) : 0.0f;
      ws[load_k + i][load_row] =
          (f < features && k < depth) ? hx_to_float<T>(w[static_cast<size_t>(f) * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = tile_t + ty * 4 + i;
    if (t >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int f = tile_f + tx * 4 + j;
      if (f >= features) continue;
      const size_t index = static_cast<size_t>(t) * ldo + f;
      if (EPI == EPI_STORE) {
        static_cast<T*>(out)[index] = hx_from_float<T>(acc[i][j]);
      } else if (EPI == EPI_STORE_F32) {
        static_cast<float*>(out)[index] = acc[i][j];
      } else {
        static_cast<float*>(out)[index] += acc[i][j];
      }
    }
  }
}

template <typename T>
int launch(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int tokens,
           int features, int depth, int epilogue, cudaStream_t stream) {
  const dim3 grid((features + BN - 1) / BN, (tokens + BM - 1) / BM);
  const T* xp = static_cast<const T*>(x);
  const T* wp = static_cast<const T*>(w);
  switch (epilogue) {
    case EPI_STORE:
      hx_launch(gemm_simt_kernel<T, EPI_STORE>, grid, 256, 0, stream, xp, ldx, wp, ldw, out, ldo, tokens, features, depth);
      break;
    case EPI_STORE_F32:
      hx_launch(gemm_simt_kernel<T, EPI_STORE_F32>, grid, 256, 0, stream, xp, ldx, wp, ldw, out, ldo, tokens, features, depth);
      break;
    case EPI_ADD_F32:
      hx_launch(gemm_simt_kernel<T, EPI_ADD_F32>, grid, 256, 0, stream, xp, ldx, wp, ldw, out, ldo, tokens, features, depth);
      break;
    default:
      hx_set_error("hx_gemm_simt: unknown epilogue %d", epilogue);
      return HX_ERR_ARGUMENT;
  }
  return HX_OK;
}

}  // namespace

// epilogue 0: out (compute dtype) = x w^T; 1: out (float32) = x w^T; 2: out (float32) += x w^T
HX_API int hx_gemm_simt(const void* x, int ldx, const void* w, int ldw, void* out, int ldo,
                        int dtype, int tokens, int features, int depth, int epilogue,
                        cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && features > 0 && depth > 0, "hx_gemm_simt: bad sizes");
  HX_REQUIRE(ldx >= depth && ldw >= depth && ldo >= features, "hx_gemm_simt: bad strides");
  HX_REQUIRE((tokens + BM - 1) / BM <= 65535, "hx_gemm_simt: too many rows (%d)", tokens);
  if (tokens == 0) return HX_OK;
  int rc;
  if (dtype == HX_F32) {
    rc = launch<float>(x, ldx, w, ldw, out, ldo, tokens, features, depth, epilogue, stream);
  } else if (dtype == HX_BF16) {
    rc = launch<__nv_bfloat16>(x, ldx, w, ldw, out, ldo, tokens, features, depth, epilogue, stream);
  } else {
    HX_REQUIRE(false, "hx_gemm_simt: unknown dtype %d", dtype);
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_gemm_simt");
  return HX_OK;
}
