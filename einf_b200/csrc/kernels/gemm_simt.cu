// out[M, N] = A[M, K] . W[N, K]^T (+ bias[N]) with 32-bit FMA accumulation on the
// CUDA cores: the matrix product of the true 32-bit path (no tensor-core mode
// rounds its inputs), and the product for operands of mixed type (bfloat16
// activations against a matrix the checkpoint stores in 32-bit).  Any M, N, K.
// Sums over K are blocked: every 256 terms the running sum is folded into a second
// accumulator, so that the rounding of a long sum (K of 18,944 in a 7B-size down
// projection) grows like the root of the block plus the root of the number of blocks and
// not like the root of K.  The order of additions depends on K alone.
//
// The reference's 32-bit path is F.linear through cuBLAS with TF32 off
// (src/einf/executors/torch/packed_qkv.py:148, qwen.py:207-208,489,773).
#include "common.cuh"

namespace einf {

constexpr int kTile = 64;   // rows of A and rows of W per block
constexpr int kTileK = 16;
constexpr int kThreads = 256;
constexpr int kTilesPerBlockSum = 16;   // 16 tiles of 16: a block of 256 terms

template <typename TA, typename TW, typename TOut>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(const TA* __restrict__ a, const TW* __restrict__ w, const float* __restrict__ bias,
                 TOut* __restrict__ out, int m, int n, int k, long long lda, long long ldo) {
  __shared__ float a_s[kTileK][kTile + 4];
  __shared__ float w_s[kTileK][kTile + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int load_row = threadIdx.x >> 2;                   // 0..63
  const int load_k = (threadIdx.x & 3) * 4;                // 0, 4, 8, 12
  float acc[4][4], total[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = total[i][j] = 0.f;

  int tiles_in_block = 0;
  for (int k0 = 0; k0 < k; k0 += kTileK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + load_k + e;
      const int ar = row0 + load_row, wr = col0 + load_row;
      a_s[load_k + e][load_row] = (ar < m && kk < k) ? to_float(a[(size_t)ar * lda + kk]) : 0.f;
      w_s[load_k + e][load_row] = (wr < n && kk < k) ? to_float(w[(size_t)wr * k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_s[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_s[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    if (++tiles_in_block == kTilesPerBlockSum) {
      tiles_in_block = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          total[i][j] += acc[i][j];
          acc[i][j] = 0.f;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= n) continue;
      float v = total[i][j] + acc[i][j];
      if (bias) v += bias[c];
      out[(size_t)r * ldo + c] = from_float<TOut>(v);
    }
  }
}

}  // namespace einf

using namespace einf;

template <typename TA, typename TW>
static int launch(const void* a, const void* w, const float* bias, void* out, int out_dtype, int m, int n,
                  int k, long long lda, long long ldo, cudaStream_t stream) {
  dim3 grid((n + kTile - 1) / kTile, (m + kTile - 1) / kTile);
  if (out_dtype == kFloat32) {
    gemm_simt_kernel<TA, TW, float><<<grid, kThreads, 0, stream>>>((const TA*)a, (const TW*)w, bias,
                                                                  (float*)out, m, n, k, lda, ldo);
  } else {
    gemm_simt_kernel<TA, TW, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        (const TA*)a, (const TW*)w, bias, (__nv_bfloat16*)out, m, n, k, lda, ldo);
  }
  return (int)cudaGetLastError();
}

// lda / ldo: row strides of A and out in elements (rows of A may be a strided view).
extern "C" int einf_gemm_simt(const void* a, int a_dtype, const void* w, int w_dtype, const float* bias,
                              void* out, int out_dtype, int m, int n, int k, long long lda,
                              long long ldo, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (a_dtype == kFloat32) {
    if (w_dtype == kFloat32) return launch<float, float>(a, w, bias, out, out_dtype, m, n, k, lda, ldo, stream);
    return launch<float, __nv_bfloat16>(a, w, bias, out, out_dtype, m, n, k, lda, ldo, stream);
  }
  if (w_dtype == kFloat32)
    return launch<__nv_bfloat16, float>(a, w, bias, out, out_dtype, m, n, k, lda, ldo, stream);
  return launch<__nv_bfloat16, __nv_bfloat16>(a, w, bias, out, out_dtype, m, n, k, lda, ldo, stream);
}
