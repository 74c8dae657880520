// The true 32-bit matrix product of the fp32 path:
//   C[m, n] (+)= sum_k A[m, k] W[n, k]  (+ bias[n])
// with W stored (out, in) row-major as in the checkpoint, plain FFMA in fp32 (no
// TF32, no tensor cores). Each output element adds its products for k = 0, 1,
// 2, ... in that order whatever the tile and whatever M is, so a row's result
// is the same to the bit whether it is computed alone or among 2,048 others.
// This is what makes "whole prompt == token by token == batched" exact in the
// fp32 path. The reference's counterpart is cuBLAS with fp32 accumulation
// (`src/core_kernels/linear.cu:85-142`).
#include "common.cuh"

namespace {

constexpr int BN = 64, BK = 16;

// BM x 64 tile per block of 256 threads; a thread owns TM x 4 outputs.
template <int BM>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long long lda, const float* __restrict__ W,
                const float* __restrict__ bias, float* __restrict__ C, long long ldc, int M,
                int N, int K, int accumulate) {
  constexpr int TM = BM / 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? A[(long long)m * lda + k] : 0.f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const int n = n0 + r, k = k0 + c;
      Ws[c][r] = (n < N && k < K) ? W[(long long)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      float* c = C + (long long)m * ldc + n;
      *c = accumulate ? *c + v : v;
    }
  }
}

}  // namespace

SAKV_EXPORT int sakv_gemm_f32(const float* A, long long lda, const float* W, const float* bias,
                              float* C, long long ldc, int M, int N, int K, int accumulate,
                              cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || lda < K || ldc < N) return cudaErrorInvalidValue;
  if (M == 0) return 0;
  if (M <= 16) {
    const dim3 grid((N + BN - 1) / BN, (M + 15) / 16);
    gemm_f32_kernel<16><<<grid, 256, 0, stream>>>(A, lda, W, bias, C, ldc, M, N, K, accumulate);
  } else {
    const dim3 grid((N + BN - 1) / BN, (M + 63) / 64);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    gemm_f32_kernel<64><<<grid, 256, 0, stream>>>(A, lda, W, bias, C, ldc, M, N, K, accumulate);
  }
  return launch_status();
}
