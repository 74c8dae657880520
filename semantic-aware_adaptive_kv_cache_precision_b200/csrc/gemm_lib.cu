// The library's matrix product with the residual add inside it: R[t, n] += sum_k X[t, k] W[n, k]
// with bf16 operands, fp32 sums and an fp32 R that cuBLAS reads and writes (beta = 1), as the
// reference accumulates its o_proj and down_proj into the residual stream
// (`src/core_kernels/linear.cu:131-142`: cublasGemmEx, OP_T / OP_N, CUBLAS_COMPUTE_32F, beta 1).
// torch offers no product of bf16 operands into an fp32 tensor that it also adds to; without
// it the product goes to a tensor of its own and a second kernel folds it into the stream.
// Used for steps of many tokens (prefill); the handle's workspace is the caller's, so that
// nothing is allocated when a step is captured in a CUDA graph.
#include "common.cuh"
#include <cublas_v2.h>

namespace {

constexpr int kDevices = 64;
cublasHandle_t g_handles[kDevices];

cublasHandle_t handle_of_current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) return nullptr;
  if (!g_handles[device] && cublasCreate(&g_handles[device]) != CUBLAS_STATUS_SUCCESS)
    g_handles[device] = nullptr;
  return g_handles[device];
}

}  // namespace

// acc [T, N] (fp32, rows `lda` apart) += x [T, K] (bf16, rows `ldx` apart) * w [N, K]^T (bf16,
// contiguous). `workspace`: device memory for the library (256-byte aligned), or null.
// Returns 0, or 1000 + the library's status.
SAKV_EXPORT int sakv_lib_accumulate(const void* x, long long ldx, const void* w, float* acc,
                                    long long lda, int T, int N, int K, void* workspace,
                                    long long workspace_bytes, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0 || ldx < K || lda < N) return cudaErrorInvalidValue;
  cublasHandle_t handle = handle_of_current_device();
  if (!handle) return cudaErrorInitializationError;
  cublasStatus_t s = cublasSetStream(handle, stream);
  if (s == CUBLAS_STATUS_SUCCESS && workspace)
    s = cublasSetWorkspace(handle, workspace, static_cast<size_t>(workspace_bytes));
  const float one = 1.f;
  // row-major R [T, N] is column-major [N, T]: R^T = W X^T, W row-major [N, K] being column-major
  // [K, N], transposed; X row-major [T, K] being column-major [K, T], as it is
  if (s == CUBLAS_STATUS_SUCCESS)
    s = cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, N, T, K, &one, w, CUDA_R_16BF, K, x,
                     CUDA_R_16BF, static_cast<int>(ldx), &one, acc, CUDA_R_32F,
                     static_cast<int>(lda), CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  return s == CUBLAS_STATUS_SUCCESS ? 0 : 1000 + static_cast<int>(s);
}
