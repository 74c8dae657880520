// RMSNorm of rows of the fp32 residual stream:
//   out = (x * rsqrt(mean(x^2) + eps)) * w
// sum of squares, scale and products in fp32, one rounding at the store
// (`src/core_kernels/rmsnorm.cu:33-84`). One block per output row; `rows`, if
// given, picks which input row each output row normalises (used to take only
// the positions whose logits are wanted). The order of the additions depends on
// the row length alone, never on how many rows are in the batch.
#include "common.cuh"

namespace {

template <typename W, typename Out>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                               const W* __restrict__ weight, Out* __restrict__ out, int hidden,
                               float eps) {
  __shared__ float scratch[33];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* in = x + src * hidden;
  Out* o = out + (long long)blockIdx.x * hidden;
  float acc = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = in[i];
    acc += v * v;
  }
  const float total = block_sum(acc, scratch);
  const float scale = rsqrtf(total / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = narrow<Out>(in[i] * scale * widen(weight[i]));
}

}  // namespace

SAKV_EXPORT int sakv_rmsnorm(const float* x, const int32_t* rows, const void* weight,
                             int weight_dtype, void* out, int out_dtype, int n_rows, int hidden,
                             float eps, cudaStream_t stream) {
  if (n_rows < 0 || hidden <= 0) return cudaErrorInvalidValue;
  if (n_rows == 0) return 0;
  const int threads = 256;
#define LAUNCH(W, O)                                                                       \
  rmsnorm_kernel<W, O><<<n_rows, threads, 0, stream>>>(x, rows, (const W*)weight, (O*)out, \
                                                       hidden, eps)
  if (weight_dtype == SAKV_F32 && out_dtype == SAKV_F32) LAUNCH(float, float);
  else if (weight_dtype == SAKV_F32 && out_dtype == SAKV_BF16) LAUNCH(float, __nv_bfloat16);
  else if (weight_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (weight_dtype == SAKV_BF16 && out_dtype == SAKV_F32) LAUNCH(__nv_bfloat16, float);
  else return cudaErrorInvalidValue;
#undef LAUNCH
  return launch_status();
}
