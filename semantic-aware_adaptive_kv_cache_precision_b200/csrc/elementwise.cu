// Embedding gather, gated activation, residual add, row gather.
//
// The reference's versions: `src/core_kernels/embed.cu:27-43` (an id outside the
// table gives a zero row), `src/core_kernels/swiglu.cu:26-38`
// (`g / (1 + expf(-g)) * u` in fp32), `src/core_kernels/residual.cu:17-26`.
#include "common.cuh"

namespace {

template <typename Table>
__global__ void embed_kernel(const int32_t* __restrict__ ids, const Table* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab, long long count) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long token = i / hidden;
    const int col = static_cast<int>(i - token * hidden);
    const int id = ids[token];
    out[i] = (id >= 0 && id < vocab) ? widen(table[(long long)id * hidden + col]) : 0.f;
  }
}

// gate_up[t, 0:I] = gate, gate_up[t, I:2I] = up  ->  out[t, 0:I]
template <typename T>
__global__ void gated_silu_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                                  int inter, long long count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / inter;
    const int c = static_cast<int>(i - t * inter);
    const float g = widen(gate_up[t * 2 * inter + c]);
    const float u = widen(gate_up[t * 2 * inter + inter + c]);
    const float silu = g / (1.0f + expf(-g));
    out[i] = narrow<T>(silu * u);
  }
}

template <typename T>
__global__ void add_into_kernel(float* __restrict__ acc, const T* __restrict__ y,
                                long long count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x)
    acc[i] += widen(y[i]);
}

}  // namespace

SAKV_EXPORT int sakv_embed(const int32_t* ids, const void* table, int table_dtype, float* out,
                           int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens < 0 || hidden <= 0 || vocab <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * hidden;
  const int grid = grid_for(count, 256);
  if (table_dtype == SAKV_F32)
    return launch_overlapped(embed_kernel<float>, dim3(grid), dim3(256), 0, stream, 1, ids,
                             (const float*)table, out, hidden, vocab, count);
  if (table_dtype == SAKV_BF16)
    return launch_overlapped(embed_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, 1, ids,
                             (const __nv_bfloat16*)table, out, hidden, vocab, count);
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_gated_silu(const void* gate_up, void* out, int dtype, int tokens, int inter,
                                cudaStream_t stream) {
  if (tokens < 0 || inter <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * inter;
  const int grid = grid_for(count, 256);
  if (dtype == SAKV_F32)
    gated_silu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, count);
  else if (dtype == SAKV_BF16)
    gated_silu_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, count);
  else
    return cudaErrorInvalidValue;
  return launch_status();
}

SAKV_EXPORT int sakv_add_into(float* acc, const void* y, int dtype, long long count,
                              cudaStream_t stream) {
  if (count < 0) return cudaErrorInvalidValue;
  if (count == 0) return 0;
  const int grid = grid_for(count, 256);
  if (dtype == SAKV_F32)
    add_into_kernel<float><<<grid, 256, 0, stream>>>(acc, (const float*)y, count);
  else if (dtype == SAKV_BF16)
    add_into_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(acc, (const __nv_bfloat16*)y, count);
  else
    return cudaErrorInvalidValue;
  return launch_status();
}
