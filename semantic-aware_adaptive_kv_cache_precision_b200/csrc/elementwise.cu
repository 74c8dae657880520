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

// Eight bf16 (one 16-byte access) of gate and of up per thread; rows are `inter` wide with
// inter % 8 == 0, so a group of eight never straddles the gate/up boundary. blockIdx.x and
// the thread give the group within a row, blockIdx.y walks the rows, two rows at a time in
// flight. exp and the division are the fast forms (errors near 1e-6 relative, a thousandth of
// the bf16 rounding that follows): with the exact ones the kernel is bound by instruction
// issue, not by memory.
__device__ __forceinline__ uint4 gated8(const uint4& g, const uint4& u) {
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 r;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 gf = __bfloat1622float2(gp[j]), uf = __bfloat1622float2(up[j]);
    rp[j] = __floats2bfloat162_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x,
                                  __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y);
  }
  return r;
}

__global__ void gated_silu_bf16x8_kernel(const uint4* __restrict__ gate_up, uint4* __restrict__ out,
                                         int inter8, int tokens) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= inter8) return;
  for (int t = blockIdx.y * 2; t < tokens; t += gridDim.y * 2) {
    const uint4* row = gate_up + (long long)t * 2 * inter8;
    const bool two = t + 1 < tokens;
    const uint4 g0 = row[c], u0 = row[inter8 + c];
    uint4 g1 = g0, u1 = u0;
    if (two) {
      g1 = row[2 * inter8 + c];
      u1 = row[3 * inter8 + c];
    }
    out[(long long)t * inter8 + c] = gated8(g0, u0);
    if (two) out[(long long)(t + 1) * inter8 + c] = gated8(g1, u1);
  }
}

__global__ void add_into_f32x4_kernel(float4* __restrict__ acc, const float4* __restrict__ y,
                                      long long count4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 a = acc[i];
    const float4 b = y[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    acc[i] = a;
  }
}

template <typename T>
__global__ void add_into_kernel(float* __restrict__ acc, const T* __restrict__ y,
                                long long count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x)
    acc[i] += widen(y[i]);
}

// x = x * scale, then (cap > 0) x = cap * tanh(x / cap): an embedding's or a head's scale,
// and the soft cap some architectures put on their logits. fp32 in place.
__global__ void scale_cap_kernel(float* __restrict__ x, long long count, float scale, float cap) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

}  // namespace

SAKV_EXPORT int sakv_scale_cap(float* x, long long count, float scale, float cap,
                               cudaStream_t stream) {
  if (count < 0 || cap < 0.f) return cudaErrorInvalidValue;
  if (count == 0) return 0;
  return launch_overlapped(scale_cap_kernel, dim3(grid_for(count, 256)), dim3(256), 0, stream, 1,
                           x, count, scale, cap);
}

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
  if (dtype == SAKV_BF16 && inter % 8 == 0 && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
    const int across = (inter / 8 + 127) / 128;
    int down = (tokens + 1) / 2;
    const int most = (sm_count() * 16 + across - 1) / across;
    if (down > most) down = most;
    gated_silu_bf16x8_kernel<<<dim3(across, down), 128, 0, stream>>>(
        (const uint4*)gate_up, (uint4*)out, inter / 8, tokens);
    return launch_status();
  }
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
  if (dtype == SAKV_F32 && count % 4 == 0 && !((uintptr_t)acc & 15) && !((uintptr_t)y & 15)) {
    add_into_f32x4_kernel<<<grid_for(count / 4, 256, 32), 256, 0, stream>>>(
        (float4*)acc, (const float4*)y, count / 4);
    return launch_status();
  }
  const int grid = grid_for(count, 256);
  if (dtype == SAKV_F32)
    add_into_kernel<float><<<grid, 256, 0, stream>>>(acc, (const float*)y, count);
  else if (dtype == SAKV_BF16)
    add_into_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(acc, (const __nv_bfloat16*)y, count);
  else
    return cudaErrorInvalidValue;
  return launch_status();
}
