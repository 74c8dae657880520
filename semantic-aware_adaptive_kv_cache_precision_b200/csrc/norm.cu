// RMSNorm of rows of the fp32 residual stream:
//   out = (x * rsqrt(mean(x^2) + eps)) * w
// sum of squares, scale and products in fp32, one rounding at the store
// (`src/core_kernels/rmsnorm.cu:33-84`). One block per output row; `rows`, if
// given, picks which input row each output row normalises (used to take only
// the positions whose logits are wanted). The order of the additions depends on
// the row length alone, never on how many rows are in the batch.
//
// With `add` (fp32, `parts` tensors of x's shape, `part_stride` elements apart) the kernel
// first folds them into the stream, x += add[0] + add[1] + ..., stores x and normalises
// the sum: the residual add of the layer before and this norm read and write the stream
// once instead of twice, and a product whose K ranges were summed apart is put together
// here, in a fixed order.
#include "common.cuh"

namespace {

// Rows up to kThreads * 4 * kPerThread wide are read once and kept in registers (the
// weight is fetched before the reduction, so the row costs one memory round trip);
// wider rows are read a second time.
constexpr int kThreads = 256;
constexpr int kPerThread = 4;          // float4 loads per thread: rows up to 4096 wide

// Four weights, or four results, in one access where the type allows it.
__device__ __forceinline__ void load4(const float* p, float (&w)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&w)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo),
                                            *reinterpret_cast<const uint32_t*>(&hi));
}

template <typename W, typename Out, bool kAdd = false>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ add,
               int parts, long long part_stride, const int32_t* __restrict__ rows,
               const W* __restrict__ weight, Out* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  let_next_kernel_start();
  const bool fits = hidden <= kThreads * 4 * kPerThread && (hidden & 3) == 0 &&
                    !((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15);
  float wv[kPerThread][4];
  if (fits) {                      // the weight does not depend on the kernel before
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 4;
      if (c < hidden) load4(weight + c, wv[i]);
    }
  }
  wait_for_previous_kernel();
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* in = x + src * hidden;
  const float* more = kAdd ? add + src * hidden : nullptr;
  Out* o = out + (long long)blockIdx.x * hidden;
  if (fits) {
    float4 v[kPerThread];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 4;
      v[i] = c < hidden ? *reinterpret_cast<const float4*>(in + c) : make_float4(0, 0, 0, 0);
      if (kAdd && c < hidden) {
        float4 sum = *reinterpret_cast<const float4*>(more + c);
#pragma unroll 4
        for (int s = 1; s < parts; ++s) {
          const float4 a = *reinterpret_cast<const float4*>(more + s * part_stride + c);
          sum.x += a.x;
          sum.y += a.y;
          sum.z += a.z;
          sum.w += a.w;
        }
        v[i].x += sum.x;
        v[i].y += sum.y;
        v[i].z += sum.z;
        v[i].w += sum.w;
        *reinterpret_cast<float4*>(in + c) = v[i];
      }
      acc += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    const float scale = rsqrtf(block_sum(acc, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 4;
      if (c < hidden)
        store4(o + c, v[i].x * scale * wv[i][0], v[i].y * scale * wv[i][1],
               v[i].z * scale * wv[i][2], v[i].w * scale * wv[i][3]);
    }
    return;
  }
  float acc = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = in[i];
    if (kAdd) {                          // (read again below by this thread)
      float sum = more[i];
      for (int s = 1; s < parts; ++s) sum += more[s * part_stride + i];
      in[i] = v = v + sum;
    }
    acc += v * v;
  }
  const float scale = rsqrtf(block_sum(acc, scratch) / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = narrow<Out>(in[i] * scale * widen(weight[i]));
}

// The same for MANY rows in bfloat16 (a prefill step): a warp takes a row at a time and keeps
// it in registers, a lane every 32nd group of four floats, so that a warp's access is 512
// contiguous bytes; the sum of squares needs shuffles only, no block-wide barrier; and the
// grid is sized to the GPU and walks the rows, so that no wave is left half full. (One block a
// row, as above, took 12.0 us for 2,048 rows of 1,536 with a sum to fold: 44 MB at 3.7 TB/s.)
// The order of a row's additions depends on its length alone. `kPer`: groups of four a lane
// holds, hidden <= 128 * kPer.
template <int kPer, bool kAdd>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ add, int parts,
                    long long part_stride, const int32_t* __restrict__ rows,
                    const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                    int n_rows, int hidden, float eps) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int groups = hidden >> 2;                       // float4 groups of a row
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_rows; r += warps) {
    const long long src = rows ? rows[r] : r;
    float* in = x + src * hidden;
    float4 v[kPer];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int g = lane + 32 * i;
      v[i] = g < groups ? reinterpret_cast<const float4*>(in)[g] : make_float4(0, 0, 0, 0);
    }
    if (kAdd) {
      const float* more = add + src * hidden;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        const int g = lane + 32 * i;
        if (g < groups) {
          float4 sum = reinterpret_cast<const float4*>(more)[g];
          for (int s = 1; s < parts; ++s) {
            const float4 a = reinterpret_cast<const float4*>(more + s * part_stride)[g];
            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
          }
          v[i].x += sum.x; v[i].y += sum.y; v[i].z += sum.z; v[i].w += sum.w;
          reinterpret_cast<float4*>(in)[g] = v[i];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      acc += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    const float scale = rsqrtf(warp_sum(acc) / static_cast<float>(hidden) + eps);
    __nv_bfloat16* o = out + (long long)r * hidden;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int g = lane + 32 * i;
      if (g < groups) {
        float w[4];
        load4(weight + 4 * g, w);
        store4(o + 4 * g, v[i].x * scale * w[0], v[i].y * scale * w[1], v[i].z * scale * w[2],
               v[i].w * scale * w[3]);
      }
    }
  }
}

template <int kPer>
int launch_rows(float* x, const float* add, int parts, long long part_stride, const int32_t* rows,
                const __nv_bfloat16* weight, __nv_bfloat16* out, int n_rows, int hidden, float eps,
                cudaStream_t stream) {
  const int blocks = min((n_rows + 7) / 8, sm_count() * 8);
  if (add)
    return launch_overlapped(rmsnorm_rows_kernel<kPer, true>, dim3(blocks), dim3(256), 0, stream, 1,
                             x, add, parts, part_stride, rows, weight, out, n_rows, hidden, eps);
  return launch_overlapped(rmsnorm_rows_kernel<kPer, false>, dim3(blocks), dim3(256), 0, stream, 1,
                           x, add, parts, part_stride, rows, weight, out, n_rows, hidden, eps);
}

constexpr int kManyRows = 256;     // from here on the warp-a-row kernel runs (bfloat16 only)

}  // namespace

// `add`: null, or `parts` fp32 tensors [n_rows, hidden], `part_stride` elements apart, that
// are folded into x first (then `rows` must be null, and the weight and the output bf16).
SAKV_EXPORT int sakv_rmsnorm(float* x, const float* add, int parts, long long part_stride, const int32_t* rows, const void* weight,
                             int weight_dtype, void* out, int out_dtype, int n_rows, int hidden,
                             float eps, cudaStream_t stream) {
  if (n_rows < 0 || hidden <= 0 || (add && (rows || parts < 1)))
    return cudaErrorInvalidValue;
  if (n_rows == 0) return 0;
  const int threads = kThreads;
  // Many rows in bfloat16: a warp a row. (The 32-bit path keeps the kernel above for every
  // count of rows, so that a row's result never depends on how many rows came with it.)
  if (n_rows >= kManyRows && weight_dtype == SAKV_BF16 && out_dtype == SAKV_BF16 &&
      (hidden & 127) == 0 && hidden <= 128 * 32 &&
      !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(add) |
         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) &&
      (part_stride & 3) == 0) {
    const __nv_bfloat16* w = (const __nv_bfloat16*)weight;
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    if (hidden <= 128 * 16)
      return launch_rows<16>(x, add, parts, part_stride, rows, w, o, n_rows, hidden, eps, stream);
    return launch_rows<32>(x, add, parts, part_stride, rows, w, o, n_rows, hidden, eps, stream);
  }
  if (add) {
    if ((reinterpret_cast<uintptr_t>(add) & 15) || weight_dtype != SAKV_BF16 ||
        out_dtype != SAKV_BF16)
      return cudaErrorInvalidValue;
    return launch_overlapped(rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16, true>, dim3(n_rows),
                             dim3(threads), 0, stream, 1, x, add, parts, part_stride, rows,
                             (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, hidden, eps);
  }
#define LAUNCH(W, O)                                                                          \
  return launch_overlapped(rmsnorm_kernel<W, O>, dim3(n_rows), dim3(threads), 0, stream, 1, x, \
                           (const float*)nullptr, 0, 0LL, rows, (const W*)weight, (O*)out,     \
                           hidden, eps)
  if (weight_dtype == SAKV_F32 && out_dtype == SAKV_F32) LAUNCH(float, float);
  if (weight_dtype == SAKV_F32 && out_dtype == SAKV_BF16) LAUNCH(float, __nv_bfloat16);
  if (weight_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (weight_dtype == SAKV_BF16 && out_dtype == SAKV_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return cudaErrorInvalidValue;
}
