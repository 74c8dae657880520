// The plain attention kernel: one warp for each (token, query head), every key
// of the cache taken one after the other with a running maximum and sum.
//
//   s_j = (q * scale) . k_j      for the keys j the query may see: j <= pos, and
//                                 pos - j < window where the layer has a window
//   out = sum_j exp(s_j - m) v_j / sum_j exp(s_j - m)
//
// q * scale, the scores, exp, the sums and the output are fp32; k and v are
// widened from their stored type (`src/core_kernels/attention.cu:541-657`).
// Keys are visited in the order of their positions, so the result for a token
// is the same to the bit whether the token came in a whole prompt, alone in a
// decode step or beside other sequences in a batch. It serves the fp32 path for
// prefill and for decode, and is what the tensor-core kernels are tested
// against.
//
// Keys and values of cache entry: [block, kv_head, 64, head_dim]; a sequence's
// blocks are block_table[seq, :]. Queries are read from the fused projection
// buffer with row stride `q_stride`; the output is [token, heads * head_dim].
#include "common.cuh"

namespace {

constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void attention_plain_kernel(const T* __restrict__ q, long long q_stride,
                                       T* __restrict__ out, const T* __restrict__ k_cache,
                                       const T* __restrict__ v_cache,
                                       const int32_t* __restrict__ positions,
                                       const int32_t* __restrict__ token_seq,
                                       const int32_t* __restrict__ block_table, int max_blocks,
                                       int tokens, int heads, int kv_heads, int head_dim,
                                       float scale, int window) {
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)tokens * heads) return;
  const int t = static_cast<int>(warp / heads);
  const int h = static_cast<int>(warp - (long long)t * heads);
  const int g = h / (heads / kv_heads);
  const int pos = positions[t];
  const int32_t* table = block_table + (long long)token_seq[t] * max_blocks;
  const int per_lane = (head_dim + 31) / 32;

  float qr[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    qr[i] = (i < per_lane && e < head_dim)
                ? widen(q[(long long)t * q_stride + (long long)h * head_dim + e]) * scale
                : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = first; j <= pos; ++j) {
    const int block = table[j / kCacheBlock];
    const long long base =
        (((long long)block * kv_heads + g) * kCacheBlock + j % kCacheBlock) * head_dim;
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (i < per_lane && e < head_dim) part += qr[i] * widen(k_cache[base + e]);
    }
    const float s = warp_sum(part);
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (i < per_lane && e < head_dim) acc[i] = acc[i] * corr + p * widen(v_cache[base + e]);
    }
    m = m_new;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    if (i < per_lane && e < head_dim)
      out[((long long)t * heads + h) * head_dim + e] = narrow<T>(acc[i] * inv);
  }
}

}  // namespace

SAKV_EXPORT int sakv_attention_plain(const void* q, int dtype, long long q_stride, void* out,
                                     const void* k_cache, const void* v_cache,
                                     const int32_t* positions, const int32_t* token_seq,
                                     const int32_t* block_table, int max_blocks, int tokens,
                                     int heads, int kv_heads, int head_dim, float scale, int window,
                                     cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || head_dim <= 0 ||
      head_dim > 32 * kMaxPerLane || max_blocks <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const int threads = 128;
  const long long warps = (long long)tokens * heads;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (dtype == SAKV_F32)
    attention_plain_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        (const float*)q, q_stride, (float*)out, (const float*)k_cache, (const float*)v_cache,
        positions, token_seq, block_table, max_blocks, tokens, heads, kv_heads, head_dim, scale,
        window);
  else if (dtype == SAKV_BF16)
    attention_plain_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
        (const __nv_bfloat16*)v_cache, positions, token_seq, block_table, max_blocks, tokens,
        heads, kv_heads, head_dim, scale, window);
  else
    return cudaErrorInvalidValue;
  return launch_status();
}
