// Rotary position encoding of queries and keys, fused with the cache write.
//
// Rotate-half pairing over the first `rot` sizes of each head: for j < rot/2,
//   out[j]         = x[j] cos - x[j + rot/2] sin
//   out[j + rot/2] = x[j + rot/2] cos + x[j] sin
// with cos/sin of pos * theta^(-2j/rot) read from a table that the host builds
// in float64 and stores in fp32 (`src/core_kernels/rope.cu:32-54`,
// `src/core_kernels/rope_table.cu:18-31`). The rotation is fp32 with one
// rounding at the store.
//
// Input is the fused projection output qkv[t, :] = [q (A heads) | k (G heads) |
// v (G heads)]. Queries are rotated in place; keys are rotated and written to
// the cache, values are copied to the cache. A token's place in the cache is
// block_table[seq, pos / 64] * 64 + pos % 64 of its sequence's blocks; the
// layout of one cache entry is [block, kv_head, 64, head_dim].
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, long long row_stride,
                                  const int32_t* __restrict__ positions,
                                  const int32_t* __restrict__ token_seq,
                                  const int32_t* __restrict__ block_table, int max_blocks,
                                  const float* __restrict__ cos_table,
                                  const float* __restrict__ sin_table, int rot,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int heads,
                                  int kv_heads, int head_dim, int write_cache) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const int t = blockIdx.x;
  const int h = blockIdx.y;  // 0..A-1 queries, A..A+G-1 keys, A+G..A+2G-1 values
  const int pos = positions[t];
  T* row = qkv + (long long)t * row_stride + (long long)h * head_dim;
  const int half = rot / 2;
  const bool is_q = h < heads;
  const bool is_k = !is_q && h < heads + kv_heads;
  T* dst = nullptr;
  if (!is_q) {
    if (!write_cache) return;
    const int g = is_k ? h - heads : h - heads - kv_heads;
    const int block = block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock];
    if (block < 0) return;
    dst = (is_k ? k_cache : v_cache) +
          (((long long)block * kv_heads + g) * kCacheBlock + pos % kCacheBlock) * head_dim;
  }
  if (is_q || is_k) {
    T* o = is_q ? row : dst;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float c = 1.f, s = 0.f;
      if (cos_table) {
        c = cos_table[(long long)pos * half + j];
        s = sin_table[(long long)pos * half + j];
      }
      const float x1 = widen(row[j]), x2 = widen(row[j + half]);
      o[j] = narrow<T>(x1 * c - x2 * s);
      o[j + half] = narrow<T>(x2 * c + x1 * s);
    }
    if (!is_q)
      for (int j = rot + threadIdx.x; j < head_dim; j += blockDim.x) o[j] = row[j];
  } else {
    for (int j = threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = row[j];
  }
}

}  // namespace

SAKV_EXPORT int sakv_rope_store(void* qkv, int dtype, long long row_stride,
                                const int32_t* positions, const int32_t* token_seq,
                                const int32_t* block_table, int max_blocks,
                                const float* cos_table, const float* sin_table, int rot,
                                void* k_cache, void* v_cache, int tokens, int heads, int kv_heads,
                                int head_dim, int write_cache, cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || rot < 0 || rot > head_dim ||
      (rot & 1) || max_blocks <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const dim3 grid(tokens, heads + 2 * kv_heads);
  const int threads = head_dim / 2 >= 64 ? 64 : 32;
  if (dtype == SAKV_F32)
    return launch_overlapped(rope_store_kernel<float>, grid, dim3(threads), 0, stream, 1,
                             (float*)qkv, row_stride, positions, token_seq, block_table,
                             max_blocks, cos_table, sin_table, rot, (float*)k_cache,
                             (float*)v_cache, heads, kv_heads, head_dim, write_cache);
  if (dtype == SAKV_BF16)
    return launch_overlapped(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, 1,
                             (__nv_bfloat16*)qkv, row_stride, positions, token_seq, block_table,
                             max_blocks, cos_table, sin_table, rot, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, heads, kv_heads, head_dim, write_cache);
  return cudaErrorInvalidValue;
}
