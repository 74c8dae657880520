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

// The same for bf16 with head sizes and rotary sizes that are multiples of 16: one block
// per token, one thread per group of 8 dims of a rotary pair (two 16-byte accesses in,
// two out) or per 16-byte piece of what is only copied.
__global__ void rope_store_bf16_vec_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride,
                                           const int32_t* __restrict__ positions,
                                           const int32_t* __restrict__ token_seq,
                                           const int32_t* __restrict__ block_table, int max_blocks,
                                           const float* __restrict__ cos_table,
                                           const float* __restrict__ sin_table, int rot,
                                           __nv_bfloat16* __restrict__ k_cache,
                                           __nv_bfloat16* __restrict__ v_cache, int heads,
                                           int kv_heads, int head_dim, int write_cache) {
  let_next_kernel_start();
  // Positions, sequence indices and block lists are the step's inputs, written before its
  // first kernel started: these dependent loads are done while the kernel before this one
  // (which writes qkv) is still running.
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot / 2;
  const int block = write_cache
                        ? block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock]
                        : -1;
  wait_for_previous_kernel();
  const int per_head = head_dim / 8;                 // 16-byte pieces per head
  const int rot_pieces = half / 8;                   // pieces of the first half of the rotary part
  const int all_heads = heads + 2 * kv_heads;
  for (int item = threadIdx.x; item < all_heads * per_head; item += blockDim.x) {
    const int h = item / per_head, piece = item - h * per_head;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    __nv_bfloat16* row = qkv + (long long)t * row_stride + (long long)h * head_dim;
    __nv_bfloat16* dst = row;
    if (!is_q) {
      if (block < 0) continue;
      const int g = is_k ? h - heads : h - heads - kv_heads;
      dst = (is_k ? k_cache : v_cache) +
            (((long long)block * kv_heads + g) * kCacheBlock + pos % kCacheBlock) * head_dim;
    }
    const int e = piece * 8;                         // first dim of this piece
    if ((is_q || is_k) && cos_table && e < rot) {
      if (piece >= rot_pieces) continue;             // the partner piece does both halves
      const uint4 a = *reinterpret_cast<const uint4*>(row + e);
      const uint4 b = *reinterpret_cast<const uint4*>(row + e + half);
      const float4 c0 = *reinterpret_cast<const float4*>(cos_table + (long long)pos * half + e);
      const float4 c1 = *reinterpret_cast<const float4*>(cos_table + (long long)pos * half + e + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sin_table + (long long)pos * half + e);
      const float4 s1 = *reinterpret_cast<const float4*>(sin_table + (long long)pos * half + e + 4);
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
      const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(&b);
      uint4 lo, hi;
      __nv_bfloat16* lp = reinterpret_cast<__nv_bfloat16*>(&lo);
      __nv_bfloat16* hp = reinterpret_cast<__nv_bfloat16*>(&hi);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x1 = __bfloat162float(ap[j]), x2 = __bfloat162float(bp[j]);
        lp[j] = __float2bfloat16_rn(x1 * c[j] - x2 * s[j]);
        hp[j] = __float2bfloat16_rn(x2 * c[j] + x1 * s[j]);
      }
      *reinterpret_cast<uint4*>(dst + e) = lo;
      *reinterpret_cast<uint4*>(dst + e + half) = hi;
    } else if (!is_q) {
      *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(row + e);
    }
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
  if (dtype == SAKV_BF16 && head_dim % 16 == 0 && rot % 16 == 0 && row_stride % 8 == 0 &&
      !((uintptr_t)qkv & 15) && !((uintptr_t)k_cache & 15) && !((uintptr_t)v_cache & 15) &&
      !((uintptr_t)cos_table & 15) && !((uintptr_t)sin_table & 15) && (rot / 2) % 4 == 0) {
    const int items = (heads + 2 * kv_heads) * (head_dim / 8);
    const int threads = items >= 256 ? 256 : ((items + 31) / 32) * 32;
    return launch_overlapped(rope_store_bf16_vec_kernel, dim3(tokens), dim3(threads), 0, stream, 1,
                             (__nv_bfloat16*)qkv, row_stride, positions, token_seq, block_table,
                             max_blocks, cos_table, sin_table, rot, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, heads, kv_heads, head_dim, write_cache);
  }
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
