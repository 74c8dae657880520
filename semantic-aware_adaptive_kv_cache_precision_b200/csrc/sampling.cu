// Choosing a token from a row of fp32 logits.
//
// Greedy: the largest logit, the lowest index on a tie; NaN never wins, and a
// row with no winner gives `vocab` (an index past the end), which the host
// refuses (`src/core_kernels/argmax.cu:19-67`).
//
// Temperature T > 0: a draw from softmax(logits / T) by the Gumbel-max rule,
// argmax_i(logits[i] / T + g_i) with g_i = -log(-log(u_i)) and u_i a uniform
// number from a counter-based hash of (seed, request, step, i). The noise of a
// token depends on nothing else, so what a request samples does not depend on
// which other requests share its batch. The reference samples greedily only.
#include "common.cuh"
#include <float.h>

namespace {

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ void keep_better(float& best, int& at, float value, int index) {
  if (value > best || (value == best && index < at)) {
    best = value;
    at = index;
  }
}

// One block scans one chunk of one row and leaves its best (value, index); the last
// block of a row to finish (a ticket) picks the row's winner among the chunks. The
// ticket counter is back at zero when the kernel ends.
constexpr int kChunk = 8192;

__global__ void choose_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                              float temperature, unsigned long long seed,
                              const int32_t* __restrict__ request,
                              const int32_t* __restrict__ step, int32_t* __restrict__ out,
                              float* __restrict__ chunk_best, int32_t* __restrict__ chunk_at,
                              int32_t* __restrict__ tickets) {
  __shared__ float best_s[32];
  __shared__ int at_s[32];
  __shared__ int last;
  let_next_kernel_start();
  wait_for_previous_kernel();
  const int r = blockIdx.y, chunks = gridDim.x;
  const float* row = logits + (long long)r * row_stride;
  unsigned long long key = 0;
  if (temperature > 0.f) {
    key = splitmix64(seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(unsigned)(request[r] + 1));
    key = splitmix64(key ^ ((unsigned long long)(unsigned)step[r] * 0xD1B54A32D192ED03ull));
  }
  float best = -INFINITY;
  int at = vocab;
  const int begin = blockIdx.x * kChunk, end = min(vocab, begin + kChunk);
  for (int c = begin + threadIdx.x; c < end; c += blockDim.x) {
    float v = row[c];
    if (temperature > 0.f) {
      const unsigned long long z = splitmix64(key + (unsigned long long)c * 0x9E3779B97F4A7C15ull);
      const float u = (static_cast<float>(z >> 41) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
      v = v / temperature + (-logf(-logf(u)));
    }
    keep_better(best, at, v, c);
  }
  for (int o = 16; o > 0; o >>= 1)
    keep_better(best, at, __shfl_down_sync(0xffffffffu, best, o),
                __shfl_down_sync(0xffffffffu, at, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_s[warp] = best;
    at_s[warp] = at;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 1; w < warps; ++w) keep_better(best_s[0], at_s[0], best_s[w], at_s[w]);
    chunk_best[(long long)r * chunks + blockIdx.x] = best_s[0];
    chunk_at[(long long)r * chunks + blockIdx.x] = at_s[0];
    __threadfence();
    last = atomicAdd(tickets + r, 1) == chunks - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  best = -INFINITY;
  at = vocab;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x)
    keep_better(best, at, __ldcg(chunk_best + (long long)r * chunks + c),
                __ldcg(chunk_at + (long long)r * chunks + c));
  for (int o = 16; o > 0; o >>= 1)
    keep_better(best, at, __shfl_down_sync(0xffffffffu, best, o),
                __shfl_down_sync(0xffffffffu, at, o));
  if (lane == 0) {
    best_s[warp] = best;
    at_s[warp] = at;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 1; w < warps; ++w) keep_better(best_s[0], at_s[0], best_s[w], at_s[w]);
    out[r] = at_s[0];
    tickets[r] = 0;
  }
}

}  // namespace

// Scratch per row: one (value, index) pair per chunk of 8192 logits, and a ticket that is
// zero between launches. `sakv_choose_chunks(vocab)` says how many chunks a row has.
SAKV_EXPORT int sakv_choose_chunks(int vocab) { return (vocab + kChunk - 1) / kChunk; }

SAKV_EXPORT int sakv_choose(const float* logits, long long row_stride, int rows, int vocab,
                            float temperature, unsigned long long seed, const int32_t* request,
                            const int32_t* step, int32_t* out, float* chunk_best,
                            int32_t* chunk_at, int32_t* tickets, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || row_stride < vocab || !(temperature >= 0.f) || !chunk_best ||
      !chunk_at || !tickets || rows > 65535)
    return cudaErrorInvalidValue;
  if (temperature > 0.f && (!request || !step)) return cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const dim3 grid((vocab + kChunk - 1) / kChunk, rows);
  return launch_overlapped(choose_kernel, grid, dim3(256), 0, stream, 1, logits, row_stride, vocab,
                           temperature, seed, request, step, out, chunk_best, chunk_at, tickets);
}
