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

// A candidate (value, index) as ONE 64-bit number whose order is the rule of the choice: the
// larger value first, among equal values the lower index, and a NaN below everything (it is
// the number 0, "no candidate"). The high half is the value's bits made monotone (negative
// numbers flipped whole, the others with their sign bit set), the low half the index counted
// down from 2^32 - 1; the largest number of a row is then its winner, and finding it is a
// plain maximum, whatever the order in which threads, warps and blocks are merged.
using Pick = unsigned long long;

__device__ __forceinline__ Pick pick_of(float value, int index) {
  if (value != value) return 0ull;
  const unsigned bits = __float_as_uint(value);
  const unsigned monotone = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
  return (static_cast<Pick>(monotone) << 32) | static_cast<Pick>(0xFFFFFFFFu - static_cast<unsigned>(index));
}

__device__ __forceinline__ int index_of(Pick pick, int none) {
  return pick == 0ull ? none : static_cast<int>(0xFFFFFFFFu - static_cast<unsigned>(pick & 0xFFFFFFFFull));
}

// The largest pick of a block of up to 1024 threads, in thread 0 (butterfly inside a warp,
// then the warps' picks through shared memory).
__device__ __forceinline__ Pick block_best(Pick mine, Pick* warp_picks /* 32 */) {
  for (int o = 16; o > 0; o >>= 1) {
    const Pick other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  __syncthreads();                      // the array may still be read from the call before
  if ((threadIdx.x & 31) == 0) warp_picks[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int warps = (blockDim.x + 31) >> 5;
    mine = static_cast<int>(threadIdx.x) < warps ? warp_picks[threadIdx.x] : 0ull;
    for (int o = 16; o > 0; o >>= 1) {
      const Pick other = __shfl_xor_sync(0xffffffffu, mine, o);
      mine = other > mine ? other : mine;
    }
  }
  return mine;
}

// One block scans one chunk of one row and leaves its best pick; the last block of a row to
// finish (a ticket) picks the row's winner among the chunks. The ticket counter is back at
// zero when the kernel ends.
constexpr int kChunk = 8192;

__global__ void choose_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                              float temperature, unsigned long long seed,
                              const int32_t* __restrict__ request,
                              const int32_t* __restrict__ step, int32_t* __restrict__ out,
                              Pick* __restrict__ chunk_pick, int32_t* __restrict__ tickets) {
  __shared__ Pick warp_picks[32];
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
  Pick mine = 0ull;
  const int begin = blockIdx.x * kChunk, end = min(vocab, begin + kChunk);
  for (int c = begin + threadIdx.x; c < end; c += blockDim.x) {
    float v = row[c];
    if (temperature > 0.f) {
      const unsigned long long z = splitmix64(key + (unsigned long long)c * 0x9E3779B97F4A7C15ull);
      const float u = (static_cast<float>(z >> 41) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
      v = v / temperature + (-logf(-logf(u)));
    }
    const Pick here = pick_of(v, c);
    mine = here > mine ? here : mine;
  }
  mine = block_best(mine, warp_picks);
  if (threadIdx.x == 0) {
    chunk_pick[(long long)r * chunks + blockIdx.x] = mine;
    __threadfence();
    last = atomicAdd(tickets + r, 1) == chunks - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  mine = 0ull;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const Pick here = __ldcg(chunk_pick + (long long)r * chunks + c);
    mine = here > mine ? here : mine;
  }
  mine = block_best(mine, warp_picks);
  if (threadIdx.x == 0) {
    out[r] = index_of(mine, vocab);
    tickets[r] = 0;
  }
}

}  // namespace

// Scratch per row: one 64-bit pick per chunk of 8192 logits (`chunk_pick`, 8-byte aligned), and
// a ticket that is zero between launches. `sakv_choose_chunks(vocab)` says how many chunks a row has.
SAKV_EXPORT int sakv_choose_chunks(int vocab) { return (vocab + kChunk - 1) / kChunk; }

SAKV_EXPORT int sakv_choose(const float* logits, long long row_stride, int rows, int vocab,
                            float temperature, unsigned long long seed, const int32_t* request,
                            const int32_t* step, int32_t* out, unsigned long long* chunk_pick,
                            int32_t* tickets, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || row_stride < vocab || !(temperature >= 0.f) || !chunk_pick ||
      (reinterpret_cast<uintptr_t>(chunk_pick) & 7) || !tickets || rows > 65535)
    return cudaErrorInvalidValue;
  if (temperature > 0.f && (!request || !step)) return cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const dim3 grid((vocab + kChunk - 1) / kChunk, rows);
  return launch_overlapped(choose_kernel, grid, dim3(256), 0, stream, 1, logits, row_stride, vocab,
                           temperature, seed, request, step, out, chunk_pick, tickets);
}
