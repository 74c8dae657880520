// The feed-forward's gated product for MANY tokens (prefill) on tcgen05 tensor cores, with the
// activation in its epilogue:
//
//   out[m, n] = silu(x W_gate^T)[m, n] * (x W_up^T)[m, n]          bf16
//
// (Measured at 2,048 tokens, 1536 -> 2 x 8960: 84.1 us against 91.5 us for the library's
// product followed by the activation kernel; at 8,192 tokens 330 against 377 us, 1.37
// PFLOP/s, which is what the library's own products sustain under the power cap. The same kernel without the activation loses to the library on the other
// projections, whose few tiles of 256 x 256 leave SMs idle, so it is not offered for them.)
//
// Tokens lie on the MMA's 128 rows, weight rows on its columns: one tcgen05.mma is
// 128 x 256 x 16, which the tensor cores take at their full rate (128 cycles). A block's
// tile is 256 tokens x 256 weight rows (gated: 128 rows of the gate matrix and the same 128
// of the up matrix, so both halves of a gated output meet in one accumulator row): two
// products of 128 tokens share each weight tile, which is what keeps the traffic from L2
// under what the tensor cores can take (a tile of 128 tokens was measured at 57 % of their
// rate), and their two accumulators fill the 512 columns of tensor memory. Blocks are
// persistent: block b takes tiles b, b + grid, ..., token tiles fastest, so that the blocks
// running at one time share a few weight tiles in L2 and the weights cross HBM about once.
//
//   warp 0     TMA: per K step of 64 two boxes of x [128 x 64] and two boxes of W [128 x 64]
//              into a ring of three 64 KB stages (128-byte swizzle),
//   warps 1, 10  MMA issue: lane 0 of each takes ONE of the tile's two products through every
//              stage and commits the stage and its accumulator. (A lane pays a barrier wait of
//              some 300 cycles a stage before its products, 128 cycles each, may go out; with
//              one lane for both products the tensor pipe idled a fifth of the time.)
//   warps 2-9  epilogue, four warps for each of the tile's two products (a warp reaches the
//              32 lanes of its number modulo 4): thread = token row; reads its gate and up sums
//              16 at a time, applies silu(g) * u in fp32, stores 32 bytes at a time.
//
// The reference calls cuBLAS for every projection and runs SwiGLU as a kernel of its own
// (`src/core_kernels/linear.cu:85-142`, `src/core_kernels/swiglu.cu:26-38`). Every mbarrier
// wait is bounded; no cluster, no multicast.
#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int BM = 128;            // tokens per product = tensor-memory lanes
constexpr int kHalves = 2;         // products per tile: a tile is 256 tokens, two accumulators
constexpr int BN = 256;            // weight rows per tile = accumulator columns
constexpr int BK = 64;             // K step: one 128-byte swizzle row of bf16
constexpr int kStages = 3;
constexpr int kXBytes = kHalves * BM * BK * 2;  // 32 KB: two boxes of 128 tokens
constexpr int kWBytes = BN * BK * 2;            // 32 KB: two boxes of 128 rows
constexpr int kStageBytes = kXBytes + kWBytes;  // 64 KB
constexpr int kThreads = 64 + kHalves * 128 + 32;   // TMA, MMA, four epilogue warps a product, MMA
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr uint32_t kTmemCols = 512;

struct Params {
  int M, N, K;           // tokens; output columns (rows of each of gate and up); inner size
  int up_offset;         // row of W where the up matrix starts
  __nv_bfloat16* out;
  long long ldo;
  int m_tiles, n_tiles;
  int* error;
};

struct Barriers {
  uint64_t full[kStages], empty[kStages];
  uint64_t acc_full[kHalves];        // an accumulator of a tile is complete
  uint64_t acc_empty[kHalves];       // the epilogue has read one of them
  uint32_t tmem;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = p.m_tiles * p.n_tiles;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tma::mbar_init(&bar->full[s], 1);
      tma::mbar_init(&bar->empty[s], kHalves);       // each MMA lane lets go of it
    }
    for (int i = 0; i < kHalves; ++i) tma::mbar_init(&bar->acc_full[i], 1);
    for (int i = 0; i < kHalves; ++i) tma::mbar_init(&bar->acc_empty[i], 128);
    tma::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(&bar->tmem, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = bar->tmem;

  if (warp == 0) {
    // ---- TMA producer -----------------------------------------------------------------
    if (lane == 0) {
      tma::prefetch_map(&x_map);
      tma::prefetch_map(&w_map);
      int stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;     // token tiles fastest
        const int rows_a = n_tile * 128, rows_b = p.up_offset + n_tile * 128;   // gate, up
        for (int kb = 0; kb < n_kb; ++kb) {
          // (waiting for the parity before the ring's own: the first pass finds every stage free)
          if (!tma::mbar_wait(&bar->empty[stage], phase ^ 1, p.error, 601)) {
            ok = false;
            break;
          }
          uint8_t* dst = smem + stage * kStageBytes;
          tma::mbar_expect_tx(&bar->full[stage], kStageBytes);
          for (int h = 0; h < kHalves; ++h)
            tma::load_2d(dst + h * (kXBytes / kHalves), &x_map, kb * BK,
                         (m_tile * kHalves + h) * BM, &bar->full[stage]);
          tma::load_2d(dst + kXBytes, &w_map, kb * BK, rows_a, &bar->full[stage]);
          tma::load_2d(dst + kXBytes + kWBytes / 2, &w_map, kb * BK, rows_b, &bar->full[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2 + kHalves * 4) {
    // ---- MMA issue: this lane's product of every tile ------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, BN);
      const int h = warp == 1 ? 0 : 1;
      int stage = 0, phase = 0, round = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++round) {
        for (int kb = 0; kb < n_kb && ok; ++kb) {
          if (!tma::mbar_wait(&bar->full[stage], phase, p.error, 603)) {
            ok = false;
            break;
          }
          // the accumulator may be written again once the epilogue has read the last tile's
          if (kb == 0 && round >= 1 &&
              !tma::mbar_wait(&bar->acc_empty[h], (round - 1) & 1, p.error, 602)) {
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const uint32_t a = tma::smem_u32(smem + stage * kStageBytes) + h * (kXBytes / kHalves);
          const uint32_t b = tma::smem_u32(smem + stage * kStageBytes) + kXBytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc::mma_ss(tmem + h * BN, tc::smem_desc_k_major_sw128(a + k * 32),
                       tc::smem_desc_k_major_sw128(b + k * 32), idesc, kb > 0 || k > 0);
          tc::commit(&bar->empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc::commit(&bar->acc_full[h]);
      }
    }
  } else if (warp >= 2) {
    // ---- epilogue: thread = token row ---------------------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    int round = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++round) {
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      const int h = (warp - 2) >> 2;              // which of the tile's two products
      ok = ok && tma::mbar_wait(&bar->acc_full[h], round & 1, p.error, 604);
      tc::fence_after_sync();
      {
        const int m = (m_tile * kHalves + h) * BM + row;
        const uint32_t acc = lane_base + h * BN;
        const int n0 = n_tile * 128;
        __nv_bfloat16* dst = p.out + (long long)m * p.ldo + n0;
#pragma unroll 1
        for (int c = 0; c < 128 && ok; c += 16) {
          float g[16], u[16];
          tc::ld_32x32b_x16(acc + c, g);
          tc::ld_32x32b_x16(acc + 128 + c, u);
          if (m < p.M) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              w[i] = mma::pack_bf16(
                  __fdividef(g[2 * i], 1.0f + __expf(-g[2 * i])) * u[2 * i],
                  __fdividef(g[2 * i + 1], 1.0f + __expf(-g[2 * i + 1])) * u[2 * i + 1]);
            if (n0 + c + 16 <= p.N) {
              *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
              const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(w);
              for (int i = 0; i < 16 && n0 + c + i < p.N; ++i) dst[c + i] = wp[i];
            }
          }
        }
        tc::fence_before_sync();
        tma::mbar_arrive(&bar->acc_empty[h]);     // the products of the next tile may refill it
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

__device__ int g_error;

int launch(const CUtensorMap* x_map, const CUtensorMap* w_map, Params p, cudaStream_t stream) {
  static PerDeviceOnce configured;      // (attributes are per device)
  if (configured.needs()) {
    const cudaError_t e = cudaFuncSetAttribute(
        gemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.done();
  }
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_wide_kernel<<<grid, kThreads, kSmemBytes, stream>>>(*x_map, *w_map, p);
  return launch_status();
}

}  // namespace

// A TMA descriptor of a row-major bf16 matrix [rows, cols] read in boxes of [128 rows, 64
// columns]; `map` points to 128 bytes on the host.
SAKV_EXPORT int sakv_gemm_wide_map(void* map, const void* base, long long rows, long long cols,
                                   long long row_stride_elems) {
  if (rows <= 0 || cols <= 0 || (cols % 8) || (row_stride_elems % 8)) return cudaErrorInvalidValue;
  return tma::make_map_bf16_2d(reinterpret_cast<CUtensorMap*>(map), base, (uint64_t)rows,
                               (uint64_t)cols, (uint64_t)row_stride_elems * 2, 128, BK);
}

// out[M, N] (bf16, rows `ldo` apart) = silu(x Wg^T) * (x Wu^T) for W = [Wg; ...; Wu from row
// `up_offset` on; ...] with N rows each, over the maps of x [M, K] and W from
// sakv_gemm_wide_map. K, N and ldo multiples of 8, out 16-byte aligned.
SAKV_EXPORT int sakv_gemm_wide(const void* x_map, const void* w_map, int M, int N, int K,
                               int up_offset, void* out, long long ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (N % 8) || ldo < N || up_offset < N ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (ldo % 8))
    return cudaErrorInvalidValue;
  Params p;
  p.M = M; p.N = N; p.K = K; p.up_offset = up_offset;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.error = nullptr;
  p.m_tiles = (M + kHalves * BM - 1) / (kHalves * BM);
  p.n_tiles = (N + 127) / 128;
  return launch(reinterpret_cast<const CUtensorMap*>(x_map),
                reinterpret_cast<const CUtensorMap*>(w_map), p, stream);
}

SAKV_EXPORT int sakv_gemm_wide_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}
