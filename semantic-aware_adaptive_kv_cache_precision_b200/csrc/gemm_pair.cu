// The feed-forward's gated product for MANY tokens (prefill) on PAIRS of SMs: tcgen05.mma with
// `cta_group::2`, the activation in the epilogue.
//
//   out[m, n] = silu(x W_gate^T)[m, n] * (x W_up^T)[m, n]          bf16
//
// Two blocks, a cluster of 2 on the two SMs of a pair, work on one tile of 256 tokens x 256
// weight rows (128 rows of the gate matrix and the same 128 of the up matrix). Each block
// holds 128 of the tile's tokens and HALF of its weight rows in shared memory (the first
// block the gate rows, the second the up rows) and the 128 x 256 accumulator of its own
// tokens in tensor memory; one thread of the pair's first block issues every
// tcgen05.mma (256 x 256 x 16), which reads both blocks' shared memory. Against one block
// with the whole tile (gemm_wide.cu) an SM reads 64 instead of 96 bytes of operands a
// cycle from its shared memory and copies 48 instead of 64 into it (less traffic for the
// same product, and the kernel runs at the power cap, where less work is less time), and an
// accumulator is half as wide: TWO fit tensor memory, so the epilogue of a tile runs under
// the products of the next (measured: 5,900 cycles under a tile's 13,200), which the single
// block's two accumulators (all 512 columns) could not.
//
//   warp 0     TMA: per K step of 64 one box of x [128 tokens x 64] and one of W [128 rows x
//              64] into a ring of six 32 KB stages; the bytes of BOTH blocks are counted on
//              the first block's barrier (`cp.async.bulk.tensor...cta_group::2`, no multicast:
//              each block fetches its own boxes),
//   warp 1     tensor memory (allocated by this warp of both blocks together); in the first
//              block lane 0 issues the products and commits, to the barriers of both blocks,
//              the stage and the accumulator,
//   warps 2-5  epilogue: thread = token row; reads its gate and up sums 16 at a time,
//              silu(g) * u in fp32, stores 32 bytes at a time; then gives the accumulator
//              back at the first block's barrier.
//
// Pairs are persistent: pair c takes tiles c, c + pairs, ..., token tiles fastest, so that the
// pairs running at one time share a few weight tiles in L2. The reference calls cuBLAS for
// every projection and runs SwiGLU as a kernel of its own (`src/core_kernels/linear.cu:85-142`,
// `src/core_kernels/swiglu.cu:26-38`). Every mbarrier wait is bounded; before a block leaves,
// its copy lane has seen every stage given back, and the pair meets at a cluster barrier that
// every thread reaches whatever happened, so that no block leaves while the other may still
// signal its barriers or read its shared memory.
#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int BM = 128;            // tokens per block = tensor-memory lanes
constexpr int BN = 256;            // the tile's weight rows = accumulator columns
constexpr int BK = 64;             // K step: one 128-byte swizzle row of bf16
constexpr int kStages = 6;
constexpr int kXBytes = BM * BK * 2;            // 16 KB
constexpr int kWBytes = (BN / 2) * BK * 2;      // 16 KB: this block's half of the weight rows
constexpr int kStageBytes = kXBytes + kWBytes;  // 32 KB
constexpr int kEpilogueThreads = 128;
constexpr int kThreads = 64 + kEpilogueThreads;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr uint32_t kTmemCols = 512;             // two accumulators of 256 columns
constexpr uint16_t kBoth = 3;                   // both blocks of the pair

struct Params {
  int M, N, K;           // tokens; output columns (rows of each of gate and up); inner size
  int up_offset;         // row of W where the up matrix starts
  __nv_bfloat16* out;
  long long ldo;
  int m_tiles, n_tiles;
  int* error;
};

struct Barriers {
  uint64_t full[kStages];       // (the first block's are used) both blocks' boxes have landed
  uint64_t empty[kStages];      // the products that read the stage are done
  uint64_t acc_full[2];         // an accumulator is complete
  uint64_t acc_empty[2];        // (the first block's are used) both epilogues have read it
  uint32_t tmem;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // (the same offset in both blocks: the dynamic shared memory of a kernel starts at the
  // same address in every block)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tma::cluster_rank();           // 0: issues the products
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles = p.m_tiles * p.n_tiles;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tma::mbar_init(&bar->full[s], 1);
      tma::mbar_init(&bar->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tma::mbar_init(&bar->acc_full[i], 1);
      tma::mbar_init(&bar->acc_empty[i], 2 * kEpilogueThreads);
    }
    tma::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc_pair(&bar->tmem, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tma::cluster_sync_all();       // both blocks' barriers and tensor memory are there
  tc::fence_after_sync();
  const uint32_t tmem = bar->tmem;
  // (only now, with its shared and tensor memory in hand: a successor that waits on an SM
  // can then never hold what this block still needs)
  let_next_kernel_start();
  // (the copy lane waits for the kernel before this one by itself, after its first weight
  // boxes; everyone else here: nothing is written before that kernel is done)
  if (threadIdx.x != 0) wait_for_previous_kernel();

  if (warp == 0) {
    // ---- TMA producer: this block's tokens and its half of the weight rows ---------------
    if (lane == 0) {
      tma::prefetch_map(&x_map);
      tma::prefetch_map(&w_map);
      int stage = 0, phase = 0;
      bool ok = true;
      // The weights do not depend on the kernel before this one (the norm that writes x):
      // the weight boxes of the first tile's first stages are on their way before this lane
      // waits for it, and only the boxes of x come after the wait.
      const int early = pair < tiles ? min(kStages, n_kb) : 0;
      {
        const int n_tile = pair / p.m_tiles;
        const int w_row = (rank == 0 ? 0 : p.up_offset) + n_tile * (BN / 2);
        for (int kb = 0; kb < early; ++kb) {
          const uint32_t full = tma::cluster_address(tma::smem_u32(&bar->full[kb]), 0);
          if (rank == 0) tma::mbar_expect_tx(&bar->full[kb], 2 * kStageBytes);
          tma::load_2d_pair(smem + kb * kStageBytes + kXBytes, &w_map, kb * BK, w_row, full);
        }
      }
      wait_for_previous_kernel();
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;     // token tiles fastest
        const int x_row = (m_tile * 2 + static_cast<int>(rank)) * BM;
        const int w_row = (rank == 0 ? 0 : p.up_offset) + n_tile * (BN / 2);   // gate / up
        for (int kb = 0; kb < n_kb; ++kb) {
          uint8_t* dst = smem + stage * kStageBytes;
          const uint32_t full = tma::cluster_address(tma::smem_u32(&bar->full[stage]), 0);
          if (tile == pair && kb < early) {          // (its weights are on their way)
            tma::load_2d_pair(dst, &x_map, kb * BK, x_row, full);
          } else {
            // (waiting for the parity before the ring's own: the first pass finds every stage free)
            if (!tma::mbar_wait(&bar->empty[stage], phase ^ 1, p.error, 701)) {
              ok = false;
              break;
            }
            if (rank == 0) tma::mbar_expect_tx(&bar->full[stage], 2 * kStageBytes);
            tma::load_2d_pair(dst, &x_map, kb * BK, x_row, full);
            tma::load_2d_pair(dst + kXBytes, &w_map, kb * BK, w_row, full);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // Before this block may leave: every stage it filled has been given back (the last
      // commits of the first block arrive at THIS block's barriers too).
      for (int s = 0; s < kStages && ok; ++s) {
        ok = tma::mbar_wait(&bar->empty[stage], phase ^ 1, p.error, 705);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue: one lane of the pair's first block ---------------------------------
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(2 * BM, BN);
      int stage = 0, phase = 0, round = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++round) {
        const int buf = round & 1;
        // the accumulator may be written again once both epilogues have read its last tile
        if (round >= 2 && !tma::mbar_wait(&bar->acc_empty[buf], ((round >> 1) - 1) & 1, p.error, 702)) {
          ok = false;
          break;
        }
        for (int kb = 0; kb < n_kb && ok; ++kb) {
          if (!tma::mbar_wait(&bar->full[stage], phase, p.error, 703)) {
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const uint32_t a = tma::smem_u32(smem + stage * kStageBytes);
          const uint32_t b = a + kXBytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc::mma_ss_pair(tmem + buf * BN, tc::smem_desc_k_major_sw128(a + k * 32),
                            tc::smem_desc_k_major_sw128(b + k * 32), idesc, kb > 0 || k > 0);
          tc::commit_pair(&bar->empty[stage], kBoth);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc::commit_pair(&bar->acc_full[buf], kBoth);
      }
    }
  } else {
    // ---- epilogue: thread = token row ---------------------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    int round = 0;
    bool ok = true;
    for (int tile = pair; tile < tiles; tile += pairs, ++round) {
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      const int buf = round & 1;
      ok = ok && tma::mbar_wait(&bar->acc_full[buf], (round >> 1) & 1, p.error, 704);
      tc::fence_after_sync();
      const int m = (m_tile * 2 + static_cast<int>(rank)) * BM + row;
      const uint32_t acc = lane_base + buf * BN;
      const int n0 = n_tile * (BN / 2);
      __nv_bfloat16* dst = p.out + (long long)m * p.ldo + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 2 && ok; c += 16) {
        float g[16], u[16];
        tc::ld_32x32b_x16(acc + c, g);
        tc::ld_32x32b_x16(acc + BN / 2 + c, u);
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
      // (given back whatever happened: the issuing lane counts 256 arrivals a tile)
      tma::mbar_arrive_cluster(tma::cluster_address(tma::smem_u32(&bar->acc_empty[buf]), 0));
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  tma::cluster_sync_all();       // nothing of the other block is in flight towards this one
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc_pair(tmem, kTmemCols);
  }
}

__device__ int g_error;

// Pairs that can run at one time (0: the device places no such cluster).
int resident_pairs() {
  static int known[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (known[device]) return known[device] - 1;
  int clusters = 0;
  if (cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemBytes) == cudaSuccess) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * sm_count());
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel, &config) != cudaSuccess)
      clusters = 0;
    cudaGetLastError();
  }
  known[device] = clusters + 1;
  return clusters;
}

}  // namespace

// How many pairs of SMs the kernel can hold at one time on this device (74 on a B200; 0 if it
// cannot run here).
SAKV_EXPORT int sakv_gemm_pair_resident() { return resident_pairs(); }

// A TMA descriptor of a row-major bf16 matrix [rows, cols] read in boxes of [128 rows, 64
// columns]; `map` points to 128 bytes on the host.
SAKV_EXPORT int sakv_gemm_pair_map(void* map, const void* base, long long rows, long long cols,
                                   long long row_stride_elems) {
  if (rows <= 0 || cols <= 0 || (cols % 8) || (row_stride_elems % 8)) return cudaErrorInvalidValue;
  return tma::make_map_bf16_2d(reinterpret_cast<CUtensorMap*>(map), base, (uint64_t)rows,
                               (uint64_t)cols, (uint64_t)row_stride_elems * 2, BM, BK);
}

// out[M, N] (bf16, rows `ldo` apart) = silu(x Wg^T) * (x Wu^T) for W = [Wg; ...; Wu from row
// `up_offset` on; ...] with N rows each, over tensor maps of x [M, K] and W from
// sakv_gemm_pair_map. K, N and ldo multiples of 8, out
// 16-byte aligned.
SAKV_EXPORT int sakv_gemm_pair(const void* x_map, const void* w_map, int M, int N, int K,
                               int up_offset, void* out, long long ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (N % 8) || ldo < N || up_offset < N ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (ldo % 8))
    return cudaErrorInvalidValue;
  const int pairs_here = resident_pairs();
  if (pairs_here <= 0) return cudaErrorNotSupported;
  Params p;
  p.M = M; p.N = N; p.K = K; p.up_offset = up_offset;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.error = nullptr;
  p.m_tiles = (M + 2 * BM - 1) / (2 * BM);
  p.n_tiles = (N + BN / 2 - 1) / (BN / 2);
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  const int tiles = p.m_tiles * p.n_tiles;
  const int pairs = tiles < pairs_here ? tiles : pairs_here;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see common.cuh
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&config, gemm_pair_kernel,
                                           *reinterpret_cast<const CUtensorMap*>(x_map),
                                           *reinterpret_cast<const CUtensorMap*>(w_map), p);
  return e != cudaSuccess ? static_cast<int>(e) : launch_status();
}

SAKV_EXPORT int sakv_gemm_pair_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}
