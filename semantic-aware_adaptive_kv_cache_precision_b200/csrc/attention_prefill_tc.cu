// Prefill attention on tcgen05 tensor cores, head size 128: causal grouped-query flash
// attention of the step's new tokens over their sequences' caches, for batches of unequal
// lengths and for chunks that continue a cached prefix (the same contract as the mma.sync
// kernel in attention_prefill.cu, which serves head size 64 and is this kernel's test twin).
//
//   grid  = (heads, work items: a query tile of up to 128 tokens and a run of its key tiles);
//   block = 6 warps:
//     warp 0     TMA: the query tile once, then the sequence's key/value blocks (64 keys, one
//                cache block each) into a ring of stages,
//     warp 1     one lane issues every tcgen05.mma and owns tensor memory,
//     warps 2-5  softmax: ONE THREAD PER QUERY ROW (tensor-memory lane = row), so maxima and
//                sums need no shuffles.
//   per key tile j:   S_j = Q K_j^T      128 x 64 x 128, both operands K-major from shared
//                                        memory, S in tensor memory (two buffers)
//                     P_j = 2^(S_j c - m) in registers, written as bf16 pairs into tensor
//                                        memory over the first half of S_j
//                     O  += P_j V_j       128 x 128 x 64, P the A operand from tensor memory,
//                                        V MN-major exactly as TMA wrote the cache block, O
//                                        accumulating in tensor memory
//   The exponent's reference m trails the true running maximum: it is moved (and O and the
//   row sum rescaled, in tensor memory) only when the maximum has grown by more than 2^8,
//   so most tiles cost a row nothing but 64 exponentials. The MMA lane runs ahead: S_{j+1}
//   is issued before P_j V_j, so the tensor cores work on the next scores while the softmax
//   warps exponentiate the current ones; two blocks share an SM (256 of the 512 columns of
//   tensor memory each) and fill each other's gaps.
//
// Scores, maxima, exponentials, sums and the output are fp32; P is rounded to bf16 for
// P.V, as keys and values are stored. Every mbarrier wait is bounded; no cluster, no
// multicast. The reference's prefill shape is 16 queries x 1 head per block on CUDA cores
// (`src/core_kernels/attention.cu:449-746, 910-950`).
#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int D = 128;               // head size
constexpr int KT = kCacheBlock;      // keys per tile
constexpr int QT = 128;              // queries per tile = tensor-memory lanes
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr int kQBytes = QT * D * 2;              // two boxes of [128 x 64]
constexpr int kTileBytes = KT * D * 2;           // K or V: two boxes of [64 x 64]
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kSmemBytes = kQBytes + kStages * kStageBytes + 256;              // 96.25 KB
constexpr uint32_t kTmemCols = 256;              // S: 2 x 64 (P over the first 32 of each), O: 128
constexpr uint32_t kSCol = 0, kOCol = 128;
constexpr float kLazy = 8.f;                     // move the reference when the maximum grew by 2^8

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];     // keys: free again as soon as S_j is done
  uint64_t v_full[kStages], v_empty[kStages];     // values: free once P_j V_j is done
  uint64_t s_full[2];
  uint64_t p_full;       // P_j lies in tensor memory over S_j (and stale value rows are zeroed)
  uint64_t pv_done;      // P_j V_j has been added to O: O may be rescaled or read
  uint32_t tmem;
};

// V tile as the B operand of P.V: N (head dims) contiguous, 64 per 128-byte row, the next
// 64 dims one box (8 KB) further; 8 keys per 1024-byte swizzle group.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((KT * 128) >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// One block's work: a query tile and a run of its sequence's key tiles. A tile with many key
// tiles may be dealt to several blocks; each then leaves a partial (reference exponent, row
// sum, unnormalised output) that `fold_partials_kernel` merges.
struct WorkItem {
  int sequence;        // index into the step's sequences
  int row0;            // first token row of the tile in the step
  int rows;            // <= 128
  int pos0;            // position of the first row in its sequence
  int first_key_tile;  // first key tile (of 64 keys) this block walks
  int key_tiles;       // how many
  int partial;         // -1: write the output; else the index of this block's partial
  int reserved;
};
static_assert(sizeof(WorkItem) == 32, "eight ints");

__global__ void __launch_bounds__(kThreads, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                            const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map,
                            __nv_bfloat16* __restrict__ out, const WorkItem* __restrict__ work,
                            float* __restrict__ part_o, float* __restrict__ part_ml,
                            const int32_t* __restrict__ seq_lens,
                            const int32_t* __restrict__ block_table, int max_blocks, int heads,
                            int kv_heads, float scale_log2e, int window, int* __restrict__ error) {
  // 96.25 KB, so that two blocks fit an SM. The swizzled tiles need a 1024-byte aligned
  // base; a block that does not get one says so.
  extern __shared__ __align__(1024) uint8_t smem[];
  if (tma::smem_u32(smem) & 1023) {
    if (threadIdx.x == 0 && error) atomicCAS(error, 0, 499);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + kQBytes;
  Barriers* bar = reinterpret_cast<Barriers*>(kv_s + kStages * kStageBytes);

  // blockIdx.x = head, blockIdx.y = tile: the tiles come heaviest first, so the blocks that
  // start first are the long ones of every head, and the short ones fill in behind them
  const WorkItem item = work[blockIdx.y];
  const int b = item.sequence, row0 = item.row0, rows = item.rows, pos0 = item.pos0;
  const int h = blockIdx.x;
  const int g = h / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = seq_lens[b];
  const int last_pos = pos0 + rows - 1;
  const int t0 = item.first_key_tile;
  const int n = item.key_tiles;                  // key tiles t0 .. t0 + n - 1

  if (threadIdx.x == 0) {
    tma::mbar_init(&bar->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      tma::mbar_init(&bar->k_full[s], 1);
      tma::mbar_init(&bar->k_empty[s], 1);
      tma::mbar_init(&bar->v_full[s], 1);
      tma::mbar_init(&bar->v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) tma::mbar_init(&bar->s_full[i], 1);
    tma::mbar_init(&bar->p_full, QT);
    tma::mbar_init(&bar->pv_done, 1);
    tma::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(&bar->tmem, kTmemCols);
  if (warp == 0 && lane == 0) {
    tma::prefetch_map(&q_map);
    tma::prefetch_map(&k_map);
    tma::prefetch_map(&v_map);
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = bar->tmem;
  // (with its shared and tensor memory in hand: a successor that waits on this SM can never
  // hold what this block still needs)
  let_next_kernel_start();
  // All of the above ran beside the end of the kernel before this one (the position kernel,
  // which wrote the queries and the new keys and values); from here on its results are read.
  wait_for_previous_kernel();

  if (warp == 0) {
    // ---- TMA ----------------------------------------------------------------------------
    if (lane == 0) {
      tma::mbar_expect_tx(&bar->q_full, kQBytes);
      tma::load_2d(q_s, &q_map, h * D, row0, &bar->q_full);
      tma::load_2d(q_s + QT * 128, &q_map, h * D + 64, row0, &bar->q_full);
      // Keys and values have rings of their own: a key stage is free again as soon as its
      // scores are computed, long before its values are used, so the next keys are already
      // on their way while the softmax of this tile runs.
      for (int j = 0; j < n; ++j) {
        const int stage = j % kStages;
        const int block = block_table[(long long)b * max_blocks + t0 + j];
        const int krow0 = (block * kv_heads + g) * KT;
        uint8_t* dst = kv_s + stage * kStageBytes;
        if (j >= kStages &&
            !tma::mbar_wait(&bar->k_empty[stage], ((j / kStages) - 1) & 1, error, 401))
          break;
        tma::mbar_expect_tx(&bar->k_full[stage], kTileBytes);
        tma::load_2d(dst, &k_map, 0, krow0, &bar->k_full[stage]);
        tma::load_2d(dst + KT * 128, &k_map, 64, krow0, &bar->k_full[stage]);
        if (j >= kStages &&
            !tma::mbar_wait(&bar->v_empty[stage], ((j / kStages) - 1) & 1, error, 411))
          break;
        tma::mbar_expect_tx(&bar->v_full[stage], kTileBytes);
        tma::load_2d(dst + kTileBytes, &v_map, 0, krow0, &bar->v_full[stage]);
        tma::load_2d(dst + kTileBytes + KT * 128, &v_map, 64, krow0, &bar->v_full[stage]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue -------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::idesc_bf16_f32(QT, KT);                    // K-major both
      constexpr uint32_t idesc_pv = tc::idesc_bf16_f32(QT, D) | (1u << 16);        // B MN-major
      bool ok = tma::mbar_wait(&bar->q_full, 0, error, 402);
      const uint32_t q_addr = tma::smem_u32(q_s);
      auto issue_pv = [&](int i) {
        const int stage = i % kStages;
        if (!tma::mbar_wait(&bar->p_full, i & 1, error, 403)) return false;
        if (!tma::mbar_wait(&bar->v_full[stage], (i / kStages) & 1, error, 412)) return false;
        tc::fence_after_sync();
        const uint32_t v_addr = tma::smem_u32(kv_s + stage * kStageBytes + kTileBytes);
        // A = P_i from tensor memory, where the softmax wrote it over the first half of S_i
#pragma unroll
        for (int k = 0; k < KT / 16; ++k)
          tc::mma_ts(tmem + kOCol, tmem + kSCol + (i & 1) * KT + k * 8,
                     smem_desc_mn_major_sw128(v_addr + k * 2048), idesc_pv, i > 0 || k > 0);
        tc::commit(&bar->pv_done);
        tc::commit(&bar->v_empty[stage]);
        return true;
      };
      for (int j = 0; j < n && ok; ++j) {
        const int bj = j & 1, stage = j % kStages;
        // (S_j goes where S_{j-2} and then P_{j-2} lay: P_{j-2} V_{j-2} was issued before
        // this, and the tensor pipe runs one thread's products in the order it issued them)
        ok = tma::mbar_wait(&bar->k_full[stage], (j / kStages) & 1, error, 405);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t k_addr = tma::smem_u32(kv_s + stage * kStageBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          tc::mma_ss(tmem + kSCol + bj * KT,
                     tc::smem_desc_k_major_sw128(q_addr + (k >> 2) * (QT * 128) + (k & 3) * 32),
                     tc::smem_desc_k_major_sw128(k_addr + (k >> 2) * (KT * 128) + (k & 3) * 32),
                     idesc_s, k > 0);
        tc::commit(&bar->s_full[bj]);
        tc::commit(&bar->k_empty[stage]);
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok && n > 0) issue_pv(n - 1);
    }
  } else {
    // ---- softmax: one thread per query row ---------------------------------------------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                         // row of the tile = tensor-memory lane
    const int pos = pos0 + r;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_true = -INFINITY;      // running maximum of the scaled scores
    float m_ref = -INFINITY;       // what the exponentials, the row sum and O are relative to
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int bj = j & 1;
      if (!tma::mbar_wait(&bar->s_full[bj], (j >> 1) & 1, error, 407)) { ok = false; break; }
      tc::fence_after_sync();
      float s[KT];
      tc::ld_32x32b_x64(lane_base + kSCol + bj * KT, s);
      const int key0 = (t0 + j) * KT;
      const bool needs_mask = key0 + KT - 1 > pos0 || (window > 0 && key0 < last_pos - window + 1);
      if (needs_mask) {
#pragma unroll
        for (int c = 0; c < KT; ++c) {
          const int key = key0 + c;
          const bool seen = key <= pos && (window <= 0 || key > pos - window);
          s[c] = seen ? s[c] : -INFINITY;
        }
      }
      // four chains of three-input maxima: the row is one thread's, and a single chain of 64
      // would wait on itself (two warps a scheduler hide little)
      float big4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < KT; c += 8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) big4[q] = mma::max3(big4[q], s[c + 2 * q], s[c + 2 * q + 1]);
      }
      const float big = fmaxf(fmaxf(big4[0], big4[1]), fmaxf(big4[2], big4[3]));
      m_true = fmaxf(m_true, big * scale_log2e);
      bool waited = j == 0;          // whether P_{j-1} V_{j-1} is known to be done
      const bool move = m_true > m_ref + kLazy;      // (also true the first time a key is seen)
      if (__any_sync(0xffffffffu, move)) {
        const float factor = move ? mma::exp2_fast(m_ref - m_true) : 1.f;   // 0 when m_ref = -inf
        if (j >= 1) {
          // O is touched: P_{j-1} V_{j-1} must be done
          if (!tma::mbar_wait(&bar->pv_done, (j - 1) & 1, error, 408)) { ok = false; break; }
          waited = true;
          tc::fence_after_sync();
#pragma unroll
          for (int c = 0; c < D; c += 16) {
            float v[16];
            tc::ld_32x32b_x16(lane_base + kOCol + c, v);
#pragma unroll
            for (int i = 0; i < 16; i += 2) mma::mul2(v[i], v[i + 1], factor);
            tc::st_32x32b_x16(lane_base + kOCol + c, v);
          }
          tc::fence_before_sync();
        }
        if (move) {
          l *= factor;
          m_ref = m_true;
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // P row, bf16 pairs, into tensor memory over the first half of this row of S_j: the A
      // operand of P.V. Exponents two at a time (one fma for both), four running sums.
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[KT / 2];
      const float minus_m = -m_use;
#pragma unroll
      for (int i = 0; i < KT / 2; ++i) {
        float e0, e1;
        mma::fma2(e0, e1, s[2 * i], s[2 * i + 1], scale_log2e, minus_m);
        const float p0 = mma::exp2_fast(e0), p1 = mma::exp2_fast(e1);
        mma::add2(sum4[(i & 1) * 2], sum4[(i & 1) * 2 + 1], p0, p1);
        packed[i] = mma::pack_bf16(p0, p1);
      }
      tc::st_32x32b_x32(lane_base + kSCol + bj * KT, packed);
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l += sum;
      // the sequence's last block: value rows past its end are stale; zero them before P.V
      const int valid = kv_len - key0;
      if (valid < KT) {
        if (!tma::mbar_wait(&bar->v_full[j % kStages], (j / kStages) & 1, error, 413)) {
          ok = false;
          break;
        }
        uint8_t* vt = kv_s + ((j % kStages) * kStageBytes) + kTileBytes;
        for (int row = valid + (r >> 4); row < KT; row += QT / 16)
          *reinterpret_cast<uint4*>(vt + ((r & 15) >> 3) * (KT * 128) + row * 128 + ((r & 7) << 4)) =
              make_uint4(0, 0, 0, 0);
        tma::fence_proxy_async();
      }
      // every product is waited for once, in order (the barrier's phases are told apart by
      // one bit); here it has long been done
      if (!waited && !tma::mbar_wait(&bar->pv_done, (j - 1) & 1, error, 408)) { ok = false; break; }
      tc::fence_before_sync();
      tma::mbar_arrive(&bar->p_full);
    }
    if (ok && n > 0 && tma::mbar_wait(&bar->pv_done, (n - 1) & 1, error, 410)) {
      tc::fence_after_sync();
      if (item.partial >= 0) {
        // a share of the tile's keys: leave (m_ref, l, O) for the fold
        const long long slot = ((long long)item.partial * heads + h) * QT + r;
        part_ml[slot * 2] = m_ref;
        part_ml[slot * 2 + 1] = l;
        float* po = part_o + slot * D;
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          float v[16];
          tc::ld_32x32b_x16(lane_base + kOCol + c, v);
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(po + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        l = 1.f;                // (nothing below is stored)
      }
      const float inv = 1.f / l;
      __nv_bfloat16* dst = out + ((long long)(row0 + r) * heads + h) * D;
      if (item.partial < 0)
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        float v[16];
        tc::ld_32x32b_x16(lane_base + kOCol + c, v);
        if (r < rows) {
          uint32_t w[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = mma::pack_bf16(v[2 * i] * inv, v[2 * i + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
    tc::fence_before_sync();
  }
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

constexpr int kFoldRows = 8;      // rows (warps) per block of the fold

// folds[i] = {first partial, count, first token row, rows}: out = sum_s O_s 2^(m_s - M) /
// sum_s l_s 2^(m_s - M) for each row of the tile and each head (blockIdx.y).
__global__ void fold_partials_kernel(const int4* __restrict__ folds, const float* __restrict__ part_o,
                                     const float* __restrict__ part_ml,
                                     __nv_bfloat16* __restrict__ out, int heads) {
  let_next_kernel_start();
  const int4 f = folds[blockIdx.x / (QT / kFoldRows)];      // (the step's plan: there before this step)
  const int h = blockIdx.y;
  wait_for_previous_kernel();
  const int r = (blockIdx.x % (QT / kFoldRows)) * kFoldRows + (threadIdx.x >> 5);   // a warp per row
  if (r < f.w) {
    // A lane takes four of the row's 128 sizes (one 16-byte read a partial); the partials
    // are taken four at a time with every read of a round in flight together, so that a fold
    // of up to four partials costs one round trip for the maxima and sums and one for the
    // outputs. Rounds are merged like tiles of an online softmax, always in order.
    const int lane = threadIdx.x & 31;
    constexpr int kRound = 4;
    float big = -INFINITY, total = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < f.y; s0 += kRound) {
      float2 ml[kRound];
      float4 o[kRound];
#pragma unroll
      for (int j = 0; j < kRound; ++j) {
        const bool live = s0 + j < f.y;
        const long long slot = ((long long)(f.x + s0 + (live ? j : 0)) * heads + h) * QT + r;
        ml[j] = live ? *reinterpret_cast<const float2*>(part_ml + slot * 2)
                     : make_float2(-INFINITY, 0.f);
        o[j] = live ? *reinterpret_cast<const float4*>(part_o + slot * D + lane * 4)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float top = big;
#pragma unroll
      for (int j = 0; j < kRound; ++j) top = fmaxf(top, ml[j].x);
      if (top == -INFINITY) continue;
      const float keep = mma::exp2_fast(big - top);          // 0 the first time
      total *= keep;
      acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
      big = top;
#pragma unroll
      for (int j = 0; j < kRound; ++j) {
        const float w = mma::exp2_fast(ml[j].x - big);       // 0 for a partial that saw no key
        total += w * ml[j].y;
        acc.x += w * o[j].x; acc.y += w * o[j].y; acc.z += w * o[j].z; acc.w += w * o[j].w;
      }
    }
    const float inv = total > 0.f ? 1.f / total : 0.f;
    __nv_bfloat16* dst = out + ((long long)(f.z + r) * heads + h) * D + lane * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(mma::pack_bf16(acc.x * inv, acc.y * inv),
                                                mma::pack_bf16(acc.z * inv, acc.w * inv));
  }
}

__device__ int g_error;


}  // namespace

// A TMA descriptor of the step's fused projection buffer [tokens, width] (bf16), read in boxes
// of 128 rows x 64 columns; `map` points to 128 bytes on the host.
SAKV_EXPORT int sakv_prefill_attention_tc_qmap(void* map, const void* qkv, long long tokens,
                                               long long width, long long row_stride) {
  if (tokens <= 0 || width <= 0 || (width % 8) || (row_stride % 8)) return cudaErrorInvalidValue;
  return tma::make_map_bf16_2d(reinterpret_cast<CUtensorMap*>(map), qkv, (uint64_t)tokens,
                               (uint64_t)width, (uint64_t)row_stride * 2, QT, 64);
}

// `work`: n_work items of 8 ints (see WorkItem); `folds`: n_folds items of 4 ints {first
// partial, count, first token row, rows}; `part_o`, `part_ml`: scratch for the partials,
// [partials, heads, 128, 128] and [partials, heads, 128, 2] floats (unused without folds).
SAKV_EXPORT int sakv_prefill_attention_tc(const void* q_map, const void* k_map, const void* v_map,
                                          void* out, const int32_t* q_tiles, int n_tiles,
                                          const int32_t* folds, int n_folds, float* part_o,
                                          float* part_ml, const int32_t* seq_lens,
                                          const int32_t* block_table,
                                          int max_blocks, int heads, int kv_heads, int head_dim,
                                          float scale, int window, cudaStream_t stream) {
  if (n_tiles < 0 || n_tiles > 65535 || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
      max_blocks <= 0 || head_dim != D || (reinterpret_cast<uintptr_t>(q_tiles) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || n_folds < 0 || n_folds > (1 << 20) ||
      (n_folds > 0 && (!folds || !part_o || !part_ml ||
                       (reinterpret_cast<uintptr_t>(folds) & 15) ||
                       (reinterpret_cast<uintptr_t>(part_o) & 15))))
    return cudaErrorInvalidValue;
  if (n_tiles == 0) return 0;
  static PerDeviceOnce configured;      // (attributes are per device)
  int* error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  if (configured.needs()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess)      // all of the SM's memory as shared memory: two blocks fit
      e = cudaFuncSetAttribute(prefill_attention_tc_kernel,
                               cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.done();
  }
  int status = launch_overlapped(
      prefill_attention_tc_kernel, dim3(heads, n_tiles), dim3(kThreads), kSmemBytes, stream, 1,
      *(const CUtensorMap*)q_map, *(const CUtensorMap*)k_map, *(const CUtensorMap*)v_map,
      (__nv_bfloat16*)out, (const WorkItem*)q_tiles, part_o, part_ml, seq_lens, block_table,
      max_blocks, heads, kv_heads, scale * 1.4426950408889634f, window, error);
  if (status == 0 && n_folds > 0)
    status = launch_overlapped(fold_partials_kernel, dim3(n_folds * (QT / kFoldRows), heads),
                               dim3(kFoldRows * 32), 0, stream, 1, (const int4*)folds,
                               (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out,
                               heads);
  return status;
}

SAKV_EXPORT int sakv_prefill_attention_tc_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}
