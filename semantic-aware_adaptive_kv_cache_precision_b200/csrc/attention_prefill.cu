// Prefill attention in bfloat16: causal grouped-query flash attention of the step's
// new tokens over their sequences' caches (which already hold these tokens' keys
// and values), for batches of sequences of unequal length and for chunks that
// continue a cached prefix.
//
//   grid  = (query tiles of all sequences, heads); block = 4 warps (registers are handed
//   out four warps at a time, so a fifth warp for the copies would cost a whole block of
//   occupancy; lane 0 of warp 0 issues the copies between its tiles instead)
//   a query tile is up to 64 consecutive tokens of one sequence; each compute warp
//   owns 16 of them (the rows of m16n8k16 tensor-core products) and walks over the
//   sequence's key tiles (one cache block of 64 keys each, fetched by TMA with the
//   128-byte swizzle into a ring of stages guarded by full/empty mbarriers) with a
//   running maximum and sum per row.
//
// Scores, maximum, exp2, sums and the output accumulate in fp32; probabilities are
// rounded to bf16 for P.V. A query at position p sees keys j <= p and, with a
// window w, only j > p - w. The reference's prefill shape is 16 queries x 1 head
// per block on CUDA cores (`src/core_kernels/attention.cu:449-746, 910-950`).
#include "common.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace {

constexpr int KT = kCacheBlock;      // keys per tile
constexpr int QT = 64;               // queries per tile
constexpr int kComputeWarps = 4;
constexpr int kThreads = kComputeWarps * 32;
constexpr int kStages = 3;
static_assert(QT == kComputeWarps * 16, "one m16 row tile per compute warp");

template <int D>
struct Smem {
  static constexpr int kBoxes = D / 64;
  static constexpr int kTileBytes = KT * D * 2;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kBytes = kStages * kStageBytes + 1024 + 256;
};

// q_tiles[i] = {sequence, first token row of the tile in the step, rows, position of the first row}
template <int D>
__global__ void __launch_bounds__(kThreads)
prefill_attention_kernel(const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map,
                         const __nv_bfloat16* __restrict__ q, long long q_stride,
                         __nv_bfloat16* __restrict__ out, const int4* __restrict__ q_tiles,
                         const int32_t* __restrict__ seq_lens,
                         const int32_t* __restrict__ block_table, int max_blocks, int heads,
                         int kv_heads, float scale_log2e, int window, int* __restrict__ error) {
  using S = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty = full + kStages;

  const int4 tile = q_tiles[blockIdx.x];
  const int b = tile.x, row0 = tile.y, rows = tile.z, pos0 = tile.w;
  const int h = blockIdx.y;
  const int g = h / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = seq_lens[b];
  const int last_pos = pos0 + rows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int t0 = first_key / KT;
  const int t1 = last_pos / KT + 1;            // key tiles [t0, t1)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tma::mbar_init(&full[s], 1);
      tma::mbar_init(&empty[s], kComputeWarps);
    }
    tma::fence_barrier_init();
  }
  __syncthreads();

  // Tile i of the sequence's keys goes to stage i % kStages. Lane 0 of warp 0 keeps the
  // ring full: it starts with kStages tiles and, after its own tile i, asks for tile
  // i + kStages as soon as every warp has let go of tile i.
  auto request = [&](int i) {
    const int t = t0 + i;
    const int stage = i % kStages;
    const int block = block_table[(long long)b * max_blocks + t];
    const int krow0 = (block * kv_heads + g) * KT;
    uint8_t* dst = smem + stage * S::kStageBytes;
    tma::mbar_expect_tx(&full[stage], S::kStageBytes);
    for (int x = 0; x < S::kBoxes; ++x) {
      tma::load_2d(dst + x * (KT * 128), &k_map, x * 64, krow0, &full[stage]);
      tma::load_2d(dst + S::kTileBytes + x * (KT * 128), &v_map, x * 64, krow0, &full[stage]);
    }
  };
  const int n_key_tiles = t1 - t0;
  if (threadIdx.x == 0) {
    tma::prefetch_map(&k_map);
    tma::prefetch_map(&v_map);
    for (int i = 0; i < min(kStages, n_key_tiles); ++i) request(i);
  }

  // ---- compute warps: rows warp*16 + lane/4 and + 8 of the query tile -----------------
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int p_row[2] = {pos0 + r0, pos0 + r1};          // positions of this thread's two rows
  uint32_t qf[D / 16][4];
  {
    const int c = (lane & 3) * 2;
    const __nv_bfloat16* q0 = q + (long long)(row0 + r0) * q_stride + (long long)h * D;
    const __nv_bfloat16* q1 = q + (long long)(row0 + r1) * q_stride + (long long)h * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int col = ks * 16 + c;
      qf[ks][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
      qf[ks][1] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
      qf[ks][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
      qf[ks][3] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  bool alive = true;

  for (int t = t0, i = 0; t < t1; ++t, ++i) {
    const int stage = i % kStages;
    if (!tma::mbar_wait(&full[stage], (i / kStages) & 1, error, 202)) {
      alive = false;
      break;
    }
    const uint32_t kbase = tma::smem_u32(smem + stage * S::kStageBytes);
    const uint32_t vbase = kbase + S::kTileBytes;
    const int key0 = t * KT;
    if (kv_len - key0 < KT) {
      // the sequence's last block: value rows past its end are stale; zero them (every
      // compute warp takes this branch together, so the named barrier is safe)
      uint8_t* vt = smem + stage * S::kStageBytes + S::kTileBytes;
      for (int r = kv_len - key0 + warp; r < KT; r += kComputeWarps)
        for (int x = 0; x < S::kBoxes; ++x)
          reinterpret_cast<uint32_t*>(vt + x * (KT * 128) + r * 128)[lane] = 0u;
      asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32));
    }
    // S = Q K^T: 16 rows x 64 keys = 8 n-tiles
    float s[KT / 8][4];
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    {
      const int krow = (lane & 7) + ((lane >> 4) << 3);
      const int half = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int chunk = ks * 2 + half;
        const uint32_t base = kbase + (chunk >> 3) * (KT * 128);
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          uint32_t b0, b1, b2, b3;
          mma::ldmatrix_x4(mma::swizzled(base, kk * 16 + krow, chunk & 7), b0, b1, b2, b3);
          mma::bf16_16816(s[2 * kk], qf[ks], b0, b1);
          mma::bf16_16816(s[2 * kk + 1], qf[ks], b2, b3);
        }
      }
    }
    // Mask (a tile wholly inside every row's view needs none), then the running maximum
    // of the raw scores; the scale is applied inside the exponent: p = 2^(s * c - m).
    const bool needs_mask = key0 + KT - 1 > pos0 || (window > 0 && key0 < last_pos - window + 1);
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        if (needs_mask) {
          const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const bool seen = key <= p_row[r] && (window <= 0 || key > p_row[r] - window);
          s[nt][e] = seen ? s[nt][e] : -INFINITY;
        }
        tile_max[r] = fmaxf(tile_max[r], s[nt][e]);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m[r], tile_max[r] * scale_log2e);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;      // a row that has seen nothing yet
      corr[r] = mma::exp2_fast(m[r] - m_use[r]);
      m[r] = m_new;
      l[r] *= corr[r];
    }
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = mma::exp2_fast(fmaf(s[nt][e], scale_log2e, -m_use[r]));
        s[nt][e] = p;
        l[r] += p;
      }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
        o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
      }
    }
    // O += P V: four k-steps of 16 keys
    {
      const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int half = lane >> 4;
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t pf[4];
        pf[0] = mma::pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[1] = mma::pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[2] = mma::pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[3] = mma::pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          const int chunk = j * 2 + half;
          uint32_t b0, b1, b2, b3;
          mma::ldmatrix_x4_trans(
              mma::swizzled(vbase + (chunk >> 3) * (KT * 128), kk * 16 + vrow, chunk & 7), b0, b1,
              b2, b3);
          mma::bf16_16816(o[2 * j], pf, b0, b1);
          mma::bf16_16816(o[2 * j + 1], pf, b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) {
      tma::mbar_arrive(&empty[stage]);
      if (warp == 0 && i + kStages < n_key_tiles) {
        if (!tma::mbar_wait(&empty[stage], (i / kStages) & 1, error, 201)) alive = false;
        else request(i + kStages);
      }
    }
    alive = __shfl_sync(0xffffffffu, alive, 0);
    if (!alive) break;
  }
  if (!alive) return;

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const float inv0 = 1.f / l[0], inv1 = 1.f / l[1];
  const int c = (lane & 3) * 2;
  __nv_bfloat16* o0 = out + ((long long)(row0 + r0) * heads + h) * D;
  __nv_bfloat16* o1 = out + ((long long)(row0 + r1) * heads + h) * D;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    if (r0 < rows)
      *reinterpret_cast<uint32_t*>(o0 + nt * 8 + c) = mma::pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
    if (r1 < rows)
      *reinterpret_cast<uint32_t*>(o1 + nt * 8 + c) = mma::pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
  }
}

__device__ int g_error;

template <int D>
int launch(const CUtensorMap* k_map, const CUtensorMap* v_map, const __nv_bfloat16* q,
           long long q_stride, __nv_bfloat16* out, const int4* q_tiles, int n_tiles,
           const int32_t* seq_lens, const int32_t* block_table, int max_blocks, int heads,
           int kv_heads, float scale, int window, cudaStream_t stream) {
  static PerDeviceOnce configured;      // (attributes are per device)
  int* error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  if (configured.needs()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<D>::kBytes);
    if (e == cudaSuccess)      // all of the SM's memory as shared memory: two blocks fit
      e = cudaFuncSetAttribute(prefill_attention_kernel<D>,
                               cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.done();
  }
  const dim3 grid(n_tiles, heads);
  prefill_attention_kernel<D><<<grid, kThreads, Smem<D>::kBytes, stream>>>(
      *k_map, *v_map, q, q_stride, out, q_tiles, seq_lens, block_table, max_blocks, heads,
      kv_heads, scale * 1.4426950408889634f, window, error);
  return launch_status();
}

}  // namespace

SAKV_EXPORT int sakv_prefill_attention(const void* k_map, const void* v_map, const void* q,
                                       long long q_stride, void* out, const int32_t* q_tiles,
                                       int n_tiles, const int32_t* seq_lens,
                                       const int32_t* block_table, int max_blocks, int heads,
                                       int kv_heads, int head_dim, float scale, int window,
                                       cudaStream_t stream) {
  if (n_tiles < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || max_blocks <= 0 ||
      heads > 65535 || (reinterpret_cast<uintptr_t>(q_tiles) & 15))
    return cudaErrorInvalidValue;
  if (n_tiles == 0) return 0;
#define GO(D)                                                                                 \
  return launch<D>((const CUtensorMap*)k_map, (const CUtensorMap*)v_map,                     \
                   (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,                   \
                   (const int4*)q_tiles, n_tiles, seq_lens, block_table, max_blocks, heads,  \
                   kv_heads, scale, window, stream)
  if (head_dim == 64) GO(64);
  if (head_dim == 128) GO(128);
#undef GO
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_prefill_attention_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}
