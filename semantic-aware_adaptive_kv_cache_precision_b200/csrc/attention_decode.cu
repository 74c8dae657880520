// Decode attention in bfloat16: one new token per sequence attends over its cached
// keys and values, split along the keys (flash-decoding) so that a small batch
// still fills the GPU. The splits are folded together by a second kernel, or, when the
// caller gives no scratch for partials, by the split blocks themselves as one thread-block
// cluster, through distributed shared memory.
//
//   grid  = (splits, kv_heads, sequences); block = 4 warps (registers are handed out four
//   warps at a time, so a fifth warp for the copies would halve the occupancy; lane 0 of
//   warp 0 issues the copies between its tiles instead)
//   tile  = one cache block: 64 keys x head_dim, fetched by TMA (128-byte swizzle)
//           into a ring of shared-memory stages guarded by full/empty mbarriers
//   warp w of a block takes keys 16w..16w+15 of every tile for ALL query heads of
//   the KV head's group (rows of an m16n8k16 tensor-core product), keeps its own
//   running maximum, sum and output, and the four warps are merged at the end.
//
// Scores, maximum, exp2, sums and the output accumulate in fp32; probabilities
// are rounded to bf16 for the P.V product, as keys and values are stored. The
// reference's decode shape is one block per KV group with split runs of keys
// folded by `combine_kernel` (`src/core_kernels/attention.cu:754-815, 878-950`).
#include "common.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace {

constexpr int KT = kCacheBlock;      // keys per tile
constexpr int kComputeWarps = 4;
constexpr int kThreads = kComputeWarps * 32;
constexpr int kStages = 3;

template <int D>
struct Smem {
  static constexpr int kBoxes = D / 64;               // 64-wide boxes per row of head_dim
  static constexpr int kTileBytes = KT * D * 2;       // one K or V tile
  static constexpr int kStageBytes = 2 * kTileBytes;  // K then V
  static constexpr int kBytes = kStages * kStageBytes + 1024 /* alignment */ + 256;
};

// Largest cluster over which the splits of one (sequence, KV head) are folded inside the
// kernel (16 needs the opt-in to non-portable cluster sizes; the launcher asks the device).
constexpr int kMaxFoldCluster = 16;

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the shared-memory address `mine` (of this block) in the block of rank `rank` of the cluster
__device__ __forceinline__ uint32_t peer_address(uint32_t mine, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(rank));
  return remote;
}
__device__ __forceinline__ float peer_f32(uint32_t address) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ float2 peer_f32x2(uint32_t address) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];"
               : "=f"(v.x), "=f"(v.y) : "r"(address) : "memory");
  return v;
}

// kFold: the `splits` blocks of a (sequence, KV head) are one thread-block cluster (along
// blockIdx.x) and fold their partials themselves: each leaves its merged (maximum, sum,
// output) per query head in its own shared memory, the cluster synchronises, and block
// `split` finishes its share of the group's head_dim * group outputs from the peers' shared
// memory, in the order of the splits whatever its rank. No partials in global memory and no
// second kernel: one kernel boundary fewer in a decode step's chain.
template <int D, bool kFold>
__global__ void __launch_bounds__(kThreads)
decode_attention_kernel(const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map,
                        const __nv_bfloat16* __restrict__ q, long long q_stride,
                        const int32_t* __restrict__ seq_lens,
                        const int32_t* __restrict__ block_table, int max_blocks,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int heads, int kv_heads, int splits,
                        float scale_log2e, int window, int* __restrict__ error,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        int rotary_rows, __nv_bfloat16* __restrict__ k_out,
                        __nv_bfloat16* __restrict__ v_out) {
  // With `cos_t`/`sin_t` (rotary tables [positions, D / 2], rotation over the whole head) the
  // queries, keys and values in `q`'s rows are as the projection left them: this kernel
  // rotates its queries as it loads them, and the one block of a (sequence, KV head) whose
  // keys include the newest position rotates that key, writes it and the value into the
  // cache (`k_out`, `v_out`: the cache entry; null when another layer owns the entry) and
  // into its own tile. The position kernel that would do this, and the wait for it, are
  // saved.
  using S = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty = full + kStages;

  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int group = heads / kv_heads;       // query heads per KV head (<= 16 here)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  let_next_kernel_start();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tma::mbar_init(&full[s], 1);
      tma::mbar_init(&empty[s], kComputeWarps);
    }
    tma::fence_barrier_init();
    tma::prefetch_map(&k_map);
    tma::prefetch_map(&v_map);
  }
  // The lengths and block lists are the step's inputs, written before its first kernel
  // started, and every cached key but the newest was written by an earlier step: all of
  // that is read, and those tiles are on their way, before this kernel waits for the one
  // before it, which wrote the queries and the newest key and value.
  // (a length outside [0, max_blocks * 64] cannot come from the engine; a caller of the
  // exported function that passes one gets zeros for that sequence, not a wild read)
  const int given_len = seq_lens[b];
  const int kv_len = given_len < 0 || given_len > max_blocks * KT ? 0 : given_len;
  const int first_key = (window > 0 && kv_len - window > 0) ? kv_len - window : 0;
  const int first_tile = first_key / KT;
  const int n_tiles = (kv_len + KT - 1) / KT;
  const int count = n_tiles - first_tile;
  const int per_split = (count + splits - 1) / splits;
  const int t0 = first_tile + split * per_split;
  const int t1 = min(n_tiles, t0 + per_split);

  // Tile i of this split goes to stage i % kStages. Lane 0 of warp 0 keeps the ring full:
  // kStages tiles to begin with, then tile i + kStages once every warp has let go of tile i.
  // (The cache blocks of the split's first kListed tiles are fetched once, by a thread each,
  // before the wait: a request between two tiles then finds its block in shared memory
  // instead of paying a trip to global memory in the middle of the loop.)
  constexpr int kListed = kThreads;
  __shared__ int listed[kListed];
  auto request = [&](int i, bool from_list) {
    const int stage = i % kStages;
    const int block = from_list && i < kListed ? listed[i]
                                               : block_table[(long long)b * max_blocks + t0 + i];
    const int row0 = (block * kv_heads + g) * KT;
    uint8_t* dst = smem + stage * S::kStageBytes;
    tma::mbar_expect_tx(&full[stage], S::kStageBytes);
    for (int x = 0; x < S::kBoxes; ++x) {
      tma::load_2d(dst + x * (KT * 128), &k_map, x * 64, row0, &full[stage]);
      tma::load_2d(dst + S::kTileBytes + x * (KT * 128), &v_map, x * 64, row0, &full[stage]);
    }
  };
  const int n_key_tiles = max(t1 - t0, 0);
  const int newest = n_tiles - 1 - t0;         // the tile that holds the newest key, if in this split
  // (when this kernel itself writes the newest key, nobody before it does: every tile early)
  const bool fused = cos_t != nullptr;
  const bool writes = fused && k_out != nullptr && newest >= 0 && newest < n_key_tiles &&
                      kv_len > 0 && kv_len - 1 < rotary_rows;
  if (threadIdx.x == 0)
    for (int i = 0; i < min(kStages, n_key_tiles); ++i)
      if (i != newest || (fused && k_out != nullptr)) request(i, false);
  if (threadIdx.x < n_key_tiles)
    listed[threadIdx.x] = block_table[(long long)b * max_blocks + t0 + threadIdx.x];
  // rotary factors of this sequence's newest position, for the columns this lane holds
  // (clamped into the tables: a position they do not hold is the caller's fault, but is not
  // read from beyond them)
  const int pos = min(max(kv_len - 1, 0), max(rotary_rows - 1, 0));
  constexpr int HS = D / 32;                     // k-steps of 16 in half a head
  float2 cs[HS][2], sn[HS][2];
  if (fused) {
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < HS; ++ks) {
      cs[ks][0] = *reinterpret_cast<const float2*>(cos_t + (long long)pos * (D / 2) + ks * 16 + c);
      cs[ks][1] = *reinterpret_cast<const float2*>(cos_t + (long long)pos * (D / 2) + ks * 16 + c + 8);
      sn[ks][0] = *reinterpret_cast<const float2*>(sin_t + (long long)pos * (D / 2) + ks * 16 + c);
      sn[ks][1] = *reinterpret_cast<const float2*>(sin_t + (long long)pos * (D / 2) + ks * 16 + c + 8);
    }
  }
  wait_for_previous_kernel();
  if (threadIdx.x == 0 && !(fused && k_out != nullptr) && newest >= 0 &&
      newest < min(kStages, n_key_tiles))
    request(newest, false);
  __syncthreads();

  // The newest key and value, by the warp whose 16 keys of the tile include its row: lanes
  // 0 .. D/16-1 take 8 sizes of the key's first half and their partners in the second, rotate
  // them and keep both pieces; lanes 16 .. 16+D/8-1 take 8 sizes of the value.
  const int new_row = pos % KT;
  const bool patcher = writes && warp == new_row / 16;
  uint4 piece_a = make_uint4(0, 0, 0, 0), piece_b = piece_a;
  if (patcher) {
    const __nv_bfloat16* kv = q + (long long)b * q_stride + (long long)heads * D;
    if (lane < D / 16) {
      const __nv_bfloat16* src = kv + (long long)g * D + lane * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(src);
      const uint4 bb = *reinterpret_cast<const uint4*>(src + D / 2);
      const float* ct = cos_t + (long long)pos * (D / 2) + lane * 8;
      const float* st = sin_t + (long long)pos * (D / 2) + lane * 8;
      const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
      const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(&bb);
      __nv_bfloat16* lo = reinterpret_cast<__nv_bfloat16*>(&piece_a);
      __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(&piece_b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x1 = __bfloat162float(ap[j]), x2 = __bfloat162float(bp[j]);
        lo[j] = __float2bfloat16_rn(x1 * ct[j] - x2 * st[j]);
        hi[j] = __float2bfloat16_rn(x2 * ct[j] + x1 * st[j]);
      }
    } else if (lane >= 16 && lane < 16 + D / 8) {
      piece_a = *reinterpret_cast<const uint4*>(kv + (long long)(kv_heads + g) * D + (lane - 16) * 8);
    }
    // into the cache, for the steps to come
    const int block = block_table[(long long)b * max_blocks + n_tiles - 1];
    const long long at = (((long long)block * kv_heads + g) * KT + new_row) * D;
    if (lane < D / 16) {
      *reinterpret_cast<uint4*>(k_out + at + lane * 8) = piece_a;
      *reinterpret_cast<uint4*>(k_out + at + D / 2 + lane * 8) = piece_b;
    } else if (lane >= 16 && lane < 16 + D / 8) {
      *reinterpret_cast<uint4*>(v_out + at + (lane - 16) * 8) = piece_a;
    }
  }

  // ---- compute warps ------------------------------------------------------------
  // Query rows of this warp's m16 tile: row r = head g*group + r, rows >= group are zero.
  uint32_t qf[D / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
    const __nv_bfloat16* qb = q + (long long)b * q_stride + (long long)g * group * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int col = ks * 16 + c;
      qf[ks][0] = r0 < group ? *reinterpret_cast<const uint32_t*>(qb + r0 * D + col) : 0u;
      qf[ks][1] = r1 < group ? *reinterpret_cast<const uint32_t*>(qb + r1 * D + col) : 0u;
      qf[ks][2] = r0 < group ? *reinterpret_cast<const uint32_t*>(qb + r0 * D + col + 8) : 0u;
      qf[ks][3] = r1 < group ? *reinterpret_cast<const uint32_t*>(qb + r1 * D + col + 8) : 0u;
    }
    if (fused) {
#pragma unroll
      for (int ks = 0; ks < HS; ++ks)
#pragma unroll
        for (int slot = 0; slot < 4; ++slot) {
          const float2 cc = cs[ks][slot >> 1], ss = sn[ks][slot >> 1];
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&qf[ks][slot]);
          const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&qf[ks + HS][slot]);
          const float2 x1 = __bfloat1622float2(a), x2 = __bfloat1622float2(bb);
          qf[ks][slot] = mma::pack_bf16(x1.x * cc.x - x2.x * ss.x, x1.y * cc.y - x2.y * ss.y);
          qf[ks + HS][slot] = mma::pack_bf16(x2.x * cc.x + x1.x * ss.x, x2.y * cc.y + x1.y * ss.y);
        }
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  bool alive = true;

  for (int t = t0, i = 0; t < t1; ++t, ++i) {
    const int stage = i % kStages;
    if (!tma::mbar_wait(&full[stage], (i / kStages) & 1, error, 102)) {
      alive = false;
      break;
    }
    if (patcher && i == newest) {
      // the copy brought the row as the cache held it; this warp alone reads it
      uint8_t* kt = smem + stage * S::kStageBytes;
      uint8_t* vt = kt + S::kTileBytes;
      if (lane < D / 16) {
        const int d0 = lane * 8, d1 = D / 2 + lane * 8;
        *reinterpret_cast<uint4*>(kt + (d0 >> 6) * (KT * 128) + new_row * 128 +
                                  ((((d0 & 63) >> 3) ^ (new_row & 7)) << 4)) = piece_a;
        *reinterpret_cast<uint4*>(kt + (d1 >> 6) * (KT * 128) + new_row * 128 +
                                  ((((d1 & 63) >> 3) ^ (new_row & 7)) << 4)) = piece_b;
      } else if (lane >= 16 && lane < 16 + D / 8) {
        const int d0 = (lane - 16) * 8;
        *reinterpret_cast<uint4*>(vt + (d0 >> 6) * (KT * 128) + new_row * 128 +
                                  ((((d0 & 63) >> 3) ^ (new_row & 7)) << 4)) = piece_a;
      }
      __syncwarp();
    }
    const uint32_t kbase = tma::smem_u32(smem + stage * S::kStageBytes);
    const uint32_t vbase = kbase + S::kTileBytes;
    const int key0 = t * KT + warp * 16;            // this warp's first key of the tile
    const int valid = kv_len - key0;                 // keys of this warp that exist
    if (valid < 16) {
      // Rows past the sequence's end hold whatever the block held before: zero this
      // warp's own value rows there, so that 0 * garbage cannot become NaN.
      uint8_t* vt = smem + stage * S::kStageBytes + S::kTileBytes;
      for (int r = max(valid, 0); r < 16; ++r)
        for (int x = 0; x < S::kBoxes; ++x)
          reinterpret_cast<uint32_t*>(vt + x * (KT * 128) + (warp * 16 + r) * 128)[lane] = 0u;
      __syncwarp();
    }
    // S = Q K^T for 16 keys: two n-tiles of 8 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);   // key row this lane addresses
      const int half = (lane >> 3) & 1;                              // dims 0-7 or 8-15 of the k-step
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int chunk = ks * 2 + half;                             // 16-byte chunk along head_dim
        uint32_t b0, b1, b2, b3;
        mma::ldmatrix_x4(mma::swizzled(kbase + (chunk >> 3) * (KT * 128), row, chunk & 7), b0, b1,
                         b2, b3);
        mma::bf16_16816(s[0], qf[ks], b0, b1);
        mma::bf16_16816(s[1], qf[ks], b2, b3);
      }
    }
    // scale, mask, running maximum and sum (rows lane/4 and lane/4 + 8)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = key < kv_len && key >= first_key;
        s[nt][e] = seen ? s[nt][e] * scale_log2e : -INFINITY;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[nt][e]);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m[r], tile_max[r]);
      corr[r] = (m_new == -INFINITY) ? 1.f : exp2f(m[r] - m_new);
      m[r] = m_new;
      l[r] *= corr[r];
    }
    uint32_t pf[4];
    {
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          p[nt][e] = (m[r] == -INFINITY) ? 0.f : exp2f(s[nt][e] - m[r]);
          l[r] += p[nt][e];
        }
      pf[0] = mma::pack_bf16(p[0][0], p[0][1]);
      pf[1] = mma::pack_bf16(p[0][2], p[0][3]);
      pf[2] = mma::pack_bf16(p[1][0], p[1][1]);
      pf[3] = mma::pack_bf16(p[1][2], p[1][3]);
    }
    // O = O * corr + P V
    {
      const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);   // key row
      const int half = lane >> 4;                                           // dims 0-7 / 8-15
#pragma unroll
      for (int j = 0; j < D / 16; ++j) {
        o[2 * j][0] *= corr[0]; o[2 * j][1] *= corr[0]; o[2 * j][2] *= corr[1]; o[2 * j][3] *= corr[1];
        o[2 * j + 1][0] *= corr[0]; o[2 * j + 1][1] *= corr[0];
        o[2 * j + 1][2] *= corr[1]; o[2 * j + 1][3] *= corr[1];
        const int chunk = j * 2 + half;
        uint32_t b0, b1, b2, b3;
        mma::ldmatrix_x4_trans(mma::swizzled(vbase + (chunk >> 3) * (KT * 128), row, chunk & 7),
                               b0, b1, b2, b3);
        mma::bf16_16816(o[2 * j], pf, b0, b1);
        mma::bf16_16816(o[2 * j + 1], pf, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) {
      tma::mbar_arrive(&empty[stage]);
      if (warp == 0 && i + kStages < n_key_tiles) {
        if (!tma::mbar_wait(&empty[stage], (i / kStages) & 1, error, 101)) alive = false;
        else request(i + kStages, true);
      }
    }
    alive = __shfl_sync(0xffffffffu, alive, 0);
    if (!alive) break;
  }

  // ---- merge the four warps through shared memory ------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32));   // every tile has been consumed
  constexpr int kRow = D + 8;       // padded: the eight rows a warp stores at once miss each other's banks
  float* sm_o = reinterpret_cast<float*>(smem);                // [warp][16][kRow]
  float* sm_m = sm_o + kComputeWarps * 16 * kRow;              // [warp][16]
  float* sm_l = sm_m + kComputeWarps * 16;
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      float* row0 = sm_o + (warp * 16 + r0) * kRow + nt * 8 + c;
      float* row1 = row0 + 8 * kRow;
      *reinterpret_cast<float2*>(row0) = make_float2(o[nt][0], o[nt][1]);
      *reinterpret_cast<float2*>(row1) = make_float2(o[nt][2], o[nt][3]);
    }
    if ((lane & 3) == 0) {
      sm_m[warp * 16 + r0] = m[0]; sm_m[warp * 16 + r0 + 8] = m[1];
      sm_l[warp * 16 + r0] = l[0]; sm_l[warp * 16 + r0 + 8] = l[1];
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32));
  if (!kFold && !alive) return;
  // (a block of a folding cluster stays for the cluster's barriers whatever happened to it;
  // what it leaves then counts for nothing: maximum -inf, sum 0)
  float* fold_o = sm_l + kComputeWarps * 16;                   // [group][D]   (kFold)
  float2* fold_ml = reinterpret_cast<float2*>(fold_o + 16 * D);   // [group]
  // a warp takes query heads warp, warp + 4, ...; a lane four sizes of the head: one 16-byte
  // read per warp's share of a row, one 16-byte (bf16: 8-byte) store
#pragma unroll 2
  for (int r = warp; r < group; r += kComputeWarps) {
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w) big = fmaxf(big, sm_m[w * 16 + r]);
    float weight[kComputeWarps], total = 0.f;
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w) {
      weight[w] = (sm_m[w * 16 + r] == -INFINITY) ? 0.f : exp2f(sm_m[w * 16 + r] - big);
      total += weight[w] * sm_l[w * 16 + r];
    }
    if (kFold && !alive) {
      big = -INFINITY;
      total = 0.f;
    }
    const int h = g * group + r;
    if (lane < D / 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(sm_o + (w * 16 + r) * kRow + lane * 4);
        acc.x += weight[w] * v.x; acc.y += weight[w] * v.y;
        acc.z += weight[w] * v.z; acc.w += weight[w] * v.w;
      }
      if (kFold) {
        if (!alive) acc = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(fold_o + r * D + lane * 4) = acc;
      } else if (splits == 1) {
        const float inv = total > 0.f ? 1.f / total : 0.f;      // no key at all: zeros
        *reinterpret_cast<uint2*>(out + ((long long)b * heads + h) * D + lane * 4) =
            make_uint2(mma::pack_bf16(acc.x * inv, acc.y * inv),
                       mma::pack_bf16(acc.z * inv, acc.w * inv));
      } else {
        *reinterpret_cast<float4*>(part_o + (((long long)b * heads + h) * splits + split) * D +
                                   lane * 4) = acc;
      }
    }
    if (kFold) {
      if (lane == 0) fold_ml[r] = make_float2(big, total);
    } else if (splits > 1 && lane == 0) {
      float* ml = part_ml + (((long long)b * heads + h) * splits + split) * 2;
      ml[0] = big;
      ml[1] = total;
    }
  }
  if (kFold) {
    cluster_sync_all();          // every block's (maximum, sum, output) lies in its shared memory
    // The group's outputs are one row of group * D elements (head r, size), dealt to the
    // blocks in equal runs. A thread takes one element of its block's run at a time and
    // reads the splits' maxima, sums and outputs eight at a time, all loads of a round in
    // flight together; rounds are merged like tiles of an online softmax, in order.
    const int elements = group * D;
    const int run = (elements + splits - 1) / splits;
    const int e_end = min(elements, (split + 1) * run);
    constexpr int kRound = 8;
    for (int e = split * run + threadIdx.x; e < e_end; e += kThreads) {
      const int r = e / D;
      const uint32_t ml_at = tma::smem_u32(fold_ml + r), o_at = tma::smem_u32(fold_o + e);
      float big = -INFINITY, total = 0.f, acc = 0.f;
      for (int s0 = 0; s0 < splits; s0 += kRound) {
        float2 v[kRound];
        float o_s[kRound];
#pragma unroll
        for (int j = 0; j < kRound; ++j) {
          const bool live = s0 + j < splits;
          const int rank = live ? s0 + j : 0;
          v[j] = live ? peer_f32x2(peer_address(ml_at, rank)) : make_float2(-INFINITY, 0.f);
          o_s[j] = live ? peer_f32(peer_address(o_at, rank)) : 0.f;
        }
        float round_max = big;
#pragma unroll
        for (int j = 0; j < kRound; ++j) round_max = fmaxf(round_max, v[j].x);
        if (round_max == -INFINITY) continue;
        const float keep = exp2f(big - round_max);          // 0 the first time
        total *= keep;
        acc *= keep;
        big = round_max;
#pragma unroll
        for (int j = 0; j < kRound; ++j) {
          const float w = exp2f(v[j].x - big);              // 0 for a split that saw no key
          total += w * v[j].y;
          acc += w * o_s[j];
        }
      }
      out[((long long)b * heads + g * group) * D + e] =
          __float2bfloat16_rn(total > 0.f ? acc / total : 0.f);
    }
    cluster_sync_all();          // nobody leaves while a peer may still read its shared memory
  }
}

// out[b, h, :] = sum_s w_s o_s / sum_s w_s l_s with w_s = exp2(m_s - max m). The splits are
// taken sixteen at a time, with all of a round's loads (maxima, sums, outputs) in flight
// together, and rounds are merged like tiles of an online softmax: up to 16 splits cost one
// memory round trip.
__global__ void combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               __nv_bfloat16* __restrict__ out, int splits, int head_dim) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  constexpr int kRound = 16;
  const long long bh = blockIdx.x;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + bh * splits;
  for (int dim = threadIdx.x; dim < head_dim; dim += blockDim.x) {
    float big = -INFINITY, total = 0.f, acc = 0.f;
    for (int s0 = 0; s0 < splits; s0 += kRound) {
      float2 v[kRound];
      float o[kRound];
#pragma unroll
      for (int j = 0; j < kRound; ++j) {
        const bool live = s0 + j < splits;
        v[j] = live ? ml[s0 + j] : make_float2(-INFINITY, 0.f);
        o[j] = live ? part_o[(bh * splits + s0 + j) * head_dim + dim] : 0.f;
      }
      float round_max = big;
#pragma unroll
      for (int j = 0; j < kRound; ++j) round_max = fmaxf(round_max, v[j].x);
      if (round_max == -INFINITY) continue;
      const float keep = exp2f(big - round_max);          // 0 the first time
      total *= keep;
      acc *= keep;
      big = round_max;
#pragma unroll
      for (int j = 0; j < kRound; ++j) {
        const float w = exp2f(v[j].x - big);              // 0 for a split that saw no key
        total += w * v[j].y;
        acc += w * o[j];
      }
    }
    out[bh * head_dim + dim] = __float2bfloat16_rn(total > 0.f ? acc / total : 0.f);
  }
}

// The same for more than 16 splits (one sequence, or few): the block has several groups of
// `head_dim` threads (`blockDim.x = groups * head_dim`, at most kFoldGroups); group j takes
// rounds j, j + groups, ..., so that up to 64 splits still cost one round trip, and group 0
// merges the groups' results through shared memory, always in the order of the groups.
// (Kept apart from the kernel above: with both in one, the decode step at 8 sequences, which
// has one group, was 1.5 % slower.)
constexpr int kFoldGroups = 4;
__global__ void combine_groups_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               __nv_bfloat16* __restrict__ out, int splits, int head_dim) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  constexpr int kRound = 16;
  extern __shared__ float3 merged[];      // [groups - 1][head_dim]; nothing for one group
  const long long bh = blockIdx.x;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + bh * splits;
  const int groups = blockDim.x / head_dim, group = threadIdx.x / head_dim;
  const int dim = threadIdx.x - group * head_dim;
  float big = -INFINITY, total = 0.f, acc = 0.f;
  for (int s0 = group * kRound; s0 < splits; s0 += groups * kRound) {
    float2 v[kRound];
    float o[kRound];
#pragma unroll
    for (int j = 0; j < kRound; ++j) {
      const bool live = s0 + j < splits;
      v[j] = live ? ml[s0 + j] : make_float2(-INFINITY, 0.f);
      o[j] = live ? part_o[(bh * splits + s0 + j) * head_dim + dim] : 0.f;
    }
    float round_max = big;
#pragma unroll
    for (int j = 0; j < kRound; ++j) round_max = fmaxf(round_max, v[j].x);
    if (round_max == -INFINITY) continue;
    const float keep = exp2f(big - round_max);          // 0 the first time
    total *= keep;
    acc *= keep;
    big = round_max;
#pragma unroll
    for (int j = 0; j < kRound; ++j) {
      const float w = exp2f(v[j].x - big);              // 0 for a split that saw no key
      total += w * v[j].y;
      acc += w * o[j];
    }
  }
  if (groups > 1) {
    if (group > 0) merged[(group - 1) * head_dim + dim] = make_float3(big, total, acc);
    __syncthreads();
    if (group > 0) return;
    for (int j = 0; j < groups - 1; ++j) {
      const float3 other = merged[j * head_dim + dim];
      const float top = fmaxf(big, other.x);
      if (top == -INFINITY) continue;
      const float mine = exp2f(big - top), theirs = exp2f(other.x - top);
      total = total * mine + other.y * theirs;
      acc = acc * mine + other.z * theirs;
      big = top;
    }
  }
  out[bh * head_dim + dim] = __float2bfloat16_rn(total > 0.f ? acc / total : 0.f);
}

__device__ int g_error;

// The largest cluster the folding kernel can be launched with on this device: 16 where the
// opt-in to non-portable sizes is granted and such a cluster fits, else 8 (0: none).
template <int D>
int max_fold_cluster() {
  static int known[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (known[device]) return known[device] - 1;
  auto kernel = decode_attention_kernel<D, true>;
  int best = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::kBytes) ==
      cudaSuccess) {
    const bool wide = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed,
                                           1) == cudaSuccess;
    for (int size : {16, 8}) {
      if (size > 8 && !wide) continue;
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(size, 1, 1);
      config.blockDim = dim3(kThreads);
      config.dynamicSmemBytes = Smem<D>::kBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = size;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      config.attrs = attr;
      config.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) == cudaSuccess && clusters > 0) {
        best = size;
        break;
      }
    }
    cudaGetLastError();      // (a refused size is an answer, not an error to keep)
  }
  known[device] = best + 1;
  return best;
}

// `part_o == nullptr` with more than one split: the splits fold themselves as a cluster.
template <int D>
int launch(const CUtensorMap* k_map, const CUtensorMap* v_map, const __nv_bfloat16* q,
           long long q_stride, const int32_t* seq_lens, const int32_t* block_table, int max_blocks,
           __nv_bfloat16* out, float* part_o, float* part_ml, int sequences, int heads,
           int kv_heads, int splits, float scale, int window, const float* cos_t,
           const float* sin_t, int rotary_rows, __nv_bfloat16* k_out, __nv_bfloat16* v_out,
           cudaStream_t stream) {
  static PerDeviceOnce configured;      // (attributes are per device)
  int* error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  if (configured.needs()) {
    cudaError_t e = cudaSuccess;
    for (int fold = 0; fold < 2 && e == cudaSuccess; ++fold) {
      const void* kernel = fold ? (const void*)decode_attention_kernel<D, true>
                                : (const void*)decode_attention_kernel<D, false>;
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Smem<D>::kBytes);
      if (e == cudaSuccess)      // all of the SM's memory as shared memory: two blocks fit
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
    }
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.done();
  }
  const dim3 grid(splits, kv_heads, sequences);
  if (splits > 1 && part_o == nullptr) {
    if (splits > max_fold_cluster<D>()) return cudaErrorInvalidValue;
    return launch_overlapped_cluster(decode_attention_kernel<D, true>, grid, dim3(kThreads),
                                     Smem<D>::kBytes, stream, dim3(splits, 1, 1), *k_map, *v_map,
                                     q, q_stride, seq_lens, block_table, max_blocks, out, part_o,
                                     part_ml, heads, kv_heads, splits,
                                     scale * 1.4426950408889634f, window, error, cos_t, sin_t,
                                     rotary_rows, k_out, v_out);
  }
  int status = launch_overlapped(decode_attention_kernel<D, false>, grid, dim3(kThreads),
                                 Smem<D>::kBytes, stream, 1, *k_map, *v_map, q, q_stride,
                                 seq_lens, block_table, max_blocks, out, part_o, part_ml, heads,
                                 kv_heads, splits, scale * 1.4426950408889634f, window, error,
                                 cos_t, sin_t, rotary_rows, k_out, v_out);
  const int fold_groups = min(kFoldGroups, (splits + 15) / 16);
  if (status == 0 && splits > 1 && fold_groups == 1)
    status = launch_overlapped(combine_kernel, dim3(sequences * heads), dim3(D <= 128 ? D : 128),
                               0, stream, 1, (const float*)part_o, (const float*)part_ml, out,
                               splits, D);
  else if (status == 0 && splits > 1)
    status = launch_overlapped(combine_groups_kernel, dim3(sequences * heads),
                               dim3(D * fold_groups), (fold_groups - 1) * D * sizeof(float3),
                               stream, 1, (const float*)part_o, (const float*)part_ml, out,
                               splits, D);
  return status;
}

}  // namespace

// A tensor map over one cache entry [blocks, kv_heads, 64, head_dim] seen as rows of
// head_dim, read in boxes of 64 rows x 64 columns. `map` points to 128 bytes on the host.
SAKV_EXPORT int sakv_decode_attention_map(void* map, const void* cache, long long blocks,
                                          int kv_heads, int head_dim) {
  if (blocks <= 0 || kv_heads <= 0 || head_dim % 64) return cudaErrorInvalidValue;
  return tma::make_map_bf16_2d(reinterpret_cast<CUtensorMap*>(map), cache,
                               (uint64_t)blocks * kv_heads * KT, head_dim,
                               (uint64_t)head_dim * 2, KT, 64);
}

SAKV_EXPORT int sakv_decode_attention(const void* k_map, const void* v_map, const void* q,
                                      long long q_stride, const int32_t* seq_lens,
                                      const int32_t* block_table, int max_blocks, void* out,
                                      float* part_o, float* part_ml, int sequences, int heads,
                                      int kv_heads, int head_dim, int splits, float scale,
                                      int window, const float* cos_table, const float* sin_table,
                                      int rotary_rows, void* k_cache, void* v_cache,
                                      cudaStream_t stream) {
  // `cos_table`, `sin_table` (fp32 [rotary_rows, head_dim / 2], both or neither): `q`'s rows are
  // then the projection's whole output [q | k | v], unrotated, and the kernel rotates the
  // queries and, into the cache entry `k_cache`, `v_cache` (or nowhere if those are null),
  // writes the newest position's rotated key and its value.
  if ((cos_table == nullptr) != (sin_table == nullptr) || (k_cache == nullptr) != (v_cache == nullptr) ||
      (k_cache && !cos_table) || (cos_table && rotary_rows <= 0) || ((uintptr_t)cos_table & 7) || ((uintptr_t)sin_table & 7) ||
      ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
      (cos_table && (((uintptr_t)q & 15) || (q_stride & 7))))
    return cudaErrorInvalidValue;
  if (sequences < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16 ||
      splits < 1 || max_blocks <= 0 || (part_o == nullptr) != (part_ml == nullptr) ||
      (reinterpret_cast<uintptr_t>(part_ml) & 7))
    return cudaErrorInvalidValue;
  if (sequences == 0) return 0;
  if (sequences > 65535 || kv_heads > 65535) return cudaErrorInvalidValue;
#define GO(D)                                                                                  \
  return launch<D>((const CUtensorMap*)k_map, (const CUtensorMap*)v_map,                      \
                   (const __nv_bfloat16*)q, q_stride, seq_lens, block_table, max_blocks,      \
                   (__nv_bfloat16*)out, part_o, part_ml, sequences, heads, kv_heads, splits,  \
                   scale, window, cos_table, sin_table, rotary_rows, (__nv_bfloat16*)k_cache, \
                   (__nv_bfloat16*)v_cache, stream)
  if (head_dim == 64) GO(64);
  if (head_dim == 128) GO(128);
#undef GO
  return cudaErrorInvalidValue;
}

// How many splits the kernel can fold by itself, as one thread-block cluster (16 or 8; 0 if
// the head size is not served). More splits need `part_o`, `part_ml` and the fold kernel.
SAKV_EXPORT int sakv_decode_attention_max_cluster(int head_dim) {
  if (head_dim == 64) return max_fold_cluster<64>();
  if (head_dim == 128) return max_fold_cluster<128>();
  return 0;
}

// The error word that a timed-out wait leaves (0 = none); reading it synchronises.
SAKV_EXPORT int sakv_decode_attention_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}

// ---- the same kernels for callers that cannot allocate (see attention_decode_static.h) ----
#include "attention_decode_static.h"
#include <stdio.h>

namespace {

// Scratch for the split partials, inside the library. In host code this name is only
// a stand-in for the symbol: the device address must be asked for.
static __device__ __align__(256) float g_static_scratch[SAKV_DECODE_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_scratch_address[kMaxDevices];   // per device, looked up at its first call

void say(char* why, int why_len, const char* text) {
  if (why && why_len > 0) snprintf(why, static_cast<size_t>(why_len), "%s", text);
}

}  // namespace

SAKV_EXPORT int sakv_decode_attention_static_scratch(
    const void* k_map, const void* v_map, const void* q, long long q_stride,
    const int32_t* seq_lens, const int32_t* block_table, int max_blocks, void* out, int sequences,
    int heads, int kv_heads, int head_dim, int splits, float scale, int window, char* why,
    int why_len, cudaStream_t stream) {
  if (sequences < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16 ||
      splits < 1 || max_blocks <= 0 || (head_dim != 64 && head_dim != 128) || sequences > 65535) {
    say(why, why_len, "decode attention: a size is outside what the kernel takes (head_dim 64 or "
                      "128, at most 16 query heads per KV head, at least one split)");
    return cudaErrorInvalidValue;
  }
  const long long need = (long long)sequences * heads * splits * (head_dim + 2);
  if (need > SAKV_DECODE_STATIC_SCRATCH_FLOATS) {
    if (why && why_len > 0)
      snprintf(why, static_cast<size_t>(why_len),
               "decode attention without allocation: sequences * heads * splits * (head_dim + 2) "
               "= %lld floats, the built-in scratch holds %d; use fewer splits or sequences, or "
               "the entry point that takes scratch buffers",
               need, SAKV_DECODE_STATIC_SCRATCH_FLOATS);
    return cudaErrorInvalidValue;
  }
  if (sequences == 0) return 0;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kMaxDevices) {
    say(why, why_len, "decode attention without allocation: device index beyond 63");
    return cudaErrorInvalidValue;
  }
  if (!g_static_scratch_address[device]) {
    // once per device, with that device current: the array's address on THIS device
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
    if (e != cudaSuccess || !address) {
      say(why, why_len, "decode attention without allocation: cudaGetSymbolAddress failed");
      return static_cast<int>(e != cudaSuccess ? e : cudaErrorInvalidValue);
    }
    g_static_scratch_address[device] = address;
  }
  float* part_o = g_static_scratch_address[device];
  float* part_ml = part_o + (long long)sequences * heads * splits * head_dim;
  if (head_dim == 64)
    return launch<64>((const CUtensorMap*)k_map, (const CUtensorMap*)v_map,
                      (const __nv_bfloat16*)q, q_stride, seq_lens, block_table, max_blocks,
                      (__nv_bfloat16*)out, part_o, part_ml, sequences, heads, kv_heads, splits,
                      scale, window, nullptr, nullptr, 0, nullptr, nullptr, stream);
  return launch<128>((const CUtensorMap*)k_map, (const CUtensorMap*)v_map,
                     (const __nv_bfloat16*)q, q_stride, seq_lens, block_table, max_blocks,
                     (__nv_bfloat16*)out, part_o, part_ml, sequences, heads, kv_heads, splits,
                     scale, window, nullptr, nullptr, 0, nullptr, nullptr, stream);
}
