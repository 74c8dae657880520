// The bf16 matrix product of the serving path on tcgen05 tensor cores:
//
//   C[m, n] = sum_k X[m, k] W[n, k]   (+ bias[n])        X: [M, K] activations, bf16
//                                                          W: [N, K] weights as stored, bf16
// computed "weights on the rows": a block owns 128 rows of W (the M dimension of a
// 128 x MT x 16 tcgen05.mma) and up to MT tokens (its N dimension, 16..256), so a
// decode step with a handful of tokens still streams every weight through full-width
// tensor-core instructions. Both operands are K-major tiles of 64 columns that TMA
// drops into shared memory with the 128-byte swizzle; a ring of stages guarded by
// full/empty mbarriers keeps many tiles in flight; the fp32 accumulator lives in
// tensor memory (one weight row per lane, one token per column), is read back with
// tcgen05.ld and finished in registers:
//
//   out_bf16 / out_f32 : C (+ bias)                    QKV projection, LM head
//   accumulate_f32     : R[m, n] += C                  o_proj and down_proj into the residual
//   gated_silu         : silu(C_gate) * C_up           gate and up rows [n] and [n + I] of one
//                                                      matrix, two accumulators side by side
//
// With few tokens and a small N there are too few row tiles to fill the GPU's SMs, so K is
// split over the blocks of a thread-block cluster (up to 8, along blockIdx.z): every
// block leaves its partial tile in its own shared memory, the cluster synchronises,
// and each block then finishes a share of the token columns by adding the partials of
// all blocks in rank order (the same order every time) through distributed shared
// memory. Nothing goes through global scratch. The reference calls cuBLAS for all of
// this (`src/core_kernels/linear.cu:85-142`); warps: 0 = TMA, 1 = MMA issue (the ring's even
// stages) and tensor memory, 6 = MMA issue (the odd stages, into an accumulator of its own),
// 2..5 = epilogue. TMA loads are plain per-block loads, never cluster multicast.
#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int BM = 128;          // weight rows per block (MMA M)
constexpr int BK = 64;           // columns per stage (one 128-byte swizzle row)
constexpr int kThreads = 224;      // warps: 0 TMA, 1 and 6 MMA issue, 2..5 epilogue
constexpr int kWTile = BM * BK * 2;
constexpr int kMaxSplits = 8;     // portable cluster size

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_ACCUM = 2, EPI_GATED = 3 };

struct Params {
  int M, N, K;
  int splits, kb_per_split;
  int parts;             // independent K ranges, each leaving a sum of its own (EPI_F32 only)
  long long part_stride; // elements from one part's [M, ldo] result to the next
  int stages;            // tiles in flight per block (ring of shared-memory stages)
  int dual_offset;       // row of W where the "up" half starts (gated_silu)
  int epi;
  const void* bias;      // [N] or null
  int bias_dtype;
  void* out;             // [M, ldo]
  long long ldo;
  int* error;
};

template <int MT, bool kDual>
struct Cfg {
  static constexpr int kXTile = MT * BK * 2;
  static constexpr int kStageBytes = (kDual ? 2 : 1) * kWTile + kXTile;
  static constexpr int kMaxStages = 10;
  static constexpr int kAcc = (kDual ? 2 : 1) * MT;
  static constexpr int kPartialBytes = kAcc * BM * 4;     // the split partial reuses the stages
  // With one block per SM (a grid that fits the GPU in one wave) a block takes as many
  // stages as fit, to keep enough bytes in flight; with several waves it takes fewer, so
  // that two or three blocks share an SM and one's epilogue overlaps another's streaming.
  static int stages_for(long long blocks) {
    const int sms = sm_count();
    const int budget = blocks <= sms ? 200 * 1024
                       : MT <= 32 ? (kDual ? 104 : 72) * 1024
                       : MT == 64 ? (kDual ? 160 : 100) * 1024 : 200 * 1024;
    int s = budget / kStageBytes;
    // (an even ring gives the two MMA lanes, which own the even and the odd stages, equal shares)
    if (blocks <= sms && (s & 1) && smem_bytes(s + 1) <= 227 * 1024) ++s;
    if (s > kMaxStages) s = kMaxStages;
    while (s * kStageBytes < kPartialBytes) ++s;
    return s < 2 ? 2 : s;
  }
  static int smem_bytes(int stages) { return stages * kStageBytes + 1024 + 256; }
  // two accumulators of kAcc columns: the K steps go to them in turn (see the MMA lanes)
  static constexpr int kTmemCols = 2 * kAcc <= 32 ? 32 : 2 * kAcc <= 64 ? 64 : 2 * kAcc <= 128 ? 128
                                   : 2 * kAcc <= 256 ? 256 : 512;
};

__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();      // the single-lane roles of warps 0 and 1 have to be back with their warps
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The value at shared-memory address `local` (of this block's window) in the block of
// rank `rank` of the cluster.
__device__ __forceinline__ float ld_peer(uint32_t local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float bias_at(const Params& p, int n) {
  if (!p.bias || n >= p.N) return 0.f;
  return p.bias_dtype == SAKV_F32 ? reinterpret_cast<const float*>(p.bias)[n]
                                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
}

// (the epilogue's kind is a template argument: the choice is made once, not per element)
template <int kEpi>
__device__ __forceinline__ void finish(const Params& p, int part, int m, int n, float c, float up,
                                       float bias) {
  if (m >= p.M || n >= p.N) return;
  const long long at = (long long)m * p.ldo + n + part * p.part_stride;
  if (kEpi == EPI_BF16) {
    reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(c + bias);
  } else if (kEpi == EPI_F32) {
    reinterpret_cast<float*>(p.out)[at] = c + bias;
  } else if (kEpi == EPI_ACCUM) {
    // one block adds to each element exactly once, so the sum is the same every time; the
    // reduction instruction spares the thread the round trip of reading the old value
    atomicAdd(reinterpret_cast<float*>(p.out) + at, c + bias);
  } else {
    const float silu = c / (1.0f + expf(-c));
    reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(silu * up);
  }
}

// The reduction of a cluster's partial tiles: this block finishes token columns `split`,
// `split + S`, ... of its 128 rows by reading every block's partial through distributed
// shared memory, four columns' worth of remote reads in flight at a time (measured in the
// decode step: 2, 8 and 16 columns at a time are all slower). The usual cluster sizes (S =
// 2, 4, 8) are compiled apart, so that the loops over the cluster unroll to its real size
// (the decode step at 8 sequences: 1.68 -> 1.61 ms); S = 0 is any other size.
template <int MT, int kEpi, int S>
__device__ __forceinline__ void reduce_columns(const Params& p, uint32_t base, int split,
                                               int k_part, int m0, int n, int row, float bias) {
  constexpr bool kDual = kEpi == EPI_GATED;
  constexpr int kS = S > 0 ? S : kMaxSplits;
  constexpr int kBatch = 4;
  const int splits = S > 0 ? S : p.splits;
  for (int c0 = split; c0 < MT && m0 + c0 < p.M; c0 += kBatch * splits) {
    float part[kBatch][kS], part_up[kDual ? kBatch : 1][kS];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int c = c0 + j * splits;
      const bool live = c < MT && m0 + c < p.M;
#pragma unroll
      for (int s = 0; s < kS; ++s) {
        part[j][s] = 0.f;
        if (kDual) part_up[j][s] = 0.f;
        if (live && s < splits) {
          part[j][s] = ld_peer(base + (c * BM + row) * 4, s);
          if (kDual) part_up[j][s] = ld_peer(base + ((MT + c) * BM + row) * 4, s);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int c = c0 + j * splits;
      if (c >= MT) break;
      float acc = 0.f, up = 0.f;
#pragma unroll
      for (int s = 0; s < kS; ++s) {
        acc += part[j][s];
        if (kDual) up += part_up[j][s];
      }
      finish<kEpi>(p, k_part, m0 + c, n, acc, up, bias);
    }
  }
}

__device__ __forceinline__ float4 ld_peer4(uint32_t local, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

// Four consecutive weight rows n .. n + 3 of one token column m, finished together.
template <int kEpi>
__device__ __forceinline__ void finish4(const Params& p, int part, int m, int n, float4 c,
                                        float4 up, float4 bias) {
  if (m >= p.M || n >= p.N) return;
  const long long at = (long long)m * p.ldo + n + part * p.part_stride;
  const bool whole = n + 3 < p.N && (p.ldo & 3) == 0 && (p.part_stride & 3) == 0;
  if (kEpi == EPI_ACCUM || !whole) {
    finish<kEpi>(p, part, m, n, c.x, up.x, bias.x);
    finish<kEpi>(p, part, m, n + 1, c.y, up.y, bias.y);
    finish<kEpi>(p, part, m, n + 2, c.z, up.z, bias.z);
    finish<kEpi>(p, part, m, n + 3, c.w, up.w, bias.w);
  } else if (kEpi == EPI_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + at) =
        make_float4(c.x + bias.x, c.y + bias.y, c.z + bias.z, c.w + bias.w);
  } else {
    float r[4] = {c.x + bias.x, c.y + bias.y, c.z + bias.z, c.w + bias.w};
    if (kEpi == EPI_GATED) {
      const float g[4] = {c.x, c.y, c.z, c.w}, u[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
    }
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + at) =
        make_uint2(mma::pack_bf16(r[0], r[1]), mma::pack_bf16(r[2], r[3]));
  }
}

// The same reduction for token tiles of 32 and more with a cluster of 2, 4 or 8, where the
// remote reads are many (at 64 tokens the scheme above spent 5.6 us of the gate/up product's
// 14.5 us in them). A thread no longer keeps to its own row: the 32 lanes of a warp take the
// 128 rows of ONE token column four rows each, so that a warp's remote read is 512
// contiguous bytes, and the four warps take four columns at a time; results leave as 8- or
// 16-byte stores of four rows. (Partials laid out row by row, so that a thread could read
// four of ITS columns at once, were slower: a warp's read was then 32 scattered pieces.)
template <int MT, int kEpi, int S>
__device__ __forceinline__ void reduce_quads(const Params& p, uint32_t base, int rank, int k_part,
                                             int m0, int n0, float4 bias) {
  constexpr bool kDual = kEpi == EPI_GATED;
  const int t = threadIdx.x - 64;                 // 0..127 among the epilogue threads
  const int r0 = (t & 31) * 4;                    // this thread's four rows (`bias`: theirs)
  const int n = n0 + r0;
  const int live = min(MT, p.M - m0);
  // as many columns a round as keep about sixteen 16-byte reads of a thread in flight
  constexpr int kAccs = kDual ? 2 : 1;
  constexpr int kIter = 16 / (S * kAccs) > 0 ? 16 / (S * kAccs) : 1;
#pragma unroll 1
  for (int c0 = rank + (t >> 5) * S; c0 < live; c0 += 4 * S * kIter) {
    float4 g[kIter][S], u[kDual ? kIter : 1][S];
#pragma unroll
    for (int k = 0; k < kIter; ++k) {
      const int c = c0 + k * 4 * S;
#pragma unroll
      for (int s = 0; s < S; ++s) {
        const bool on = c < live;
        g[k][s] = on ? ld_peer4(base + (c * BM + r0) * 4, s) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (kDual)
          u[k][s] = on ? ld_peer4(base + ((MT + c) * BM + r0) * 4, s)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int k = 0; k < kIter; ++k) {
      const int c = c0 + k * 4 * S;
      if (c >= live) break;
      float4 acc = g[k][0], up = kDual ? u[k][0] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 1; s < S; ++s) {
        acc.x += g[k][s].x; acc.y += g[k][s].y; acc.z += g[k][s].z; acc.w += g[k][s].w;
        if (kDual) { up.x += u[k][s].x; up.y += u[k][s].y; up.z += u[k][s].z; up.w += u[k][s].w; }
      }
      finish4<kEpi>(p, k_part, m0 + c, n, acc, up, bias);
    }
  }
}

template <int MT, int kEpi>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
               const Params p) {
  constexpr bool kDual = kEpi == EPI_GATED;
  using C = Cfg<MT, kDual>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const int stages = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * C::kStageBytes);
  uint64_t* empty = full + stages;
  uint64_t* accum = empty + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blockIdx.z = part * splits + split: a cluster is the `splits` blocks of one part
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  const int split = blockIdx.z % p.splits, k_part = blockIdx.z / p.splits;
  const int n0 = n_tile * BM, m0 = m_tile * MT;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int kb1 = min(total_kb, kb0 + p.kb_per_split);
  const int n_kb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tma::mbar_init(&full[s], 1);
      tma::mbar_init(&empty[s], 1);
    }
    tma::mbar_init(accum, n_kb > 1 ? 2 : 1);     // one arrival per MMA lane that has work
    tma::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, C::kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // Only now, with this block's shared and tensor memory in hand, may the next kernel's
  // blocks start to arrive: they can never hold what a block of this kernel still needs.
  let_next_kernel_start();

  // The bias is a weight: the epilogue's threads fetch theirs now, for their own row and (the
  // reduction by row quads) for the four rows they finish there, not behind the cluster's
  // barrier, where the fetch was 0.5 us of the QKV product's 4.7 us.
  float bias = 0.f;
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (warp >= 2 && warp < 6 && k_part == 0 && p.bias) {
    bias = bias_at(p, n0 + (warp & 3) * 32 + lane);
    if (MT >= 32 && p.splits > 1) {
      const int q = n0 + ((threadIdx.x - 64) & 31) * 4;
      bias4 = make_float4(bias_at(p, q), bias_at(p, q + 1), bias_at(p, q + 2), bias_at(p, q + 3));
    }
  }

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------
    if (lane == 0) {
      tma::prefetch_map(&w_map);
      tma::prefetch_map(&x_map);
      // Weights do not depend on the kernel before: the first ring of weight tiles is
      // already on its way while that kernel finishes; the activations follow the wait.
      const int ahead = min(n_kb, stages);
      for (int i = 0; i < ahead; ++i) {
        uint8_t* dst = smem + i * C::kStageBytes;
        const int x = (kb0 + i) * BK;
        tma::mbar_expect_tx(&full[i], C::kStageBytes);
        tma::load_2d(dst, &w_map, x, n0, &full[i]);
        if (kDual) tma::load_2d(dst + kWTile, &w_map, x, p.dual_offset + n0, &full[i]);
      }
      wait_for_previous_kernel();
      for (int i = 0; i < ahead; ++i)
        tma::load_2d(smem + i * C::kStageBytes + (kDual ? 2 : 1) * kWTile, &x_map,
                     (kb0 + i) * BK, m0, &full[i]);
      // (the ring's position is counted, not divided out: `stages` is a run-time number and
      // this lane's instructions are the pipeline's pace)
      int stage = ahead == stages ? 0 : ahead, phase = 0;
      for (int i = ahead; i < n_kb; ++i) {
        if (!tma::mbar_wait(&empty[stage], phase, p.error, 301)) break;
        uint8_t* dst = smem + stage * C::kStageBytes;
        const int x = (kb0 + i) * BK;
        tma::mbar_expect_tx(&full[stage], C::kStageBytes);
        tma::load_2d(dst, &w_map, x, n0, &full[stage]);
        if (kDual) tma::load_2d(dst + kWTile, &w_map, x, p.dual_offset + n0, &full[stage]);
        tma::load_2d(dst + (kDual ? 2 : 1) * kWTile, &x_map, x, m0, &full[stage]);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ---- MMA issue, by two lanes ------------------------------------------------------
    // A lane's turn costs it a barrier wait (some 300 cycles even when the tile is there),
    // its products (45 cycles each at 16 tokens, and the lane is held while they queue) and
    // a commit (75): one lane alone leaves the tensor pipe idle half of the time. So lane 0
    // of warp 1 takes the K steps that fall into the even STAGES of the ring, into one
    // accumulator, and lane 0 of warp 6 those of the odd stages, into a second; one waits
    // while the other's products run, and the epilogue adds the two accumulators, always in
    // that order.
    //
    // A stage belongs to one lane for good. (Dealing out the K steps in turn did not: with
    // an odd number of stages a lane then came to a stage whose last tile was the other
    // lane's, could get there before that tile had even landed, and a wait for the parity
    // after a phase that has not completed is true at once. The lane read a half-filled
    // tile, freed it a second time, and the ring's phases fell apart: `unspecified launch
    // failure` on the shapes with long K loops.) A lane waits for each phase of its own
    // stages in turn, so it can never be more than one phase ahead of a barrier.
    const int which = warp == 1 ? 0 : 1;
    if (lane == 0 && which < n_kb) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, MT);
      const uint32_t acc = tmem + which * C::kAcc;
      bool ok = true, fresh = true;     // fresh: this lane's accumulator holds nothing yet
      int stage = 0, phase = 0;
      for (int i = 0; i < n_kb && ok; ++i) {
        if ((stage & 1) == which) {
          ok = tma::mbar_wait(&full[stage], phase, p.error, 302);
          if (!ok) break;
          tc::fence_after_sync();
          const uint32_t a = tma::smem_u32(smem + stage * C::kStageBytes);
          const uint32_t b = a + (kDual ? 2 : 1) * kWTile;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t bd = tc::smem_desc_k_major_sw128(b + k * 32);
            tc::mma_ss(acc, tc::smem_desc_k_major_sw128(a + k * 32), bd, idesc, !fresh || k > 0);
            if (kDual)
              tc::mma_ss(acc + MT, tc::smem_desc_k_major_sw128(a + kWTile + k * 32), bd, idesc,
                         !fresh || k > 0);
          }
          fresh = false;
          tc::commit(&empty[stage]);    // the stage is free once these MMAs have read it
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      tc::commit(accum);                // this lane's accumulator is complete
    }
  } else if (warp < 6) {
    // ---- epilogue: warp w reads the lanes of quarter w % 4 ------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // lane of tensor memory = weight row in the tile
    const int n = n0 + row;
    wait_for_previous_kernel();       // before any write to global memory
    const bool ok = tma::mbar_wait(accum, 0, p.error, 303);
    tc::fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    // sixteen columns of the first lane's accumulator plus, if the second had a K step, its own
    const bool two = n_kb > 1;
    auto columns = [&](int c, float (&v)[16]) {
      tc::ld_32x32b_x16(taddr + c, v);
      if (two) {
        float w[16];
        tc::ld_32x32b_x16(taddr + C::kAcc + c, w);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += w[j];
      }
    };
    if (p.splits == 1) {
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < MT; c += 16) {
          float v[16], u[16];
          columns(c, v);
          if (kDual) columns(MT + c, u);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            finish<kEpi>(p, k_part, m0 + c + j, n, v[j], kDual ? u[j] : 0.f, bias);
        }
      }
    } else if (ok) {
      // this block's partial tile -> its own shared memory, [column][row] fp32
      float* mine = reinterpret_cast<float*>(smem);
#pragma unroll 1
      for (int c = 0; c < C::kAcc; c += 16) {
        float v[16];
        columns(c, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[(c + j) * BM + row] = v[j];
      }
    }
    tc::fence_before_sync();
  }
  if (p.splits > 1) {
    // Every thread of every block of the cluster comes here, whatever happened above.
    cluster_sync_all();
    if (warp >= 2 && warp < 6) {
      const int row = (warp & 3) * 32 + lane;
      const int n = n0 + row;
      const uint32_t base = tma::smem_u32(smem);
      // token columns split, split + splits, ... are finished by this block
      if (MT >= 32 && p.splits == 2)
        reduce_quads<MT, kEpi, 2>(p, base, split, k_part, m0, n0, bias4);
      else if (MT >= 32 && p.splits == 4)
        reduce_quads<MT, kEpi, 4>(p, base, split, k_part, m0, n0, bias4);
      else if (MT >= 32 && p.splits == 8)
        reduce_quads<MT, kEpi, 8>(p, base, split, k_part, m0, n0, bias4);
      else if (p.splits == 2)
        reduce_columns<MT, kEpi, 2>(p, base, split, k_part, m0, n, row, bias);
      else if (p.splits == 4)
        reduce_columns<MT, kEpi, 4>(p, base, split, k_part, m0, n, row, bias);
      else if (p.splits == 8)
        reduce_columns<MT, kEpi, 8>(p, base, split, k_part, m0, n, row, bias);
      else
        reduce_columns<MT, kEpi, 0>(p, base, split, k_part, m0, n, row, bias);
    }
    cluster_sync_all();       // nobody leaves while a peer may still read its shared memory
  }
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, C::kTmemCols);
  }
}

__device__ int g_error;

template <int MT, int kEpi>
int launch(const CUtensorMap* w_map, const CUtensorMap* x_map, Params p, int n_tiles, int m_tiles,
           cudaStream_t stream) {
  constexpr bool kDual = kEpi == EPI_GATED;
  using C = Cfg<MT, kDual>;
  static PerDeviceOnce configured;      // (attributes are per device)
  if (configured.needs()) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<MT, kEpi>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               C::smem_bytes(C::kMaxStages) > 227 * 1024
                                                   ? 227 * 1024 : C::smem_bytes(C::kMaxStages));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.done();
  }
  p.stages = C::stages_for((long long)n_tiles * m_tiles * p.splits * p.parts);
  while (C::smem_bytes(p.stages) > 227 * 1024) --p.stages;
  // The blocks that fit an SM by their shared memory must fit it by their tensor memory too
  // (512 columns): a block that waits for columns while its cluster waits for it could wait
  // for ever. A deeper ring makes the block large enough.
  while ((227 * 1024) / (C::smem_bytes(p.stages) + 1024) * C::kTmemCols > 512 &&
         C::smem_bytes(p.stages + 1) <= 227 * 1024)
    ++p.stages;
  // (A block with few K steps still asks for the whole ring: measured, the decode step is
  // 8 % slower when such blocks ask for less, as the blocks of a cluster then share SMs.)
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_error) != cudaSuccess)
    return cudaErrorInvalidValue;
  return launch_overlapped(gemm_tc_kernel<MT, kEpi>, dim3(n_tiles, m_tiles, p.splits * p.parts),
                           dim3(kThreads), (size_t)C::smem_bytes(p.stages), stream, p.splits,
                           *w_map, *x_map, p);
}

}  // namespace

// A TMA descriptor of a row-major bf16 matrix [rows, cols] read in boxes of
// [box_rows, 64 columns]; `map` points to 128 bytes on the host.
SAKV_EXPORT int sakv_gemm_tc_map(void* map, const void* base, long long rows, long long cols,
                                 long long row_stride_elems, int box_rows) {
  if (rows <= 0 || cols <= 0 || (cols % 8) || (row_stride_elems % 8) || box_rows <= 0 ||
      box_rows > 256)
    return cudaErrorInvalidValue;
  return tma::make_map_bf16_2d(reinterpret_cast<CUtensorMap*>(map), base, (uint64_t)rows,
                               (uint64_t)cols, (uint64_t)row_stride_elems * 2, box_rows, BK);
}

// `parts` > 1 (EPI_F32 only): K is cut into `parts` ranges whose sums are left apart, part i
// at `out + i * part_stride`, for the reader to add; each range is split over a cluster of
// `splits` as before. parts * splits must leave no K range empty (see sakv_gemm_tc_splits).
SAKV_EXPORT int sakv_gemm_tc(const void* w_map, const void* x_map, int M, int N, int K, int mt,
                             int splits, int parts, int epi, int dual_offset, const void* bias,
                             int bias_dtype, void* out, long long ldo, long long part_stride,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || splits < 1 || epi < 0 || epi > EPI_GATED ||
      ldo < N || parts < 1 || parts > 64 || (parts > 1 && epi != EPI_F32))
    return cudaErrorInvalidValue;
  const int total_kb = (K + BK - 1) / BK;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits * parts > total_kb) {
    if (parts > 1) return cudaErrorInvalidValue;
    splits = total_kb;
  }
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.parts = parts; p.part_stride = part_stride;
  p.kb_per_split = (total_kb + splits * parts - 1) / (splits * parts);
  if (parts == 1)
    p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;     // no empty split
  else if ((total_kb + p.kb_per_split - 1) / p.kb_per_split != splits * parts)
    return cudaErrorInvalidValue;                                    // a range would be empty
  else
    p.splits = splits;
  p.dual_offset = dual_offset;
  p.epi = epi; p.bias = bias; p.bias_dtype = bias_dtype;
  p.out = out; p.ldo = ldo; p.error = nullptr;
  const int n_tiles = (N + BM - 1) / BM;
  const int m_tiles = (M + mt - 1) / mt;
  if (m_tiles > 65535) return cudaErrorInvalidValue;
  const bool dual = epi == EPI_GATED;
  const CUtensorMap* wm = (const CUtensorMap*)w_map;
  const CUtensorMap* xm = (const CUtensorMap*)x_map;
#define GO(MT_)                                                                   \
  if (mt == MT_)                                                                  \
    return dual ? launch<MT_, EPI_GATED>(wm, xm, p, n_tiles, m_tiles, stream)     \
         : epi == EPI_BF16 ? launch<MT_, EPI_BF16>(wm, xm, p, n_tiles, m_tiles, stream)   \
         : epi == EPI_F32 ? launch<MT_, EPI_F32>(wm, xm, p, n_tiles, m_tiles, stream)     \
                          : launch<MT_, EPI_ACCUM>(wm, xm, p, n_tiles, m_tiles, stream)
  GO(16); GO(32); GO(64); GO(128);
  if (!dual) GO(256);
#undef GO
  return cudaErrorInvalidValue;
}

// The number of splits a launch asked for `splits` will really use.
SAKV_EXPORT int sakv_gemm_tc_splits(int K, int splits) {
  const int total_kb = (K + BK - 1) / BK;
  if (splits > total_kb) splits = total_kb;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits < 1) splits = 1;
  const int per = (total_kb + splits - 1) / splits;
  return (total_kb + per - 1) / per;
}

// How many clusters of `splits` blocks of the kernel for token tile `mt` can be resident
// at once (0 if it cannot be asked).
SAKV_EXPORT int sakv_gemm_tc_max_clusters(int mt, int dual, int splits) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1, 1, splits);
  config.blockDim = dim3(kThreads);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  config.attrs = attr;
  config.numAttrs = 1;
  int clusters = 0;
#define ASK(MT_, D_)                                                                           \
  if (mt == MT_ && (dual != 0) == D_) {                                                        \
    using C = Cfg<MT_, D_>;                                                                    \
    const int bytes = C::smem_bytes(C::stages_for(1));                                         \
    config.dynamicSmemBytes = bytes > 227 * 1024 ? 227 * 1024 : bytes;                         \
    cudaFuncSetAttribute(gemm_tc_kernel<MT_, (D_ ? EPI_GATED : EPI_BF16)>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                         (int)config.dynamicSmemBytes);                                        \
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_kernel<MT_, (D_ ? EPI_GATED : EPI_BF16)>, &config) !=         \
        cudaSuccess)                                                                           \
      clusters = 0;                                                                            \
    cudaGetLastError();                                                                        \
    return clusters;                                                                           \
  }
  ASK(16, false) ASK(32, false) ASK(64, false) ASK(128, false) ASK(256, false)
  ASK(16, true) ASK(32, true) ASK(64, true) ASK(128, true)
#undef ASK
  return 0;
}

SAKV_EXPORT int sakv_gemm_tc_error(int* value) {
  return static_cast<int>(cudaMemcpyFromSymbol(value, g_error, sizeof(int)));
}
