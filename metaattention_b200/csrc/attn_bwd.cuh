// Backward of attention for sm_100a, generic over a functor that gives P and dS per score element (head dims
// 128 / 128 or 64 / 64, 16-bit inputs, fp32 accumulation):
//
//   dV = P^T dO,   dP = dO V^T,   dS = dP o dP/dS,   dK = dS^T Q,   dQ = dS K
//
// One kernel template in two roles.  A CTA keeps one 128-row tile pair resident (X: K_j, V_j or Q_i, dO_i) and streams
// the other (Y1: Q_i or K_j through a three-stage TMA ring, Y2: dO_i or V_j through a two-stage one).  Per streamed tile:
//   S  = X1 Y1^T, dP = X2 Y2^T           tcgen05 SS, fp32 in tensor memory (columns [0,128) and [128,256))
//   row threads (thread = TMEM lane x column half): P and dS as 16-bit pairs
//   acc1 += P  Y2   (dV; KV role only)    tcgen05 TS, A from tensor memory, B = the streamed tile MN-major
//   acc2 += dS Y1   (dK or dQ)
// With the KV role the lanes are KV rows and the columns query rows (S^T, dP^T), so that P^T and dS^T are the A
// operands as they stand.  The functor F supplies
//   F::kUsesStats            per-query-row statistics (softmax: lse and delta) travel with the query tiles
//   F::kNegInfMask           P and dS vanish at a score of -inf: masked pairs are given that score
//   F::Ctx F::make(params)   per-thread constants
//   F::score(s, lse2, ctx, b, h, q_idx, kv_idx, p_out, g_out)   P, and the factor g that turns dP into dS
//   F::grad(g, dp, delta, ctx)                                   dS without its constant factor
//   F::out_scale(ctx)                                            the constant factor, applied to the finished dK, dQ rows
// softmax_bwd.cu instantiates it for the built-in softmax; lowered score_mod functors (elementwise programs: no row
// scales) get a library of their own, compiled from the forward-mode derivative of the traced expression.
//
// The tensor pipe executes in issue order, and both roles lean on that to keep it and the row threads busy at once:
//   KV role   ... dV(i) | S(i+1) | dK(i) | dP(i+1) ...   row threads: P(i) from S(i), then dS(i) from dP(i)
//             S(i+1) overwrites P(i) behind dV(i), dP(i+1) overwrites dS(i) behind dK(i); while the rows turn dP(i)
//             into dS(i) the pipe computes dV(i) and S(i+1), while they turn S(i+1) into P(i+1) it computes dK(i)
//             and dP(i+1).
//   Q role    ... S(i+1), dP(i+1) | dQ(i) ...            dS sits in two buffers of its own (the role has no second
//             accumulator), so S, dP of the next tile are issued once the rows hold this tile's in registers.
#pragma once

#include <cstring>
#include <type_traits>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "parallel_launch.cuh"  // tensor_map_encoder(), encode_rows_map(), CoordOrder, tma_load_rows()
#include "sm100.cuh"

namespace b200 {

constexpr int kBwdT = 128;                // rows of a tile, both ways
constexpr int kBwdRowThreads = 256;       // eight warps: one TMEM lane each, two column halves
constexpr int kBwdThreads = kBwdRowThreads + 64;   // plus the loading warp and the MMA-issuing warp
constexpr int kBwdStages1 = 3;            // ring of Y1 (read by the first and by the last MMA of its tile)
constexpr int kBwdStages2 = 2;            // ring of Y2

struct BwdParams {
  const void* custom[ATTN_B200_MAX_CUSTOM];   // device pointers of the functor's custom inputs (lowered functors)
  void* dq;
  void* dk;
  void* dv;
  const float* lse2;    // [batch, heads, seq_q_pad] lse * log2(e); +inf past seq_q (those rows get P = 0)
  const float* delta;   // [batch, heads, seq_q_pad]
  int batch, heads, heads_kv, kv_group, seq_q, seq_kv, seq_q_pad;
  int mask_left, mask_right;   // keep q_idx - mask_left <= kv_idx <= q_idx + mask_right; ATTN_B200_MASK_OPEN = no bound
  // kBits kernels (any mask that does not depend on batch or head, as keep bits): bits_q[q][kv tile][4 words] = the
  // 128 keep bits of query row q in that KV tile, bits_kv[kv][query tile][4 words] the same matrix transposed; both
  // padded with zeros to whole tiles.  Every pair of tiles is visited.
  const uint32_t* bits_q;
  const uint32_t* bits_kv;
  // optional with the bits: which tiles keep anything at all, so that the others are not visited.  tiles_q[query tile]
  // [tile_words_k] = bitmap over the KV tiles, tiles_kv[KV tile][tile_words_q] = bitmap over the query tiles
  const uint32_t* tiles_q;
  const uint32_t* tiles_kv;
  int tile_words_k, tile_words_q;
  float scale;
  long long dq_s[3], dk_s[3], dv_s[3];   // element strides (batch, seq, head)
  CoordOrder oq, ok, ov, odo;
  int* status;
};

enum BwdWaitSite { kBwdXFull = 61, kBwdYFull, kBwdYEmpty, kBwdSDone, kBwdPReady, kBwdAccDone, kBwdSdpFree, kBwdDpDone, kBwdDsReady, kBwdSmemAlign };
enum BwdBarrier {
  kBarXFull = 0,
  kBarY1Full,                               // kBwdStages1 of them
  kBarY1Empty = kBarY1Full + kBwdStages1,
  kBarY2Full = kBarY1Empty + kBwdStages1,   // kBwdStages2 of them
  kBarY2Empty = kBarY2Full + kBwdStages2,
  kBarSDone = kBarY2Empty + kBwdStages2,
  kBarDpDone,
  kBarPReadyB,
  kBarDsReady,
  kBarAccDone,
  kBarSdpFree,
  kNumBwdBarriers
};

template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kBwdT * D * 2;            // D/64 chunks of 128 rows x 128 B (64 columns)
  static constexpr int kChunkBytes = kBwdT * 128;
  static constexpr int kOffX1 = 0;
  static constexpr int kOffX2 = kOffX1 + kTileBytes;
  static constexpr int kOffY1 = kOffX2 + kTileBytes;                   // [kBwdStages1] tiles
  static constexpr int kOffY2 = kOffY1 + kBwdStages1 * kTileBytes;     // [kBwdStages2] tiles
  static constexpr int kOffLse = kOffY2 + kBwdStages2 * kTileBytes;    // [kBwdStages1][128] fp32, with Y1 (KV role)
  static constexpr int kStatBytes = kBwdT * 4;
  static constexpr int kOffDelta = kOffLse + kBwdStages1 * kStatBytes; // [kBwdStages2][128] fp32, with Y2 (KV role)
  static constexpr int kOffBar = kOffDelta + kBwdStages2 * kStatBytes;
  static constexpr int kOffMisc = kOffBar + 8 * kNumBwdBarriers;
  static constexpr int kBytes = kOffMisc + 16;                // the dynamic shared memory is declared 1024-byte aligned
  static_assert(kBytes <= 232448, "shared memory layout exceeds an SM");
};

// plain (untiled) bulk copy global -> shared, counted on an mbarrier; both addresses 16-byte aligned, bytes % 16 == 0
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// The set bits of one row of a tile bitmap, in order, over and over (the KV role walks its row once per query head of
// its group).  The caller knows how many there are and never asks an empty row.
struct KeptTiles {
  const uint32_t* words;
  int nwords, w;
  uint32_t bits;
  __device__ KeptTiles(const uint32_t* p, int n) : words(p), nwords(n), w(-1), bits(0) {}
  __device__ int next() {
    while (bits == 0) {
      if (++w >= nwords) w = 0;
      bits = words[w];
    }
    const int j = w * 32 + __ffs(bits) - 1;
    bits &= bits - 1;
    return j;
  }
  __device__ int count() const {
    int c = 0;
    for (int i = 0; i < nwords; ++i) c += __popc(words[i]);
    return c;
  }
};

// kRoleQ = false: CTA = (KV tile, KV head, batch), streams the query tiles (of every query head of its group) and
// writes dK, dV.  kRoleQ = true: CTA = (query tile, query head, batch), streams the KV tiles and writes dQ.
// Tensor memory: S [0,128), dP [128,256), accumulator 1 [256,384) (dV or dQ), accumulator 2 [384,512) (dK; the
// query role's two dS buffers).  KV role: P is written over S, dS over dP.
template <class F, bool kRoleQ, bool kBf16, int D, bool kBits = false>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int T = kBwdT, KC = D / 64, HALF = D / 2;   // chunks of a tile; columns of an accumulator row per warp group
  constexpr int N1 = kBwdStages1, N2 = kBwdStages2;
  static_assert(D == 64 || D == 128, "head dims 64 and 128");
  constexpr uint32_t kTmemCols = 512, kColS = 0, kColDP = 128, kColA = 256, kColB = 384, kColDS = 384;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sX1 = smem + L::kOffX1;
  uint8_t* sX2 = smem + L::kOffX2;
  uint8_t* sY1 = smem + L::kOffY1;
  uint8_t* sY2 = smem + L::kOffY2;
  float* sLse = reinterpret_cast<float*>(smem + L::kOffLse);
  float* sDelta = reinterpret_cast<float*>(smem + L::kOffDelta);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* x_full = bars + kBarXFull;
  uint64_t* y1_full = bars + kBarY1Full;
  uint64_t* y1_empty = bars + kBarY1Empty;
  uint64_t* y2_full = bars + kBarY2Full;
  uint64_t* y2_empty = bars + kBarY2Empty;
  uint64_t* s_done = bars + kBarSDone;
  uint64_t* dp_done = bars + kBarDpDone;
  uint64_t* p_ready = bars + kBarPReadyB;
  uint64_t* ds_ready = bars + kBarDsReady;
  uint64_t* acc_done = bars + kBarAccDone;
  uint64_t* sdp_free = bars + kBarSdpFree;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const AbortState ab{abort_flag, p.status};
  const int tile = blockIdx.x, hx = blockIdx.y, b = blockIdx.z;
  const int nq = (p.seq_q + T - 1) / T, nk = (p.seq_kv + T - 1) / T;
  // The streamed tiles are those the band q_idx - left <= kv_idx <= q_idx + right lets the resident tile meet: KV tiles
  // [j0, j0 + n_iter) for a query tile; for a KV tile the query tiles [i0, i0 + per_head) of every query head of its
  // group, head after head.  (No mask: both sides open; causal: left open, right 0.)
  const long long r0 = static_cast<long long>(tile) * T, r1 = r0 + T - 1;   // rows of the resident tile
  const int i0 = static_cast<int>(max(r0 - p.mask_right, 0LL) / T);
  const int i1 = static_cast<int>(min(static_cast<long long>(nq) - 1, (r1 + p.mask_left) / T));
  const int j0 = static_cast<int>(max(r0 - p.mask_left, 0LL) / T);
  const int j1 = static_cast<int>(min(static_cast<long long>(nk) - 1, (r1 + p.mask_right) / T));
  // with keep bits and a tile bitmap: the tiles whose bit is set in this tile's row of the bitmap
  const bool walk_tiles = kBits && p.tiles_q != nullptr;
  const uint32_t* tiles_row = !walk_tiles ? nullptr
                              : kRoleQ  ? p.tiles_q + static_cast<long long>(tile) * p.tile_words_k
                                        : p.tiles_kv + static_cast<long long>(tile) * p.tile_words_q;
  const int tiles_words = kRoleQ ? p.tile_words_k : p.tile_words_q;
  const int n_kept = walk_tiles ? KeptTiles(tiles_row, tiles_words).count() : 0;
  const int per_head = kRoleQ ? 0 : (walk_tiles ? n_kept : max(i1 - i0 + 1, 0));
  const int n_iter = kRoleQ ? (walk_tiles ? n_kept : max(j1 - j0 + 1, 0)) : p.kv_group * per_head;

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    // the operand tiles use the 128-byte swizzle, whose pattern repeats every 1024 bytes of the shared window
    if ((smem_u32(smem) & 1023u) != 0) {
      *abort_flag = 1;
      atomicCAS(p.status, 0, kStatusTimeoutBase + kBwdSmemAlign);
    }
    mbar_init(x_full, 1);
    for (int i = 0; i < N1; ++i) {
      mbar_init(y1_full + i, 1);
      mbar_init(y1_empty + i, 1);
    }
    for (int i = 0; i < N2; ++i) {
      mbar_init(y2_full + i, 1);
      mbar_init(y2_empty + i, 1);
    }
    mbar_init(s_done, 1);
    mbar_init(dp_done, 1);
    mbar_init(p_ready, kBwdRowThreads / 32);
    mbar_init(ds_ready, kBwdRowThreads / 32);
    mbar_init(acc_done, 1);
    mbar_init(sdp_free, kBwdRowThreads / 32);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool start_ok = !*abort_flag;

  if (warp == kBwdRowThreads / 32) {
    // ======================= loading warp =======================
    if (lane == 0 && start_ok && n_iter > 0) {
      mbar_arrive_expect_tx(x_full, 2 * L::kTileBytes);
      for (int c = 0; c < KC; ++c) {
        if constexpr (kRoleQ) {
          tma_load_rows(sX1 + c * L::kChunkBytes, &tmQ, x_full, c * 64, tile * T, hx, b, p.oq);
          tma_load_rows(sX2 + c * L::kChunkBytes, &tmDO, x_full, c * 64, tile * T, hx, b, p.odo);
        } else {
          tma_load_rows(sX1 + c * L::kChunkBytes, &tmK, x_full, c * 64, tile * T, hx, b, p.ok);
          tma_load_rows(sX2 + c * L::kChunkBytes, &tmV, x_full, c * 64, tile * T, hx, b, p.ov);
        }
      }
      KeptTiles kept(tiles_row, tiles_words);
      for (int it = 0; it < n_iter; ++it) {
        const int s1 = it % N1, s2 = it % N2;
        const int ys = walk_tiles ? kept.next() : (kRoleQ ? j0 + it : i0 + it % max(per_head, 1));   // the streamed tile
        uint8_t* y1 = sY1 + s1 * L::kTileBytes;
        uint8_t* y2 = sY2 + s2 * L::kTileBytes;
        // streamed tile: row offset and head in the tensors it comes from
        const int hk = hx / p.kv_group;
        const int hq = kRoleQ ? 0 : hx * p.kv_group + it / per_head, i = ys;
        const long long stat_off = kRoleQ ? 0 : (static_cast<long long>(b) * p.heads + hq) * p.seq_q_pad + i * T;
        if (!mbar_wait(y1_empty + s1, ((it / N1) & 1) ^ 1, ab, kBwdYEmpty)) break;
        mbar_arrive_expect_tx(y1_full + s1, L::kTileBytes + ((!kRoleQ && F::kUsesStats) ? L::kStatBytes : 0));
        for (int c = 0; c < KC; ++c) {
          if constexpr (kRoleQ) {
            tma_load_rows(y1 + c * L::kChunkBytes, &tmK, y1_full + s1, c * 64, ys * T, hk, b, p.ok);
          } else {
            tma_load_rows(y1 + c * L::kChunkBytes, &tmQ, y1_full + s1, c * 64, i * T, hq, b, p.oq);
          }
        }
        if constexpr (!kRoleQ && F::kUsesStats) bulk_load(sLse + s1 * T, p.lse2 + stat_off, L::kStatBytes, y1_full + s1);
        if (!mbar_wait(y2_empty + s2, ((it / N2) & 1) ^ 1, ab, kBwdYEmpty)) break;
        mbar_arrive_expect_tx(y2_full + s2, L::kTileBytes + ((!kRoleQ && F::kUsesStats) ? L::kStatBytes : 0));
        for (int c = 0; c < KC; ++c) {
          if constexpr (kRoleQ) {
            tma_load_rows(y2 + c * L::kChunkBytes, &tmV, y2_full + s2, c * 64, ys * T, hk, b, p.ov);
          } else {
            tma_load_rows(y2 + c * L::kChunkBytes, &tmDO, y2_full + s2, c * 64, i * T, hq, b, p.odo);
          }
        }
        if constexpr (!kRoleQ && F::kUsesStats) bulk_load(sDelta + s2 * T, p.delta + stat_off, L::kStatBytes, y2_full + s2);
      }
    }
  } else if (warp == kBwdRowThreads / 32 + 1) {
    // ======================= issuing warp: every MMA =======================
    // The whole warp runs this code converged and one elected lane issues each batch of MMAs with its commits: the
    // descriptors then live in uniform registers, and a batch leaves at the pipe's rate whatever the row warps do
    // (issued from inside an `if (lane == 0)` region an MMA with N = 128 took ~90 cycles under load, against the 64
    // the pipe needs for it).
    if (__all_sync(0xffffffffu, start_ok) && n_iter > 0) {
      constexpr uint32_t idesc_kk = make_idesc_f16(T, T, kBf16, false, false);      // S, dP: both operands K-major
      constexpr uint32_t idesc_mn = make_idesc_f16(T, D, kBf16, false, true);       // accumulators: B = streamed tile, MN-major
      constexpr uint64_t kChunk = L::kChunkBytes >> 4;
      const uint64_t x1_desc = make_smem_desc(smem_u32(sX1), 16, 1024), x2_desc = make_smem_desc(smem_u32(sX2), 16, 1024);
      auto wait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
        return __all_sync(0xffffffffu, mbar_wait_poll(bar, parity, ab, site));
      };
      // out = X Y^T behind the arrival of the streamed tile, then up to two commits
      auto issue_xy = [&](uint32_t out_col, uint64_t x_desc, const uint8_t* y_tile, uint64_t* full, uint32_t parity, uint64_t* c1,
                          uint64_t* c2) -> bool {
        if (!wait(full, parity, kBwdYFull)) return false;
        tc_fence_after_sync();
        const uint64_t y_desc = make_smem_desc(smem_u32(y_tile), 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int ch = 0; ch < KC; ++ch)
            umma_ss_x4<2, 2>(tmem_base + out_col, x_desc + ch * kChunk, y_desc + ch * kChunk, idesc_kk, ch > 0 ? 1u : 0u);
          if (c1 != nullptr) umma_commit(c1);
          if (c2 != nullptr) umma_commit(c2);
        }
        return true;
      };
      auto issue_s = [&](int it, uint64_t* c1) -> bool {
        return issue_xy(kColS, x1_desc, sY1 + (it % N1) * L::kTileBytes, y1_full + it % N1, (it / N1) & 1, c1, nullptr);
      };
      auto issue_dp = [&](int it, uint64_t* c1, uint64_t* c2) -> bool {
        return issue_xy(kColDP, x2_desc, sY2 + (it % N2) * L::kTileBytes, y2_full + it % N2, (it / N2) & 1, c1, c2);
      };
      // acc += A (16-bit, tensor memory columns a_col...) x streamed tile (MN-major), then up to three commits
      auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, const uint8_t* y_tile, bool accumulate, uint64_t* c0, uint64_t* c1, uint64_t* c2) {
        const uint64_t y_mn = make_smem_desc(smem_u32(y_tile), L::kChunkBytes, 1024);
        if (elect_one()) {
          if (c0 != nullptr) umma_commit(c0);   // for what was issued before this batch
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ts_x4<8, 128>(tmem_base + acc_col, tmem_base + a_col + g * 32, y_mn + g * 512, idesc_mn, (accumulate || g > 0) ? 1u : 0u);
          if (c1 != nullptr) umma_commit(c1);
          if (c2 != nullptr) umma_commit(c2);
        }
      };
      bool ok = wait(x_full, 0, kBwdXFull);
      if constexpr (kRoleQ) {
        ok = ok && issue_s(0, nullptr) && issue_dp(0, y2_empty, s_done);
        for (int it = 0; ok && it < n_iter; ++it) {
          if (it + 1 < n_iter) {
            // the row threads hold S, dP of tile it in registers: those of tile it + 1 go ahead of tile it's dQ
            if (!wait(sdp_free, it & 1, kBwdSdpFree)) break;
            if (!(issue_s(it + 1, nullptr) && issue_dp(it + 1, y2_empty + (it + 1) % N2, s_done))) break;   // V is read by dP only
          }
          if (!wait(p_ready, it & 1, kBwdPReady)) break;
          tc_fence_after_sync();
          issue_acc(kColA, kColDS + (it & 1) * 64, sY1 + (it % N1) * L::kTileBytes, it > 0, nullptr, y1_empty + it % N1,
                    it + 1 == n_iter ? acc_done : nullptr);
        }
      } else {
        ok = ok && issue_s(0, s_done) && issue_dp(0, dp_done, nullptr);
        for (int it = 0; ok && it < n_iter; ++it) {
          const bool more = it + 1 < n_iter;
          if (!wait(p_ready, it & 1, kBwdPReady)) break;
          tc_fence_after_sync();
          issue_acc(kColA, kColS, sY2 + (it % N2) * L::kTileBytes, it > 0, nullptr, nullptr, nullptr);    // dV += P^T dO
          if (more && !issue_s(it + 1, s_done)) break;     // over P(it), behind dV(it) in the pipe
          if (!wait(ds_ready, it & 1, kBwdDsReady)) break;
          tc_fence_after_sync();
          // dO(it) has been read by dV(it); its stage also holds delta(it), which the row threads have now used
          issue_acc(kColB, kColDP, sY1 + (it % N1) * L::kTileBytes, it > 0, y2_empty + it % N2, y1_empty + it % N1,
                    more ? nullptr : acc_done);   // dK += dS^T Q
          if (more && !issue_dp(it + 1, dp_done, nullptr)) break;    // over dS(it), behind dK(it)
        }
      }
    }
  } else {
    // ======================= row threads: one TMEM lane each, 64 columns =======================
    const int wq = warp & 3, wg = warp >> 2;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS, tDP = tmem_base + lane_base + kColDP;
    const typename F::Ctx fctx = F::make(p);
    float lse2_r = 0.0f, delta_r = 0.0f;
    if constexpr (kRoleQ && F::kUsesStats) {
      const long long idx = (static_cast<long long>(b) * p.heads + hx) * p.seq_q_pad + tile * T + row;
      lse2_r = p.lse2[idx];
      delta_r = p.delta[idx];
    }
    // P and g of one element.  KV role: lanes are KV rows, columns query rows; query role the other way round.  The
    // band keeps, for this thread's row, the columns [col_lo, col_hi] of the tile (set per streamed tile; everything
    // when no edge of the band crosses the pair); a functor whose P vanishes at a score of -inf (softmax) gets the mask
    // through the score
    int col_lo = 0, col_hi = T;
    uint4 keep_bits = make_uint4(0, 0, 0, 0);   // kBits: this thread's row of the streamed tile
    auto score_of = [&](auto edge_tile, float s, float l2, int ys, int hq, int col, float& pr, float& g) {
      const int q_idx = kRoleQ ? tile * T + row : ys * T + col;
      const int kv_idx = kRoleQ ? ys * T + col : tile * T + row;
      bool masked;
      if constexpr (kBits) {
        const uint32_t w = (col >> 5) == 0 ? keep_bits.x : (col >> 5) == 1 ? keep_bits.y : (col >> 5) == 2 ? keep_bits.z : keep_bits.w;
        masked = ((w >> (col & 31)) & 1u) == 0u;
      } else {
        masked = decltype(edge_tile)::value && (col < col_lo || col > col_hi);
      }
      F::score((F::kNegInfMask && masked) ? -INFINITY : s, l2, fctx, b, hq, q_idx, kv_idx, pr, g);
      if (!F::kNegInfMask && masked) pr = g = 0.0f;
    };
    // KV role: the statistics belong to the columns and sit in shared memory; every lane reads the same four at a time
    auto stat_of = [&](const float* base, int k) -> float {
      const float4 v4 = *reinterpret_cast<const float4*>(base + (k & ~3));
      return (k & 3) == 0 ? v4.x : (k & 3) == 1 ? v4.y : (k & 3) == 2 ? v4.z : v4.w;
    };
    bool ok = start_ok;
    KeptTiles kept(tiles_row, tiles_words);
    for (int it = 0; ok && it < n_iter; ++it) {
      // the streamed tile index, its query head, and whether an edge of the band crosses this pair of tiles
      const int ys = walk_tiles ? kept.next() : (kRoleQ ? j0 + it : i0 + it % max(per_head, 1));
      const int hq = kRoleQ ? hx : hx * p.kv_group + it / max(per_head, 1);
      // Pairs of tiles that an edge of the band crosses take a second copy of the row loops, with the mask: the row
      // phases sit on the kernel's serial chain, and two compares per element on every tile cost 15 %
      const long long q0 = static_cast<long long>(kRoleQ ? tile : ys) * T, k0 = static_cast<long long>(kRoleQ ? ys : tile) * T;
      const bool edge = kBits || (k0 + T - 1 > q0 + p.mask_right) || (k0 + p.mask_left < q0 + T - 1);
      if constexpr (kBits) {
        const uint32_t* bits = kRoleQ ? p.bits_q : p.bits_kv;
        const long long pitch = 4LL * (kRoleQ ? nk : nq);   // words per row: four per streamed tile
        keep_bits = *reinterpret_cast<const uint4*>(bits + (static_cast<long long>(tile) * T + row) * pitch + 4LL * ys);
      } else if (edge) {
        // kv - q of (row, col) is base + col (query role) or base - col (KV role); kept where -left <= kv - q <= right
        const long long base = kRoleQ ? k0 - q0 - row : k0 - q0 + row;
        const long long lo = kRoleQ ? -static_cast<long long>(p.mask_left) - base : base - p.mask_right;
        const long long hi = kRoleQ ? static_cast<long long>(p.mask_right) - base : base + p.mask_left;
        col_lo = static_cast<int>(max(lo, 0LL));
        col_hi = static_cast<int>(min(hi, static_cast<long long>(T)));
      }
      if constexpr (kRoleQ) {
        ok = mbar_wait(s_done, it & 1, ab, kBwdSDone);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t pds[32];
        auto rows_q = [&](auto edge_tile) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c0 = wg * 64 + u * 32;
            float s[32], dp[32];
            tmem_ld32f(tS + c0, s);
            tmem_ld32f(tDP + c0, dp);
            tmem_wait_ld();
            if (u == 1) {   // this tile's S and dP are in registers: the next tile's may be computed
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(sdp_free);
            }
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              float pr, g;
              score_of(edge_tile, s[k], lse2_r, ys, hq, c0 + k, pr, g);
              dp[k] = F::grad(g, dp[k], delta_r, fctx);
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) pds[u * 16 + k] = pack2<kBf16>(dp[2 * k], dp[2 * k + 1]);
          }
        };
        if (edge) rows_q(std::true_type{});
        else rows_q(std::false_type{});
        tmem_st32(tmem_base + lane_base + kColDS + (it & 1) * 64 + wg * 32, pds);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      } else {
        // ---- S -> P (and g, kept in registers for the second half) ----
        if constexpr (F::kUsesStats) ok = mbar_wait(y1_full + it % N1, (it / N1) & 1, ab, kBwdYFull);   // lse came with the tile
        ok = mbar_wait_poll(s_done, it & 1, ab, kBwdSDone) && ok;
        if (!ok) break;
        tc_fence_after_sync();
        const float* st_lse = sLse + (it % N1) * T;
        const float* st_delta = sDelta + (it % N2) * T;
        float g[64];
        uint32_t pk[32];
        auto rows_p = [&](auto edge_tile) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c0 = wg * 64 + u * 32;
            float s[32];
            tmem_ld32f(tS + c0, s);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              float pr;
              score_of(edge_tile, s[k], F::kUsesStats ? stat_of(st_lse + c0, k) : 0.0f, ys, hq, c0 + k, pr, g[u * 32 + k]);
              s[k] = pr;
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) pk[u * 16 + k] = pack2<kBf16>(s[2 * k], s[2 * k + 1]);
          }
        };
        if (edge) rows_p(std::true_type{});
        else rows_p(std::false_type{});
        // the 16-bit pairs of columns [64 wg, 64 wg + 64) go to 32-bit columns [32 wg, 32 wg + 32), which the other warp
        // of this lane quarter reads as fp32: both must have their values in registers first
        tc_fence_before_sync();
        ok = named_sync_and(1 + wq, 64, ok);
        if (!ok) break;
        tc_fence_after_sync();
        tmem_st32(tS + wg * 32, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
        // ---- dP -> dS, beside the pipe's dV(it) and S(it + 1) ----
        if constexpr (F::kUsesStats) ok = mbar_wait(y2_full + it % N2, (it / N2) & 1, ab, kBwdYFull);   // delta came with the tile
        ok = mbar_wait(dp_done, it & 1, ab, kBwdDpDone) && ok;
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int c0 = wg * 64 + u * 32;
          float dp[32];
          tmem_ld32f(tDP + c0, dp);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) dp[k] = F::grad(g[u * 32 + k], dp[k], F::kUsesStats ? stat_of(st_delta + c0, k) : 0.0f, fctx);
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[u * 16 + k] = pack2<kBf16>(dp[2 * k], dp[2 * k + 1]);
        }
        tc_fence_before_sync();
        ok = named_sync_and(1 + wq, 64, ok);
        if (!ok) break;
        tc_fence_after_sync();
        tmem_st32(tDP + wg * 32, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_ready);
      }
    }
    // ---- epilogue: the accumulators as 16-bit rows (dK and dQ times the functor's constant factor) ----
    if (ok && n_iter > 0) {
      ok = mbar_wait(acc_done, 0, ab, kBwdAccDone);
      tc_fence_after_sync();
    }
    if (ok) {
      const int r = tile * T + row;
      const int n_out = kRoleQ ? 1 : 2;
      for (int a = 0; a < n_out; ++a) {
        // a = 0: dQ (query role) or dV; a = 1: dK
        uint16_t* base;
        if constexpr (kRoleQ) {
          base = static_cast<uint16_t*>(p.dq) + b * p.dq_s[0] + static_cast<long long>(r) * p.dq_s[1] + hx * p.dq_s[2];
        } else {
          const long long* sd = a == 0 ? p.dv_s : p.dk_s;
          base = static_cast<uint16_t*>(a == 0 ? p.dv : p.dk) + b * sd[0] + static_cast<long long>(r) * sd[1] + hx * sd[2];
        }
        const float f = (kRoleQ || a == 1) ? F::out_scale(fctx) : 1.0f;
        const bool in_range = r < (kRoleQ ? p.seq_q : p.seq_kv);
#pragma unroll
        for (int u = 0; u < HALF / 32; ++u) {
          const int c0 = wg * HALF + u * 32;
          float v[32];
          if (n_iter > 0) {
            tmem_ld32f(tmem_base + lane_base + (a == 0 ? kColA : kColB) + c0, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = 0.0f;
          }
          if (in_range) {
            uint4* dst = reinterpret_cast<uint4*>(base + c0);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 pk;
              pk.x = pack2<kBf16>(v[8 * q4 + 0] * f, v[8 * q4 + 1] * f);
              pk.y = pack2<kBf16>(v[8 * q4 + 2] * f, v[8 * q4 + 3] * f);
              pk.z = pack2<kBf16>(v[8 * q4 + 4] * f, v[8 * q4 + 5] * f);
              pk.w = pack2<kBf16>(v[8 * q4 + 6] * f, v[8 * q4 + 7] * f);
              dst[q4] = pk;
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// What a backward launch needs beside the functor: filled from the C-ABI argument structs.
struct BwdCall {
  const void *q, *k, *v, *d_o;
  void *dq, *dk, *dv;
  int batch, heads, heads_kv, seq_q, seq_kv, dim, dtype, mask_left, mask_right;
  float scale;
  const int64_t *q_stride, *k_stride, *v_stride, *do_stride, *dq_stride, *dk_stride, *dv_stride;
  const float* lse2;
  const float* delta;
  const void* const* custom;
  const uint32_t *bits_q, *bits_kv;   // both or neither: keep bits of a general mask (the band then has to be open)
  const uint32_t *tiles_q, *tiles_kv; // with the bits, optional (both or neither): bitmaps of the tiles that keep anything
};

// dK/dV launch (one CTA per KV tile and KV head) and dQ launch (one per query tile and head) for functor F.
template <class F, bool kBf16, int D>
int launch_attn_bwd(const BwdCall& a, cudaStream_t stream, int* status) {
  using L = BwdSmem<D>;
  const int T = kBwdT;
  const int nq = (a.seq_q + T - 1) / T, nk = (a.seq_kv + T - 1) / T;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  BwdParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = encode_rows_map(&tmQ, &p.oq, a.q, a.dtype, D, a.batch, a.seq_q, a.heads, a.q_stride, T);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows_map(&tmK, &p.ok, a.k, a.dtype, D, a.batch, a.seq_kv, a.heads_kv, a.k_stride, T);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows_map(&tmV, &p.ov, a.v, a.dtype, D, a.batch, a.seq_kv, a.heads_kv, a.v_stride, T);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows_map(&tmDO, &p.odo, a.d_o, a.dtype, D, a.batch, a.seq_q, a.heads, a.do_stride, T);
  if (rc != ATTN_B200_OK) return rc;
  p.dq = a.dq;
  p.dk = a.dk;
  p.dv = a.dv;
  p.lse2 = a.lse2;
  p.delta = a.delta;
  p.batch = a.batch;
  p.heads = a.heads;
  p.heads_kv = a.heads_kv;
  p.kv_group = a.heads / a.heads_kv;
  p.seq_q = a.seq_q;
  p.seq_kv = a.seq_kv;
  p.seq_q_pad = nq * T;
  p.mask_left = a.mask_left;
  p.mask_right = a.mask_right;
  p.bits_q = a.bits_q;
  p.bits_kv = a.bits_kv;
  p.tiles_q = a.bits_q != nullptr ? a.tiles_q : nullptr;
  p.tiles_kv = a.bits_q != nullptr ? a.tiles_kv : nullptr;
  p.tile_words_k = (nk + 31) / 32;
  p.tile_words_q = (nq + 31) / 32;
  p.scale = a.scale;
  for (int i = 0; i < 3; ++i) {
    p.dq_s[i] = a.dq_stride[i];
    p.dk_s[i] = a.dk_stride[i];
    p.dv_s[i] = a.dv_stride[i];
  }
  for (int i = 0; i < ATTN_B200_MAX_CUSTOM; ++i) p.custom[i] = a.custom != nullptr ? a.custom[i] : nullptr;
  p.status = status;
  const bool with_bits = a.bits_q != nullptr;
  auto kv_kernel = with_bits ? attn_bwd_kernel<F, false, kBf16, D, true> : attn_bwd_kernel<F, false, kBf16, D, false>;
  auto q_kernel = with_bits ? attn_bwd_kernel<F, true, kBf16, D, true> : attn_bwd_kernel<F, true, kBf16, D, false>;
  if (cudaFuncSetAttribute(kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess ||
      cudaFuncSetAttribute(q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  kv_kernel<<<dim3(nk, a.heads_kv, a.batch), kBwdThreads, L::kBytes, stream>>>(tmQ, tmK, tmV, tmDO, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  q_kernel<<<dim3(nq, a.heads, a.batch), kBwdThreads, L::kBytes, stream>>>(tmQ, tmK, tmV, tmDO, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  return ATTN_B200_OK;
}

// mask_kind, the band and the keep bits of an argument struct as the mask of a call; false = not a mask the backward covers
inline bool bwd_mask_of(int mask_kind, int left, int right, const void* bits_q, const void* bits_kv, const void* tiles_q,
                        const void* tiles_kv, BwdCall& call) {
  call.bits_q = call.bits_kv = call.tiles_q = call.tiles_kv = nullptr;
  if (mask_kind == ATTN_B200_MASK_BITS) {
    if (bits_q == nullptr || bits_kv == nullptr) return false;
    if ((tiles_q == nullptr) != (tiles_kv == nullptr)) return false;
    call.tiles_q = static_cast<const uint32_t*>(tiles_q);
    call.tiles_kv = static_cast<const uint32_t*>(tiles_kv);
    if (((reinterpret_cast<uintptr_t>(bits_q) | reinterpret_cast<uintptr_t>(bits_kv)) & 15) != 0) return false;
    call.bits_q = static_cast<const uint32_t*>(bits_q);
    call.bits_kv = static_cast<const uint32_t*>(bits_kv);
    call.mask_left = call.mask_right = ATTN_B200_MASK_OPEN;
  } else if (mask_kind == ATTN_B200_MASK_NONE) {
    call.mask_left = call.mask_right = ATTN_B200_MASK_OPEN;
  } else if (mask_kind == ATTN_B200_MASK_CAUSAL) {
    call.mask_left = ATTN_B200_MASK_OPEN;
    call.mask_right = 0;
  } else if (mask_kind == ATTN_B200_MASK_BAND) {
    if (left < 0 || right < 0 || left > ATTN_B200_MASK_OPEN || right > ATTN_B200_MASK_OPEN) return false;
    call.mask_left = left;
    call.mask_right = right;
  } else {
    return false;
  }
  return true;
}

// Checks shared by every backward entry point (pointers, dims, strides, alignment of the outputs).
inline int validate_bwd_call(const BwdCall& a) {
  if (a.q == nullptr || a.k == nullptr || a.v == nullptr || a.d_o == nullptr || a.dq == nullptr || a.dk == nullptr || a.dv == nullptr)
    return ATTN_B200_E_INVALID_ARG;
  if (a.batch <= 0 || a.heads <= 0 || a.seq_q <= 0 || a.seq_kv <= 0) return ATTN_B200_E_INVALID_ARG;
  if (a.dtype != ATTN_B200_DTYPE_FP16 && a.dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a.heads_kv <= 0 || a.heads % a.heads_kv != 0) return ATTN_B200_E_INVALID_ARG;
  if (a.dim != 64 && a.dim != 128) return ATTN_B200_E_UNSUPPORTED;
  if (a.batch > 65535 || a.heads > 65535) return ATTN_B200_E_UNSUPPORTED;
  const void* outs[3] = {a.dq, a.dk, a.dv};
  const int64_t* strides[3] = {a.dq_stride, a.dk_stride, a.dv_stride};
  for (int i = 0; i < 3; ++i) {
    if ((reinterpret_cast<uintptr_t>(outs[i]) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
    for (int d = 0; d < 3; ++d)
      if (strides[i][d] % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  }
  return ATTN_B200_OK;
}

}  // namespace b200
