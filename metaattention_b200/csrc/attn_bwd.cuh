// Backward of attention for sm_100a, generic over a functor that gives P and dS per score element (head dims
// 128 / 128 or 64 / 64, 16-bit inputs, fp32 accumulation):
//
//   dV = P^T dO,   dP = dO V^T,   dS = dP o dP/dS,   dK = dS^T Q,   dQ = dS K
//
// One kernel template in two roles.  A CTA keeps one 128-row tile pair resident (X: K_j, V_j or Q_i, dO_i) and streams
// the other (Y: Q_i, dO_i or K_j, V_j) through a two-stage TMA ring.  Per streamed tile:
//   S  = X1 Y1^T, dP = X2 Y2^T           tcgen05 SS, fp32 in tensor memory (columns [0,128) and [128,256))
//   row threads (thread = TMEM lane x column half): P and dS as 16-bit pairs
//   acc1 += P  Y2   (dV; KV role only)    tcgen05 TS, A from tensor memory, B = the streamed tile MN-major
//   acc2 += dS Y1   (dK or dQ)
// With the KV role the lanes are KV rows and the columns query rows (S^T, dP^T), so that P^T and dS^T are the A
// operands as they stand.  The functor F supplies
//   F::kUsesStats            per-query-row statistics (softmax: lse and delta) travel with the query tiles
//   F::kNegInfMask           P and dS vanish at a score of -inf: masked pairs are given that score
//   F::Ctx F::make(params)   per-thread constants
//   F::apply(s, dp, lse2, delta, ctx, b, h, q_idx, kv_idx, p_out, ds_out)
// softmax_bwd.cu instantiates it for the built-in softmax; lowered score_mod functors (elementwise programs: no row
// scales) get a library of their own, compiled from the forward-mode derivative of the traced expression.
#pragma once

#include <cstring>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "parallel_launch.cuh"  // tensor_map_encoder(), encode_rows_map(), CoordOrder, tma_load_rows()
#include "sm100.cuh"

namespace b200 {

constexpr int kBwdT = 128;                // rows of a tile, both ways
constexpr int kBwdRowThreads = 256;       // eight warps: one TMEM lane each, two column halves
constexpr int kBwdThreads = kBwdRowThreads + 64;   // plus the loading warp and the MMA-issuing warp

struct BwdParams {
  const void* custom[ATTN_B200_MAX_CUSTOM];   // device pointers of the functor's custom inputs (lowered functors)
  void* dq;
  void* dk;
  void* dv;
  const float* lse2;    // [batch, heads, seq_q_pad] lse * log2(e); +inf past seq_q (those rows get P = 0)
  const float* delta;   // [batch, heads, seq_q_pad]
  int batch, heads, heads_kv, kv_group, seq_q, seq_kv, seq_q_pad;
  int causal;
  float scale;
  long long dq_s[3], dk_s[3], dv_s[3];   // element strides (batch, seq, head)
  CoordOrder oq, ok, ov, odo;
  int* status;
};

enum BwdWaitSite { kBwdXFull = 61, kBwdYFull, kBwdYEmpty, kBwdSDone, kBwdPReady, kBwdAccDone, kBwdSdpFree };
enum BwdBarrier { kBarXFull = 0, kBarYFull0, kBarYFull1, kBarYEmpty0, kBarYEmpty1, kBarSDone, kBarPReadyB, kBarAccDone, kBarSdpFree, kNumBwdBarriers };

template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kBwdT * D * 2;            // D/64 chunks of 128 rows x 128 B (64 columns)
  static constexpr int kChunkBytes = kBwdT * 128;
  static constexpr int kOffX1 = 0;
  static constexpr int kOffX2 = kOffX1 + kTileBytes;
  static constexpr int kOffY = kOffX2 + kTileBytes;           // [2 stages][Y1, Y2]
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kOffStats = kOffY + 2 * kStageBytes;   // [2 stages][lse2[128], delta[128]] fp32 (KV role)
  static constexpr int kStatsBytes = 2 * kBwdT * 4;
  static constexpr int kOffBar = kOffStats + 2 * kStatsBytes;
  static constexpr int kOffMisc = kOffBar + 8 * kNumBwdBarriers;
  static constexpr int kBytes = kOffMisc + 16 + 1024;
};

// plain (untiled) bulk copy global -> shared, counted on an mbarrier; both addresses 16-byte aligned, bytes % 16 == 0
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// kRoleQ = false: CTA = (KV tile, KV head, batch), streams the query tiles (of every query head of its group) and
// writes dK, dV.  kRoleQ = true: CTA = (query tile, query head, batch), streams the KV tiles and writes dQ.
// Tensor memory: S [0,128), dP [128,256), accumulator 1 [256,384) (dV or dQ), accumulator 2 [384,512) (dK).
// The query role has no second accumulator: it writes dS to two alternating 64-column buffers there instead of over
// dP, so that S and dP of the next tile can be computed as soon as the row threads hold this tile's in registers.
template <class F, bool kRoleQ, bool kBf16, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int T = kBwdT, KC = D / 64, HALF = D / 2;   // chunks of a tile; columns of an accumulator row per warp group
  static_assert(D == 64 || D == 128, "head dims 64 and 128");
  constexpr uint32_t kTmemCols = 512, kColS = 0, kColDP = 128, kColA = 256, kColB = 384, kColDS = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX1 = smem + L::kOffX1;
  uint8_t* sX2 = smem + L::kOffX2;
  uint8_t* sY = smem + L::kOffY;
  float* sStats = reinterpret_cast<float*>(smem + L::kOffStats);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* x_full = bars + kBarXFull;
  uint64_t* y_full = bars + kBarYFull0;
  uint64_t* y_empty = bars + kBarYEmpty0;
  uint64_t* s_done = bars + kBarSDone;
  uint64_t* p_ready = bars + kBarPReadyB;
  uint64_t* acc_done = bars + kBarAccDone;
  uint64_t* sdp_free = bars + kBarSdpFree;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const AbortState ab{abort_flag, p.status};
  const int tile = blockIdx.x, hx = blockIdx.y, b = blockIdx.z;
  const int nq = (p.seq_q + T - 1) / T, nk = (p.seq_kv + T - 1) / T;
  // the streamed tiles: KV tiles [0, n_iter) for a query tile; for a KV tile the query tiles [i0, nq) of every
  // query head of its group, head after head
  const int i0 = p.causal ? tile : 0;
  const int per_head = kRoleQ ? 0 : max(nq - i0, 0);
  const int n_iter = kRoleQ ? (p.causal ? min(nk, tile + 1) : nk) : p.kv_group * per_head;

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_init(x_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(y_full + i, 1);
      mbar_init(y_empty + i, 1);
    }
    mbar_init(s_done, 1);
    mbar_init(p_ready, kBwdRowThreads / 32);
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
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        if (!mbar_wait(y_empty + st, ((it >> 1) & 1) ^ 1, ab, kBwdYEmpty)) break;
        uint8_t* y1 = sY + st * L::kStageBytes;
        uint8_t* y2 = y1 + L::kTileBytes;
        if constexpr (kRoleQ) {
          mbar_arrive_expect_tx(y_full + st, 2 * L::kTileBytes);
          const int hk = hx / p.kv_group;
          for (int c = 0; c < KC; ++c) {
            tma_load_rows(y1 + c * L::kChunkBytes, &tmK, y_full + st, c * 64, it * T, hk, b, p.ok);
            tma_load_rows(y2 + c * L::kChunkBytes, &tmV, y_full + st, c * 64, it * T, hk, b, p.ov);
          }
        } else {
          mbar_arrive_expect_tx(y_full + st, 2 * L::kTileBytes + (F::kUsesStats ? L::kStatsBytes : 0));
          const int hq = hx * p.kv_group + it / per_head, i = i0 + it % per_head;
          for (int c = 0; c < KC; ++c) {
            tma_load_rows(y1 + c * L::kChunkBytes, &tmQ, y_full + st, c * 64, i * T, hq, b, p.oq);
            tma_load_rows(y2 + c * L::kChunkBytes, &tmDO, y_full + st, c * 64, i * T, hq, b, p.odo);
          }
          if constexpr (F::kUsesStats) {
            const long long off = (static_cast<long long>(b) * p.heads + hq) * p.seq_q_pad + i * T;
            bulk_load(sStats + st * 2 * T, p.lse2 + off, T * 4, y_full + st);
            bulk_load(sStats + st * 2 * T + T, p.delta + off, T * 4, y_full + st);
          }
        }
      }
    }
  } else if (warp == kBwdRowThreads / 32 + 1) {
    // ======================= issuing warp: every MMA =======================
    if (lane == 0 && start_ok && n_iter > 0) {
      constexpr uint32_t idesc_kk = make_idesc_f16(T, T, kBf16, false, false);      // S, dP: both operands K-major
      constexpr uint32_t idesc_mn = make_idesc_f16(T, D, kBf16, false, true);       // accumulators: B = streamed tile, MN-major
      constexpr uint64_t kChunk = L::kChunkBytes >> 4;
      const uint64_t x1_desc = make_smem_desc(smem_u32(sX1), 16, 1024), x2_desc = make_smem_desc(smem_u32(sX2), 16, 1024);
      bool ok = mbar_wait_poll(x_full, 0, ab, kBwdXFull);
      auto stage_descs = [&](int st, uint64_t& y1_desc, uint64_t& y2_desc, uint64_t& y1_mn, uint64_t& y2_mn) {
        const uint32_t y1a = smem_u32(sY + st * L::kStageBytes), y2a = y1a + L::kTileBytes;
        y1_desc = make_smem_desc(y1a, 16, 1024);
        y2_desc = make_smem_desc(y2a, 16, 1024);
        y1_mn = make_smem_desc(y1a, L::kChunkBytes, 1024);
        y2_mn = make_smem_desc(y2a, L::kChunkBytes, 1024);
      };
      auto issue_s_dp = [&](uint64_t y1_desc, uint64_t y2_desc) {
#pragma unroll
        for (int ch = 0; ch < KC; ++ch)
          umma_ss_x4<2, 2>(tmem_base + kColS, x1_desc + ch * kChunk, y1_desc + ch * kChunk, idesc_kk, ch > 0 ? 1u : 0u);
#pragma unroll
        for (int ch = 0; ch < KC; ++ch)
          umma_ss_x4<2, 2>(tmem_base + kColDP, x2_desc + ch * kChunk, y2_desc + ch * kChunk, idesc_kk, ch > 0 ? 1u : 0u);
        umma_commit(s_done);
      };
      uint64_t y1_desc, y2_desc, y1_mn, y2_mn;
      if constexpr (kRoleQ) {
        // S, dP of tile it + 1 are issued as soon as the row threads hold those of tile it in registers, ahead of
        // tile it's accumulating MMA (dS sits in a buffer of its own)
        if (ok && mbar_wait_poll(y_full, 0, ab, kBwdYFull)) {
          tc_fence_after_sync();
          stage_descs(0, y1_desc, y2_desc, y1_mn, y2_mn);
          issue_s_dp(y1_desc, y2_desc);
        } else {
          ok = false;
        }
        for (int it = 0; ok && it < n_iter; ++it) {
          const int st = it & 1;
          const uint64_t y1_mn_cur = y1_mn;
          if (it + 1 < n_iter) {
            if (!(mbar_wait_poll(y_full + (st ^ 1), ((it + 1) >> 1) & 1, ab, kBwdYFull) && mbar_wait_poll(sdp_free, it & 1, ab, kBwdSdpFree))) break;
            tc_fence_after_sync();
            stage_descs(st ^ 1, y1_desc, y2_desc, y1_mn, y2_mn);
            issue_s_dp(y1_desc, y2_desc);
          }
          if (!mbar_wait_poll(p_ready, it & 1, ab, kBwdPReady)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ts_x4<8, 128>(tmem_base + kColA, tmem_base + kColDS + st * 64 + g * 32, y1_mn_cur + g * 512, idesc_mn, (it > 0 || g > 0) ? 1u : 0u);
          umma_commit(y_empty + st);
          if (it + 1 == n_iter) umma_commit(acc_done);
        }
      } else {
        for (int it = 0; ok && it < n_iter; ++it) {
          const int st = it & 1;
          if (!mbar_wait_poll(y_full + st, (it >> 1) & 1, ab, kBwdYFull)) break;
          tc_fence_after_sync();
          stage_descs(st, y1_desc, y2_desc, y1_mn, y2_mn);
          // the pipe runs in issue order: P and dS of the tile before have been consumed when these overwrite them
          issue_s_dp(y1_desc, y2_desc);
          if (!mbar_wait_poll(p_ready, it & 1, ab, kBwdPReady)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ts_x4<8, 128>(tmem_base + kColA, tmem_base + kColS + g * 32, y2_mn + g * 512, idesc_mn, (it > 0 || g > 0) ? 1u : 0u);
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ts_x4<8, 128>(tmem_base + kColB, tmem_base + kColDP + g * 32, y1_mn + g * 512, idesc_mn, (it > 0 || g > 0) ? 1u : 0u);
          umma_commit(y_empty + st);
          if (it + 1 == n_iter) umma_commit(acc_done);
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
    bool ok = start_ok;
    for (int it = 0; ok && it < n_iter; ++it) {
      const int st = it & 1;
      // the streamed tile index, and whether it meets the resident tile on the diagonal of a causal mask
      const int ys = kRoleQ ? it : i0 + it % max(per_head, 1);
      const bool diag = p.causal && ys == tile;
      ok = mbar_wait(y_full + st, (it >> 1) & 1, ab, kBwdYFull);   // the statistics came with the tile
      ok = mbar_wait(s_done, it & 1, ab, kBwdSDone) && ok;
      if (!ok) break;
      tc_fence_after_sync();
      const float* st_lse = sStats + st * 2 * T;
      const float* st_delta = st_lse + T;
      uint32_t pp[32], pds[32];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c0 = wg * 64 + u * 32;
        float s[32], dp[32];
        tmem_ld32f(tS + c0, s);
        tmem_ld32f(tDP + c0, dp);
        tmem_wait_ld();
        if (kRoleQ && u == 1) {   // this tile's S and dP are in registers: the next tile's may be computed
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(sdp_free);
        }
        // the functor gives P and dS = dP * dP/dS (softmax: through lse and delta) for one element
        const int hq = kRoleQ ? hx : hx * p.kv_group + it / max(per_head, 1);
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          // KV role: the statistics belong to the columns and sit in shared memory; every lane reads the same four
          // at a time (one broadcast load per four columns instead of one per column and statistic)
          float l2 = 0.0f, dl = 0.0f;
          if constexpr (F::kUsesStats) {
            if constexpr (kRoleQ) {
              l2 = lse2_r;
              dl = delta_r;
            } else {
              const float4 l4 = *reinterpret_cast<const float4*>(st_lse + c0 + (k & ~3));
              const float4 d4 = *reinterpret_cast<const float4*>(st_delta + c0 + (k & ~3));
              l2 = (k & 3) == 0 ? l4.x : (k & 3) == 1 ? l4.y : (k & 3) == 2 ? l4.z : l4.w;
              dl = (k & 3) == 0 ? d4.x : (k & 3) == 1 ? d4.y : (k & 3) == 2 ? d4.z : d4.w;
            }
          }
          const int q_idx = kRoleQ ? tile * T + row : ys * T + c0 + k;
          const int kv_idx = kRoleQ ? ys * T + c0 + k : tile * T + row;
          // causal: keep kv <= q.  KV role: lanes are KV rows, columns query rows; query role the other way round.
          // A functor whose P vanishes at a score of -inf (softmax) gets the mask through the score
          const bool masked = diag && (kRoleQ ? (c0 + k > row) : (c0 + k < row));
          float pr, ds;
          F::apply((F::kNegInfMask && masked) ? -INFINITY : s[k], dp[k], l2, dl, fctx, b, hq, q_idx, kv_idx, pr, ds);
          if (!F::kNegInfMask && masked) pr = ds = 0.0f;
          s[k] = pr;
          dp[k] = ds;
        }
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          pp[u * 16 + k] = pack2<kBf16>(s[2 * k], s[2 * k + 1]);
          pds[u * 16 + k] = pack2<kBf16>(dp[2 * k], dp[2 * k + 1]);
        }
      }
      // the 16-bit pairs of columns [64 wg, 64 wg + 64) go to 32-bit columns [32 wg, 32 wg + 32), which the other warp
      // of this lane quarter reads as fp32: both must have their values in registers first
      if constexpr (kRoleQ) {
        tmem_st32(tmem_base + lane_base + kColDS + st * 64 + wg * 32, pds);
      } else {
        tc_fence_before_sync();
        ok = named_sync_and(1 + wq, 64, ok);
        if (!ok) break;
        tc_fence_after_sync();
        tmem_st32(tS + wg * 32, pp);
        tmem_st32(tDP + wg * 32, pds);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // ---- epilogue: the accumulators as 16-bit rows ----
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
              pk.x = pack2<kBf16>(v[8 * q4 + 0], v[8 * q4 + 1]);
              pk.y = pack2<kBf16>(v[8 * q4 + 2], v[8 * q4 + 3]);
              pk.z = pack2<kBf16>(v[8 * q4 + 4], v[8 * q4 + 5]);
              pk.w = pack2<kBf16>(v[8 * q4 + 6], v[8 * q4 + 7]);
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
  int batch, heads, heads_kv, seq_q, seq_kv, dim, dtype, causal;
  float scale;
  const int64_t *q_stride, *k_stride, *v_stride, *do_stride, *dq_stride, *dk_stride, *dv_stride;
  const float* lse2;
  const float* delta;
  const void* const* custom;
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
  p.causal = a.causal;
  p.scale = a.scale;
  for (int i = 0; i < 3; ++i) {
    p.dq_s[i] = a.dq_stride[i];
    p.dk_s[i] = a.dk_stride[i];
    p.dv_s[i] = a.dv_stride[i];
  }
  for (int i = 0; i < ATTN_B200_MAX_CUSTOM; ++i) p.custom[i] = a.custom != nullptr ? a.custom[i] : nullptr;
  p.status = status;
  auto kv_kernel = attn_bwd_kernel<F, false, kBf16, D>;
  auto q_kernel = attn_bwd_kernel<F, true, kBf16, D>;
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
