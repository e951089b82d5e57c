// Kernel family (2): chunked linear attention / retention forward for sm_100a.
//
//   o_i = sum_{j<=i} exp(G_i - G_j) (scale * q_i . k_j) v_j,      G = cumulative sum of log_decay
//
// evaluated block by block with a running state, the chunked ("recurrent") pattern of the
// reference (attention_engine/core/template/tl_template/linear/linear_tl.py: chunk-local cumsum
// :36-60, state kernel chunk_fwd_h :146-223, output kernel chunk_o :321-401, wrapper :1240-1268):
//
//   S        = Q K^T                                  [tokens x tokens]   (tcgen05, SS)
//   P_ij     = scale * S_ij * exp(g_i - g_j), j <= i   (threads, one row each; written to TMEM)
//   O        = diag(scale * exp(g)) (Q h) + P V        (tcgen05: SS into O, row rescale, TS on top)
//   h       <- exp(g_last) h + (V * exp(g_last - g))^T K
//
// with g the cumulative log-decay inside the block.  Differences from the reference design:
// one fused kernel instead of cumsum + state + output kernels; the state never goes to HBM (the
// reference writes every chunk's state as bf16, 1.07 GB at B=8 H=8 S=4096 256/512, and reads it
// back); the state is kept in fp32 in tensor memory, only its MMA operand copy is bf16.  Blocks
// are 128 tokens (the MMA M) instead of the reference's default 64; the result does not depend on
// the block size.
//
// One CTA per (128-column slice of dim_v, batch*head), walking the sequence in 128-token blocks.
// The state is held transposed, hT[dv_slice=128][dim_qk], so that its MMAs have M = 128 for any
// dim_qk: TMEM columns [0, DK) = hT, [256, 384) = S / P, [384, 512) = O.
// Shared memory: Q, K (DK/64 chunks of 128 rows x 128 B each), V (2 chunks), bf16 hT (DK/64 chunks;
// its lower 32 KB also stage the output rows, with dim_qk 256 its upper 32 KB hold the rescaled V).
// Eight row warps (thread = TMEM lane x column half) and one issuing warp that launches every TMA copy
// and MMA; they hand work to each other through mbarriers, and the order in which the issuing warp
// serves them is the schedule of a block (see the comment at its loop).
#include <cstring>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "parallel_launch.cuh"  // tensor_map_encoder()
#include "sm100.cuh"

namespace b200 {

constexpr int kLinT = 128;    // tokens per block
constexpr int kLinDvs = 128;  // dim_v columns per CTA
constexpr int kLinRowThreads = 256;              // eight warps: one TMEM lane each, two column halves
constexpr int kLinThreads = kLinRowThreads + 64;   // plus the warp that issues TMA copies and MMAs and the decay-scan warp

struct LinearParams {
  void* o;                 // [B,H,S,DV] 16-bit
  float* o_f32;            // [B,H,S,DV] fp32 output instead (rows are written straight from registers), or null
  const float* log_decay;  // [B,H,S] natural log of the per-token decay
  const float* v_scale;    // [B,H,S] per-token factor on the rows of v, or null
  float* stats;            // [B,H,S,2] (sum, sum of squares) over dim_v, or null
  int seq, dim_v, bh;
  int heads, heads_q, heads_k;   // heads of v; of q and k (divisors of `heads`: consecutive v heads share a q / k head)
  float q_scale;
  int split_p;             // 1: P is written as a 16-bit high part plus a 16-bit remainder (two PV passes)
  int* status;
};

__device__ __forceinline__ float clamp_h(float x) { return fminf(fmaxf(x, -65504.0f), 65504.0f); }

enum LinearWaitSite { kLinQFull = 41, kLinKFull, kLinScore, kLinQh, kLinPv, kLinState, kLinPReady, kLinVReady, kLinOStaged, kLinStageFree, kLinConvDone, kLinVFull, kLinDecay, kLinHiReady };
enum LinearBarrier { kBarQFull = 0, kBarKFull, kBarVFull, kBarScore, kBarHiReady, kBarPv, kBarState, kBarPReady, kBarVReady, kBarConvDone, kBarDecay, kNumLinBarriers };

template <int DK>
struct LinearSmem {
  static constexpr int kQBytes = kLinT * DK * 2;
  static constexpr int kVBytes = kLinT * kLinDvs * 2;
  // K and the operand copy of the state, interleaved by 64-column chunk of dim_qk: chunk c holds the 128 rows of K
  // (tokens) and then the 128 rows of the copy (dim_v), so that one N = 256 B operand yields [S | O] = Q [K^T | h].
  // The copy's part of chunks 0 and 1 also stages one block of output rows.
  static constexpr int kChunkBytes = kLinT * 128;
  static constexpr int kPairBytes = 2 * kChunkBytes;
  static constexpr int kKhBytes = (DK / 64) * kPairBytes;
  static constexpr int kStageExtra = DK == 64 ? kChunkBytes : 0;   // the second group's staged rows with a one-chunk copy
  static constexpr int kOffQ = 0;
  static constexpr int kOffKh = kOffQ + kQBytes;
  static constexpr int kOffV = kOffKh + kKhBytes;
  static constexpr int kOffStageX = kOffV + kVBytes;
  // rows of V times their decay factors, the A operand of the state update when the decay is not mild: with dim_qk
  // 256 the copy's part of chunks 2 and 3 (idle between the Q h MMA and the conversion pass), else a buffer of its own
  static constexpr bool kScaledVInH = (DK == 256);
  static constexpr int kOffV2 = kScaledVInH ? kOffKh + 2 * kPairBytes + kChunkBytes : kOffStageX + kStageExtra;
  static constexpr int kV2Stride = kScaledVInH ? kPairBytes : kChunkBytes;
  static constexpr int kOffG = kOffStageX + kStageExtra + (kScaledVInH ? 0 : kVBytes);  // float g2[2][128] + float gb[128]
  static constexpr int kOffBar = kOffG + 3 * kLinT * 4 + 32;
  static constexpr int kOffMisc = kOffBar + 8 * kNumLinBarriers;
  static constexpr int kBytes = kOffMisc + 16 + 1024;
};

template <int DK, bool kBf16>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const LinearParams p) {
  using L = LinearSmem<DK>;
  constexpr int T = kLinT, DVS = kLinDvs, KC = DK / 64;
  static_assert(DK % 64 == 0 && DK <= 256, "unsupported dim_qk");
  constexpr uint32_t kTmemCols = 512, kColH = 0, kColS = 256, kColO = 384;
  constexpr float kLog2e = 1.4426950408889634f;
  // A block whose total log2-decay is at least this is "mild": see the row threads' loop
  // (never with the remainder pass of P, which exists for the accuracy the rounded rows of V would give away)
  const float kMildLog2 = p.split_p ? 1.0f : (kBf16 ? -100.0f : -8.0f);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sKh = smem + L::kOffKh;
  uint8_t* sV = smem + L::kOffV;
  uint8_t* sStageX = smem + L::kOffStageX;
  uint8_t* sV2 = smem + L::kOffV2;
  float* g2 = reinterpret_cast<float*>(smem + L::kOffG);  // [2][T] cumulative log2-decay inside a block
  float* gb = g2 + 2 * T;   // [T] exp2(g at the end of the column's 32-token chunk - g of the column), current block
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + kBarQFull;
  uint64_t* k_full = bars + kBarKFull;
  uint64_t* v_full = bars + kBarVFull;
  uint64_t* s_bar = bars + kBarScore;
  uint64_t* hi_ready = bars + kBarHiReady;
  uint64_t* pv_bar = bars + kBarPv;
  uint64_t* st_bar = bars + kBarState;
  uint64_t* p_ready = bars + kBarPReady;
  uint64_t* v_ready = bars + kBarVReady;
  uint64_t* conv_done = bars + kBarConvDone;
  uint64_t* g_ready = bars + kBarDecay;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = (warp >> 2) & 1;           // row warps: column half owned in the row phases
  const int row = (warp & 3) * 32 + lane;   // TMEM lane owned by a row thread
  const AbortState ab{abort_flag, p.status};
  const int slice = blockIdx.x;
  const int bh = blockIdx.y;
  const int nblk = (p.seq + T - 1) / T;
  const float* ld_row = p.log_decay + static_cast<long long>(bh) * p.seq;
  const int b_idx = bh / p.heads, h_idx = bh - b_idx * p.heads;
  const int bh_q = b_idx * p.heads_q + h_idx / (p.heads / p.heads_q), bh_k = b_idx * p.heads_k + h_idx / (p.heads / p.heads_k);

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_bar, 1);
    mbar_init(hi_ready, kLinRowThreads / 32);
    mbar_init(pv_bar, 1);
    mbar_init(st_bar, 1);
    mbar_init(p_ready, kLinRowThreads / 32);
    mbar_init(v_ready, kLinRowThreads / 32);
    mbar_init(conv_done, kLinRowThreads / 32);
    mbar_init(g_ready, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
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

  if (warp == kLinRowThreads / 32) {
    // ======================= issuing warp: every TMA copy and every MMA =======================
    if (lane == 0 && start_ok) {
      auto load_q = [&](int t) {
        mbar_arrive_expect_tx(q_full, L::kQBytes);
        for (int c = 0; c < KC; ++c) tma_load_3d(sQ + c * (T * 128), &tmQ, q_full, c * 64, t * T, bh_q);
      };
      auto load_k = [&](int t) {
        mbar_arrive_expect_tx(k_full, L::kQBytes);
        for (int c = 0; c < KC; ++c) tma_load_3d(sKh + c * L::kPairBytes, &tmK, k_full, c * 64, t * T, bh_k);
      };
      auto load_v = [&](int t) {
        mbar_arrive_expect_tx(v_full, L::kVBytes);
        for (int c = 0; c < DVS / 64; ++c) tma_load_3d(sV + c * (T * 128), &tmV, v_full, slice * DVS + c * 64, t * T, bh);
      };
      // kind::f16 takes one 16-bit format for both operands: a variant with fp16 intermediates next to
      // bf16 inputs (A and B formats differing) raised a CUDA fault on B200 and is not offered.
      constexpr uint32_t idesc_s = make_idesc_f16(T, T, kBf16, false, false);          // S = Q K^T (first block)
      constexpr uint32_t idesc_sq = make_idesc_f16(T, T + DVS, kBf16, false, false);   // [S | O] = Q [K^T | hT^T]
      constexpr uint32_t idesc_pv = make_idesc_f16(T, DVS, kBf16, false, true);        // O += P V   (B = V, MN-major)
      constexpr uint32_t idesc_h = make_idesc_f16(DVS, DK, kBf16, true, true);         // hT += V'^T K (A M-major, B MN-major)
      // descriptors are built once; the issue loops only move the start-address field (units of 16 bytes)
      const uint64_t q_desc0 = make_smem_desc(smem_u32(sQ), 16, 1024), kh_desc0 = make_smem_desc(smem_u32(sKh), 16, 1024);
      const uint64_t v_mn_desc0 = make_smem_desc(smem_u32(sV), T * 128, 1024);
      const uint64_t k_mn_desc0 = make_smem_desc(smem_u32(sKh), L::kPairBytes, 1024);
      const uint64_t v2_mn_desc0 = make_smem_desc(smem_u32(sV2), L::kV2Stride, 1024);
      constexpr uint64_t kChunk = (T * 128) >> 4, kPair = L::kPairBytes >> 4;
      static_assert(kColO == kColS + T, "S and O are the two halves of one accumulator");
      // Chunks [c0, c1) of dim_qk of [S | O] = Q [K^T | hT^T]: the K rows and the rows of the state's copy of a chunk
      // lie one after the other, so both products share the reads of Q.  In the first block there is no state yet
      // and only S is computed (P V then starts O afresh).
      auto issue_sq = [&](int t, int c0, int c1, bool fresh) {
        for (int ch = c0; ch < c1; ++ch)
          umma_ss_x4<2, 2>(tmem_base + kColS, q_desc0 + ch * kChunk, kh_desc0 + ch * kPair, t == 0 ? idesc_s : idesc_sq,
                           (fresh && ch == c0) ? 0u : 1u);
      };
      // The copy's columns [0, 128) (chunks 0 and 1) are converted last, because their place stages the output rows;
      // the chunks from 2 on are ready earlier and their share of [S | O] of the coming block is issued as soon as the
      // row threads have read this block's O.
      constexpr int kLoChunks = KC < 2 ? KC : 2;

      // The tensor pipe executes in issue order and the issuing thread is held back while the pipe is full,
      // so the order below is the schedule.  Per block: the rest of [S | O], the state update (with mild decay its
      // operand is waiting), Q and K of the next block, P V, V of the next block, the early chunks of the next [S | O].
      load_q(0);
      load_k(0);
      load_v(0);
      for (int t = 0; t < nblk; ++t) {
        const bool last = (t + 1 == nblk);
        const uint32_t par = t & 1, par_prev = (t - 1) & 1;
        if (t == 0 || KC <= kLoChunks) {
          if (t > 0 && !mbar_wait_poll(conv_done, par_prev, ab, kLinConvDone)) break;
          if (!(mbar_wait_poll(q_full, par, ab, kLinQFull) && mbar_wait_poll(k_full, par, ab, kLinKFull))) break;
          tc_fence_after_sync();
          issue_sq(t, 0, KC, true);
        } else {
          if (!mbar_wait_poll(conv_done, par_prev, ab, kLinConvDone)) break;
          tc_fence_after_sync();
          issue_sq(t, 0, kLoChunks, false);
        }
        umma_commit(s_bar);
        if (!last) {
          // hT (+)= V'^T K; both operands are MN-major over tokens: 16 tokens = 2048 B per K step.  It follows [S | O]
          // in the pipe: the row threads take its completion to mean that the state's copy is no longer read.
          if (!mbar_wait_poll(v_ready, par, ab, kLinVReady)) break;
          tc_fence_after_sync();
          const bool mild = g2[(t & 1) * T + T - 1] >= kMildLog2;
          const uint64_t va_desc0 = mild ? v_mn_desc0 : v2_mn_desc0;
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ss_x4<128, 128>(tmem_base + kColH, va_desc0 + g * 512, k_mn_desc0 + g * 512, idesc_h, (t > 0 || g > 0) ? 1u : 0u);
          umma_commit(st_bar);
        }
        // Q may be replaced once [S | O] has run, K once the state update has
        if (!mbar_wait_poll(s_bar, par, ab, kLinScore)) break;
        if (!last) {
          load_q(t + 1);
          if (!mbar_wait_poll(st_bar, par, ab, kLinState)) break;
          load_k(t + 1);
        }
        // O (+)= P V
        if (!(mbar_wait_poll(p_ready, par, ab, kLinPReady) && mbar_wait_poll(v_full, par, ab, kLinVFull))) break;
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < T / 64; ++g)
          umma_ts_x4<8, 128>(tmem_base + kColO, tmem_base + kColS + g * 32, v_mn_desc0 + g * 512, idesc_pv, (t > 0 || g > 0) ? 1u : 0u);
        if (p.split_p) {
#pragma unroll
          for (int g = 0; g < T / 64; ++g)
            umma_ts_x4<8, 128>(tmem_base + kColO, tmem_base + kColS + 64 + g * 32, v_mn_desc0 + g * 512, idesc_pv, 1u);
        }
        umma_commit(pv_bar);
        if (last) break;
        if (!mbar_wait_poll(pv_bar, par, ab, kLinPv)) break;
        load_v(t + 1);  // V was read by the row threads and by P V
        if (KC > kLoChunks) {
          // P of this block is consumed (P V has run); O is free once every row warp has read it
          if (!(mbar_wait_poll(hi_ready, par, ab, kLinHiReady) && mbar_wait_poll(q_full, par ^ 1, ab, kLinQFull) &&
                mbar_wait_poll(k_full, par ^ 1, ab, kLinKFull)))
            break;
          tc_fence_after_sync();
          issue_sq(t + 1, kLoChunks, KC, true);
        }
      }
    }
  } else if (warp == kLinRowThreads / 32 + 1) {
    // ======================= decay warp: the scan of every block's log-decays =======================
    // Four consecutive tokens per lane.  Block t's table goes into g2[t & 1] (read by the row threads of block t and,
    // its last entry, by those of block t - 1) and gb (read by block t's P phase only), so it may be written once the
    // row threads are through the P phase of block t - 1.
    bool ok = start_ok;
    for (int t = 0; ok && t < nblk; ++t) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int tok = t * T + lane * 4 + k;
        x[k] = tok < p.seq ? ld_row[tok] * kLog2e : 0.0f;
      }
      x[1] += x[0];
      x[2] += x[1];
      x[3] += x[2];
      float run = x[3];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, run, d);
        if (lane >= d) run += y;
      }
      const float pre = run - x[3];
      const float g_end = __shfl_sync(0xffffffffu, run, lane | 7);   // last token of this lane's 32-token chunk
      if (t > 0 && lane == 0) ok = mbar_wait_poll(p_ready, (t - 1) & 1, ab, kLinDecay);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float g = pre + x[k];
        g2[(t & 1) * T + lane * 4 + k] = g;
        gb[lane * 4 + k] = fast_exp2(g_end - g);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(g_ready);
    }
  } else {
    // ======================= row threads: one TMEM lane (token / state row) each =======================
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tH = tmem_base + lane_base + kColH;
    const uint32_t tS = tmem_base + lane_base + kColS;
    const uint32_t tO = tmem_base + lane_base + kColO;
    // one arrival per warp: the lanes' writes are ordered before it by the warp barrier
    auto warp_arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    // 32 columns of this thread's state row: 16-bit copy to the operand buffer, and the decay of the next block
    // onto hT.  Group `wg` owns columns [64 wg, 64 wg + 64), whose place in the buffer staged its own output rows,
    // and its share of the columns from 128 on, which are free as soon as the state update has run.
    constexpr int kEarlyCols = DK > 128 ? (DK - 128) / 2 : 0;   // per group
    auto convert32 = [&](int col0, float decay_next, bool scaled_copy) {
      float hv[32];
      tmem_ld32f(tH + col0, hv);
      tmem_wait_ld();
      if (scaled_copy) {
#pragma unroll
        for (int i = 0; i < 32; ++i) hv[i] *= decay_next;
      }
      uint8_t* line = sKh + (col0 >> 6) * L::kPairBytes + L::kChunkBytes + row * 128;
      const int piece0 = (col0 & 63) >> 3;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 pk;
        pk.x = pack2<kBf16>(hv[8 * q4 + 0], hv[8 * q4 + 1]);
        pk.y = pack2<kBf16>(hv[8 * q4 + 2], hv[8 * q4 + 3]);
        pk.z = pack2<kBf16>(hv[8 * q4 + 4], hv[8 * q4 + 5]);
        pk.w = pack2<kBf16>(hv[8 * q4 + 6], hv[8 * q4 + 7]);
        *reinterpret_cast<uint4*>(line + (((piece0 + q4) ^ (row & 7)) << 4)) = pk;
      }
      if (!scaled_copy) {
#pragma unroll
        for (int i = 0; i < 32; ++i) hv[i] *= decay_next;
      }
      tmem_st32f(tH + col0, hv);
    };

    // Rows of V times their decay factors, the A operand of the state update: token `row` of block tb's V (chunk `wg`)
    // is multiplied by exp(g_last - g_row).  Every 16-byte piece of the row gets the same factor, so neither the
    // swizzle nor the order matters: lanes start at different pieces to stay off each other's banks (rows are 128
    // bytes apart).  With mild decay the result replaces V (P V then takes the same rows), which touches nothing
    // another phase of the kernel uses; else it goes to the second buffer (with 256 state columns the upper half of
    // the state copy, free once Q h has run).
    auto rescale_v = [&](int tb, bool in_place) -> bool {
      // a per-token factor of the caller on v (v_mod = v * t[b, h, token]) rides along: fetched before the wait for V
      const int tok = tb * T + row;
      const float vs = (p.v_scale != nullptr && tok < p.seq) ? p.v_scale[static_cast<long long>(bh) * p.seq + tok] : 1.0f;
      const bool v_ok = mbar_wait(v_full, tb & 1, ab, kLinVFull);
      const float* g = g2 + (tb & 1) * T;
      const float w = fast_exp2(g[T - 1] - g[row]) * vs;
      uint4* vsrc = reinterpret_cast<uint4*>(sV + wg * (T * 128) + row * 128);
      const uint4* vline = vsrc;
      uint4* v2line = reinterpret_cast<uint4*>((in_place ? sV + wg * (T * 128) : sV2 + wg * L::kV2Stride) + row * 128);
      // with strong decay P V reads V itself: the caller's factor then goes onto V in place as well
      const bool scale_v_too = !in_place && p.v_scale != nullptr;
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        const int piece = (q4 + lane) & 7;
        uint4 x = vline[piece];
        uint4 y = x;
        uint32_t* xs = reinterpret_cast<uint32_t*>(&x);
        uint32_t* ys = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          if constexpr (kBf16) {
            const __nv_bfloat162 h2 = *reinterpret_cast<__nv_bfloat162*>(&xs[e]);
            lo = __bfloat162float(h2.x);
            hi = __bfloat162float(h2.y);
          } else {
            const __half2 h2 = *reinterpret_cast<__half2*>(&xs[e]);
            lo = __half2float(h2.x);
            hi = __half2float(h2.y);
          }
          xs[e] = pack2<kBf16>(lo * w, hi * w);
          if (scale_v_too) ys[e] = pack2<kBf16>(lo * vs, hi * vs);
        }
        v2line[piece] = x;
        if (scale_v_too) vsrc[piece] = y;
      }
      fence_proxy_async_smem();
      if (tb + 1 < nblk) warp_arrive(v_ready);
      return v_ok;
    };

    bool ok = start_ok && mbar_wait(g_ready, 0, ab, kLinDecay);
    if (ok && g2[T - 1] >= kMildLog2) ok = rescale_v(0, true);
    for (int t = 0; ok && t < nblk; ++t) {
      const int buf = t & 1;
      const bool last = (t + 1 == nblk);
      const uint32_t par = t & 1;
      const float gi = g2[buf * T + row];
      const float qs = p.q_scale;
      // Mild decay (the block's total log2-decay stays inside the exponent range of the 16-bit operands with room
      // to spare): exp(g_i - g_j) is split as exp(g_i - g_last) * exp(g_last - g_j).  The second factor is the one
      // the state update puts on the rows of V anyway, so the rescaled rows replace V and serve P V too; the first
      // is a row factor that P V shares with Q h once the state's copy is taken after the block's decay
      // (Q_i h exp(g_i) = Q_i (h exp(g_last)) exp(g_i - g_last)), and is applied once, to the finished output row.
      // P is then the masked scores themselves, O = Q h needs no pass between the two MMAs, and the rows of V are
      // rescaled a block ahead, while the output rows of the block before are being stored.  Blocks with a stronger decay (gated linear attention) keep every factor <= 1:
      // exp(g_i - g_j) in P, a rescale of Q h by exp(g_i), and the rescaled V in a buffer of its own.
      const float g_last = g2[buf * T + T - 1];
      const bool mild = g_last >= kMildLog2;
      if (!mild) {
        ok = mbar_wait(s_bar, par, ab, kLinQh);   // Q h has run: O may be rescaled, the copy's upper chunks overwritten
        tc_fence_after_sync();
      }
      // ---- rows of V times their decay factors (mild decay: done in the previous block's tail) ----
      if ((!last || p.v_scale != nullptr) && !mild) ok = rescale_v(t, false) && ok;
      // ---- rows of O = Q h scaled by scale * exp(g_i) ----
      if (t > 0 && !mild) {
        const float f = qs * fast_exp2(gi);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float o[32];
          tmem_ld32f(tO + wg * 64 + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= f;
          tmem_st32f(tO + wg * 64 + c * 32, o);
        }
      }
      // ---- rows of S -> P (while Q h still runs) ----
      // Both warp groups work on every row: group `wg` owns columns [64*wg, 64*wg+64) of S and of O (a single
      // warp per scheduler running dependent arithmetic is latency-bound; two interleave).
      uint32_t pk[32], pl[32];
      {
        // exp(g_i - g_j) costs one MUFU operation per score only in the 32x32 chunk on the diagonal.  Below
        // it the factor splits into exp(g_i - g_end) * exp(g_end - g_j), g_end the last token of the column
        // chunk: a per-row and a per-column number, both at most 1.  Chunks above the diagonal are zero and
        // are not even read.  All three cases are uniform over a warp.
        const int wq = warp & 3;
        ok = mbar_wait(s_bar, par, ab, kLinScore) && ok;
        tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = 2 * wg + h;  // 32-column chunk of S
          uint32_t* pkh = pk + 16 * h;
          uint32_t* plh = pl + 16 * h;
          if (c > wq) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pkh[i] = plh[i] = 0u;
            continue;
          }
          float s[32];
          tmem_ld32f(tS + c * 32, s);
          tmem_wait_ld();
          const float* gcol = g2 + buf * T + c * 32;
          const float* bcol = gb + c * 32;
          if (mild) {
            // the column factors are in the rows of V already: only the mask is left
            if (c == wq) {
#pragma unroll
              for (int i = 0; i < 32; ++i) s[i] = (i <= lane) ? s[i] : 0.0f;
            }
          } else if (c < wq) {
            const float a = qs * fast_exp2(fminf(gi - gcol[31], 0.0f));
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] *= a * bcol[i];
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              // computed for every column and selected afterwards: a per-lane branch here diverges in every warp
              const float e = s[i] * qs * fast_exp2(fminf(gi - gcol[i], 0.0f));
              s[i] = (i <= lane) ? e : 0.0f;
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) pkh[i] = pack2<kBf16>(s[2 * i], s[2 * i + 1]);
          if (p.split_p) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float h0, h1;
              if constexpr (kBf16) {
                const __nv_bfloat162 h2 = *reinterpret_cast<__nv_bfloat162*>(&pkh[i]);
                h0 = __bfloat162float(h2.x);
                h1 = __bfloat162float(h2.y);
              } else {
                const __half2 h2 = *reinterpret_cast<__half2*>(&pkh[i]);
                h0 = __half2float(h2.x);
                h1 = __half2float(h2.y);
              }
              plh[i] = pack2<kBf16>(s[2 * i] - h0, s[2 * i + 1] - h1);
            }
          }
        }
        // P overwrites S: 16-bit pairs in columns [0, 64), and with split_p the 16-bit remainder P - round(P) in
        // columns [64, 128) for a second PV pass.  Those columns belong to the other group's half of the same rows
        // of S, so the two warps of a lane quarter must both have their S values in registers first.
        tc_fence_before_sync();
        ok = named_sync_and(1 + (warp & 3), 64, ok);
        if (!ok) break;
        tc_fence_after_sync();
        tmem_st32(tS + wg * 32, pk);
        if (p.split_p) tmem_st32(tS + 64 + wg * 32, pl);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      warp_arrive(p_ready);
      // ---- 16-bit copy of hT for the next block's Q h; hT *= exp(g_last of the next block) ----
      // The staged output rows occupy the first 32 KB of the copy's buffer, i.e. its columns [0, 128).  With more
      // columns every group converts its share of the rest as soon as the state update has run (with 256 that half
      // held the rescaled V), under P V, and its own 64 once the output store has read the staged rows.
      float decay_next = 1.0f;
      bool mild_next = false;   // the coming block multiplies Q by the state after its decay
      if (!last) {
        ok = mbar_wait(g_ready, (t + 1) & 1, ab, kLinDecay) && ok;   // written once every warp was past the P phase
        const float g_next = g2[(buf ^ 1) * T + T - 1];
        decay_next = fast_exp2(g_next);
        mild_next = g_next >= kMildLog2;
        ok = mbar_wait(st_bar, par, ab, kLinState) && ok;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kEarlyCols / 32; ++c) convert32(128 + wg * kEarlyCols + c * 32, decay_next, mild_next);
      }
      ok = mbar_wait(pv_bar, par, ab, kLinPv) && ok;
      tc_fence_after_sync();
      // ---- output rows to the staging buffer (while the state update runs) ----
      {
        // The rows go out through shared memory: the buffer of the state's operand copy is idle between the
        // Q.h MMA of this block and the conversion pass at its end.  Group `wg` writes the 64-column chunk
        // `wg` of its row as one swizzled 128-byte line (the layout TMA expects).
        const int tok = t * T + row;
        float sum = 0.f, sq = 0.f;
        uint8_t* stage = (DK == 64 && wg == 1) ? sStageX : sKh + wg * L::kPairBytes + L::kChunkBytes;
        uint8_t* line = stage + row * 128;
        const float fo = mild ? qs * fast_exp2(gi - g_last) : 1.0f;   // the row factor left out of Q h and P (mild decay)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float o[32];
          tmem_ld32f(tO + wg * 64 + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= fo;
          if (p.o_f32 != nullptr) {
            // fp32 output: this thread's 32 columns of its token row, 128 contiguous bytes
            if (tok < p.seq) {
              float4* dst = reinterpret_cast<float4*>(p.o_f32 + (static_cast<long long>(bh) * p.seq + tok) * p.dim_v +
                                                      slice * DVS + wg * 64 + c * 32);
#pragma unroll
              for (int v = 0; v < 8; ++v) dst[v] = make_float4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
          }
#pragma unroll
          for (int v = 0; v < 4 && p.o_f32 == nullptr; ++v) {
            uint4 pk;
            if (p.stats == nullptr) {
              pk.x = pack2<kBf16>(o[8 * v + 0], o[8 * v + 1]);
              pk.y = pack2<kBf16>(o[8 * v + 2], o[8 * v + 3]);
              pk.z = pack2<kBf16>(o[8 * v + 4], o[8 * v + 5]);
              pk.w = pack2<kBf16>(o[8 * v + 6], o[8 * v + 7]);
            } else {
              // normalised by a second pass: staged as fp16 (11 significant bits, clamped to the fp16 range)
              pk.x = pack2<false>(clamp_h(o[8 * v + 0]), clamp_h(o[8 * v + 1]));
              pk.y = pack2<false>(clamp_h(o[8 * v + 2]), clamp_h(o[8 * v + 3]));
              pk.z = pack2<false>(clamp_h(o[8 * v + 4]), clamp_h(o[8 * v + 5]));
              pk.w = pack2<false>(clamp_h(o[8 * v + 6]), clamp_h(o[8 * v + 7]));
            }
            *reinterpret_cast<uint4*>(line + (((c * 4 + v) ^ (row & 7)) << 4)) = pk;
          }
          if (p.stats != nullptr) {
            float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              s0 += o[i];
              s1 += o[i + 1];
              q0 = fmaf(o[i], o[i], q0);
              q1 = fmaf(o[i + 1], o[i + 1], q1);
            }
            sum += s0 + s1;
            sq += q0 + q1;
          }
        }
        if (p.stats != nullptr && tok < p.seq) {
          float* st = p.stats + (static_cast<long long>(bh) * p.seq + tok) * 2;
          atomicAdd(st, sum);
          atomicAdd(st + 1, sq);
        }
        // Each warp stores its own 32 staged rows (4 KB).  The conversion below writes every thread's state row over
        // the line that held its output row, so nothing here crosses warps; the store is given time to read the rows
        // while the warp rescales the coming block's V.
        fence_proxy_async_smem();   // also orders the copy's early chunks, converted above, before the arrival
        tc_fence_before_sync();
        warp_arrive(hi_ready);      // O has been read and the early chunks are in place: the next [S | O] may start
        const int tok0 = t * T + (warp & 3) * 32;
        if (lane == 0 && p.o_f32 == nullptr && tok0 < p.seq) {
          tma_store_3d(&tmO, stage + (warp & 3) * (32 * 128), slice * DVS + wg * 64, tok0, bh);
          tma_store_commit();
        }
      }
      if (last) break;
      if (mild_next) ok = rescale_v(t + 1, true) && ok;
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
      // ---- 16-bit copy of hT, rest: the columns whose place staged the output rows ----
      if (wg * 64 < DK) {
#pragma unroll
        for (int c = 0; c < 2; ++c) convert32(wg * 64 + c * 32, decay_next, mild_next);
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(conv_done);
    }
    if (lane == 0) tma_store_wait_all();   // the staged rows of the last block are still being read
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

// In-place normalisation of every (batch, head, token) row of o over dim_v to zero mean and unit
// variance, from the (sum, sum of squares) the forward kernel accumulated in fp32.  The rows arrive
// staged as fp16 and leave in the output dtype.  One warp per row.
// The same normalisation for an fp32 output buffer (rows written in fp32 by the forward kernel), in place.
__global__ void __launch_bounds__(256) linear_norm_f32_kernel(float* __restrict__ o, const float* __restrict__ stats, long long rows,
                                                            int dim_v, float eps) {
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float mean = stats[2 * r] / dim_v;
  const float var = fmaxf(stats[2 * r + 1] / dim_v - mean * mean, 0.0f);
  const float rstd = rsqrtf(var + eps);
  float* line = o + r * dim_v;
  for (int i = lane; i < dim_v; i += 32) line[i] = (line[i] - mean) * rstd;
}

template <bool kBf16>
__global__ void __launch_bounds__(256) linear_norm_kernel(void* __restrict__ o, const float* __restrict__ stats, long long rows,
                                                        int dim_v, float eps) {
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float mean = stats[2 * r] / dim_v;
  const float var = fmaxf(stats[2 * r + 1] / dim_v - mean * mean, 0.0f);
  const float rstd = rsqrtf(var + eps);
  uint32_t* line = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(o) + 2 * r * dim_v);
  for (int i = lane; i < dim_v / 2; i += 32) {
    uint32_t x = line[i];
    const __half2 h2 = *reinterpret_cast<__half2*>(&x);  // staged as fp16 by the forward kernel
    const float lo = __half2float(h2.x), hi = __half2float(h2.y);
    line[i] = pack2<kBf16>((lo - mean) * rstd, (hi - mean) * rstd);
  }
}

inline int encode_rows3(CUtensorMap* tm, const void* base, int dtype, uint64_t cols, uint64_t rows, uint64_t outer,
                        uint32_t box_rows = kLinT, uint64_t ld = 0) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return ATTN_B200_E_LAUNCH;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  if (ld == 0) ld = cols;
  if (ld < cols || ld % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  cuuint64_t gdim[3] = {cols, rows, outer};
  cuuint64_t gstride[2] = {ld * 2, ld * rows * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == ATTN_B200_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(tm, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ATTN_B200_OK : ATTN_B200_E_UNSUPPORTED;
}

template <int DK, bool kBf16>
int launch_linear(const AttnB200LinearArgs* a, cudaStream_t stream, int* status) {
  using L = LinearSmem<DK>;
  CUtensorMap tmQ, tmK, tmV, tmO;
  const uint64_t bh = static_cast<uint64_t>(a->batch) * a->heads;
  const int heads_q = a->heads_q > 0 ? a->heads_q : a->heads, heads_k = a->heads_k > 0 ? a->heads_k : a->heads;
  if (a->q_ld < 0 || a->k_ld < 0) return ATTN_B200_E_INVALID_ARG;
  int rc = encode_rows3(&tmQ, a->q, a->dtype, DK, a->seq, static_cast<uint64_t>(a->batch) * heads_q, kLinT, a->q_ld);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows3(&tmK, a->k, a->dtype, DK, a->seq, static_cast<uint64_t>(a->batch) * heads_k, kLinT, a->k_ld);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows3(&tmV, a->v, a->dtype, a->dim_v, a->seq, bh);
  if (rc != ATTN_B200_OK) return rc;
  const bool f32_out = a->dtype_out == ATTN_B200_DTYPE_FP32;
  // one warp's 32 rows per store; with an fp32 output the kernel does not use the map: it is encoded over v so that it stays valid
  rc = encode_rows3(&tmO, f32_out ? a->v : a->o, a->dtype, a->dim_v, a->seq, bh, 32);
  if (rc != ATTN_B200_OK) return rc;
  LinearParams p;
  std::memset(&p, 0, sizeof(p));
  p.o = a->o;
  p.o_f32 = f32_out ? static_cast<float*>(a->o) : nullptr;
  p.log_decay = a->log_decay;
  p.v_scale = a->v_scale;
  p.seq = a->seq;
  p.dim_v = a->dim_v;
  p.bh = static_cast<int>(bh);
  p.heads = a->heads;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.q_scale = a->q_scale;
  // The normalised output has an absolute tolerance whatever the head's scale.  For heads with a fast decay the
  // output is mostly the intra-block part, where the 16-bit rounding of P is the largest error (a CPU model of the
  // kernel's arithmetic gives, for gamma = 1 - 2^-5, mean-abs 3.4e-4 on an output of standard deviation 0.25, and
  // 1.1e-4 with the remainder pass), so a second PV pass over the 16-bit remainder of P is spent there.  For slow
  // decays the state path's roundings dominate and the pass changes nothing.
  p.split_p = (a->normalize || a->precise) ? 1 : 0;
  p.status = status;
  const long long rows = static_cast<long long>(bh) * a->seq;
  if (a->normalize) {
    p.stats = static_cast<float*>(a->workspace);
    if (cudaMemsetAsync(p.stats, 0, rows * 2 * sizeof(float), stream) != cudaSuccess) return ATTN_B200_E_LAUNCH;
  }
  auto kernel = linear_fwd_kernel<DK, kBf16>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  dim3 grid(a->dim_v / kLinDvs, static_cast<unsigned>(bh));
  kernel<<<grid, kLinThreads, L::kBytes, stream>>>(tmQ, tmK, tmV, tmO, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  if (a->normalize) {
    const int blocks = static_cast<int>((rows * 32 + 255) / 256);
    if (f32_out) linear_norm_f32_kernel<<<blocks, 256, 0, stream>>>(p.o_f32, p.stats, rows, a->dim_v, a->norm_eps);
    else linear_norm_kernel<kBf16><<<blocks, 256, 0, stream>>>(a->o, p.stats, rows, a->dim_v, a->norm_eps);
    if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  }
  return ATTN_B200_OK;
}

}  // namespace b200

extern "C" {

int64_t attn_b200_linear_workspace_bytes(const AttnB200LinearArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->seq <= 0) return -1;
  return a->normalize ? static_cast<int64_t>(a->batch) * a->heads * a->seq * 2 * 4 : 0;
}

int attn_b200_linear_fwd(const AttnB200LinearArgs* a, void* cuda_stream) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr || a->log_decay == nullptr)
    return ATTN_B200_E_INVALID_ARG;
  if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0) return ATTN_B200_E_INVALID_ARG;
  if (a->dtype != ATTN_B200_DTYPE_FP16 && a->dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a->dtype_out != ATTN_B200_DTYPE_SAME && a->dtype_out != ATTN_B200_DTYPE_FP32) return ATTN_B200_E_INVALID_ARG;
  if (a->dim_v <= 0 || a->dim_v % b200::kLinDvs != 0) return ATTN_B200_E_UNSUPPORTED;
  if (a->heads_q < 0 || a->heads_k < 0 || (a->heads_q > 0 && a->heads % a->heads_q != 0) || (a->heads_k > 0 && a->heads % a->heads_k != 0))
    return ATTN_B200_E_INVALID_ARG;
  if (static_cast<long long>(a->batch) * a->heads > 65535) return ATTN_B200_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  if (a->normalize) {
    const int64_t need = attn_b200_linear_workspace_bytes(a);
    if (a->workspace == nullptr || a->workspace_bytes < need) return ATTN_B200_E_WORKSPACE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ATTN_B200_E_LAUNCH;
  int* status = b200::device_status_word(dev);
  if (status == nullptr) return ATTN_B200_E_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const bool bf16 = a->dtype == ATTN_B200_DTYPE_BF16;
  switch (a->dim_qk) {
    case 64:
      return bf16 ? b200::launch_linear<64, true>(a, stream, status) : b200::launch_linear<64, false>(a, stream, status);
    case 128:
      return bf16 ? b200::launch_linear<128, true>(a, stream, status) : b200::launch_linear<128, false>(a, stream, status);
    case 256:
      return bf16 ? b200::launch_linear<256, true>(a, stream, status) : b200::launch_linear<256, false>(a, stream, status);
    default:
      return ATTN_B200_E_UNSUPPORTED;
  }
}

}  // extern "C"
