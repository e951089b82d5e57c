// Kernel family (3): MLA decode for sm_100a -- one query token per sequence, all query heads
// share one latent KV head; V is the first dim_v columns of the latent KV row.
//
//   o[b,h,:] = softmax_s( scale * q[b,h,:] . kv[b,s,:] ) . kv[b,s,:dim_v]
//
// Replaces the reference's split-KV kernels and their scheduler
// (attention_engine/core/template/cute_template_kvshared/kernels/splitkv_mla.cu:1061-1471,
//  kernels/mla_combine.cu:14-203, kernels/get_mla_metadata.cu:8-82, flash_api.cpp:23-210) and the
// TileLang variant (core/template/tl_template/attn/mla_decode_tl.py:154-303).
//
// The 128 heads of a block are the M dimension of every MMA, so a latent row is used for all heads
// at once.  The fp32 accumulator of 128 heads x 512 columns fills the whole tensor memory of an SM
// (512 columns), leaving no room for the score tile; the work of one (sequence, KV split, head
// block) is therefore shared by a CLUSTER OF TWO CTAs on two SMs:
//
//   score CTA (cluster rank 0)                           value CTA (cluster rank 1)
//   TMEM: Q[:, :512] as 16-bit pairs (256 columns) and    TMEM: O, 128 x 512 fp32 (512 columns)
//         two 128-column score tiles
//   smem: Q[:, 512:] tile, ring of 4 slots of three KV    smem: ring of five 32-row V stages, four
//         chunks (128 rows x 64 columns) each                   64-row P slots
//   warp 8: TMA, chunk by chunk                           warp 4: TMA
//   warp 9: S = Q.KV^T over 128 KV rows: 36 MMAs with      warp 5: O += P.V per 64-row half tile
//           N = 128 (full tensor rate; an MMA costs        warps 0-3: one head per thread: rescale O when
//           ~50 cycles however small N is), A from                 the score CTA moved the reference
//           TMEM for the first 512 columns                         maximum; final scaling and store
//   warps 0-7: one head per thread, the two warp groups    warp 6: re-arms a P slot's barrier and tells
//           take the two 64-column halves of a tile:               the score CTA when the slot is free
//           online softmax in the exp2 domain with lazy
//           rescale; P (16-bit) and the rescale factor go
//           into the VALUE CTA's shared memory with
//           asynchronous stores that are counted on its
//           mbarrier (no release fence, no waiting); P is
//           staged per warp so that every store
//           instruction covers 512 contiguous bytes
//
// FLOP balance 576 : 512, no recomputation.  Each latent row is fetched by both CTAs (the second
// fetch is an L2 hit); no multicast is used.  Split-KV partials are fp32; the combine kernel does
// the log-sum-exp weighted sum.
//
// Work distribution.  A cluster runs a LIST of work units (sequence, range of 128-row KV tiles) one after the other,
// with every ring and barrier phase carried across units, so that the score CTA is already loading and scoring the
// next unit while the value CTA finishes the current one.  The lists come from a scheduler in the manner of the
// reference's get_mla_metadata (kernels/get_mla_metadata.cu:8-82): the KV tiles of all sequences, each charged a
// fixed overhead, are cut into one equal payload per cluster from the ACTUAL cache lengths, on the device, so that
// ragged batches stay balanced and a batch that does not fill whole waves is split where the payload ends; a
// sequence cut by a boundary leaves fp32 partial results that the combine kernel merges.  The older mode with a
// uniform split count per sequence (one unit per cluster) is the same kernel with a one-entry list.
#include <algorithm>
#include <cstring>
#include <mutex>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "parallel_launch.cuh"  // tensor_map_encoder()
#include "sm100.cuh"

namespace b200 {

constexpr int kMlaHeads = 128;     // heads per cluster (MMA M)
constexpr int kMlaTileN = 128;     // KV rows per score tile
constexpr int kMlaThreads = 320;   // 10 warps
constexpr int kMlaSmemBytes = 232448;  // the per-block maximum: the value CTA needs all of it

struct MlaParams {
  const void* q;        // first DV columns of q (read with 16-byte loads)
  long long q_sb, q_sh; // element strides (batch, head)
  void* o;              // [B, H, DV] 16-bit, written when num_splits == 1
  float* lse;           // [B, H] or null
  float* part_o;        // [B, splits, H, DV] fp32 (num_splits > 1)
  float* part_lse;      // [B, splits, H]
  int batch, heads, seq_kv, num_splits, tiles_per_split, head_blocks;
  const int* seq_lens;     // [B] tokens per sequence, or null (= seq_kv)
  const int* block_table;  // [B, bt_stride] pool page of every page_rows-token block, or null (dense cache)
  long long bt_stride;
  int page_rows;
  float scale_log2;     // scale * log2(e)
  float scale;
  int* status;
  // scheduled mode (sched != null): cluster `part` runs the units its 8-int record describes; num_splits_cum[b] is the
  // number of partial-result rows in front of sequence b (a sequence with exactly one is written directly)
  const int* sched;
  const int* num_splits_cum;
  int num_parts;
};

constexpr int kMlaSchedInts = 8;      // ints per scheduler record: begin sequence, begin token, end sequence (inclusive),
                                      // end token (exclusive), split index of the first unit, KV tiles of the part
constexpr int kMlaSchedOverhead = 4;  // tile-times a work unit costs besides its tiles (fill, drain, Q, final exchange)

struct MlaUnit {
  int b, t0, n;   // sequence, first KV tile, number of KV tiles
  int slot;       // row of the partial results, or -1: the unit is its whole sequence and writes the output itself
  int seq_len;
};

// The units of one cluster, in order.
struct MlaWalk {
  const MlaParams& p;
  int b, b_end, begin_tile, end_token, split0;
  bool first, done;
  __device__ MlaWalk(const MlaParams& p_, int part, int legacy_b, int legacy_split) : p(p_), first(true), done(false) {
    if (p.sched != nullptr) {
      const int* m = p.sched + part * kMlaSchedInts;
      b = m[0];
      begin_tile = m[1] / kMlaTileN;
      b_end = m[2];
      end_token = m[3];
      split0 = m[4];
    } else {
      b = b_end = legacy_b;
      begin_tile = legacy_split * p.tiles_per_split;
      split0 = legacy_split;
      end_token = 0;
    }
  }
  __device__ int len_of(int seq) const { return p.seq_lens != nullptr ? max(1, min(p.seq_lens[seq], p.seq_kv)) : p.seq_kv; }
  __device__ bool next(MlaUnit& u) {
    while (!done && b <= b_end && b < p.batch) {
      u.b = b;
      u.seq_len = len_of(b);
      const int total = (u.seq_len + kMlaTileN - 1) / kMlaTileN;
      if (p.sched != nullptr) {
        u.t0 = first ? begin_tile : 0;
        const int t1 = (b == b_end) ? min(total, (end_token + kMlaTileN - 1) / kMlaTileN) : total;
        u.n = t1 - u.t0;
        const int first_row = p.num_splits_cum[b], rows = p.num_splits_cum[b + 1] - first_row;
        u.slot = rows == 1 ? -1 : first_row + (first ? split0 : 0);
      } else {
        u.t0 = begin_tile;
        u.n = max(0, min(total, begin_tile + p.tiles_per_split) - begin_tile);
        u.slot = p.num_splits == 1 ? -1 : b * p.num_splits + split0;
        done = true;
      }
      first = false;
      ++b;
      if (u.n > 0) return true;
    }
    return false;
  }
};

enum MlaWaitSite {
  kMlaSlotFull = 21, kMlaSlotEmpty, kMlaSFull, kMlaSFree, kMlaPFull, kMlaPFree, kMlaPvGo, kMlaPvDone, kMlaODone,
  kMlaFinal, kMlaQReady, kMlaOFinal, kMlaSmemLayout, kMlaQrFull, kMlaRowMax, kMlaRowSum
};

// Shared-memory layout, identical in both CTAs so that a local address maps to the peer's copy.
// Small items first (from the raw base), operand tiles after, aligned to 1024 bytes.
struct MlaSmem {
  // barrier indices
  static constexpr int kSlotFull = 0;    // [12] score: KV chunk ring / value: [5] V stages
  static constexpr int kSlotEmpty = 12;  // [12]
  static constexpr int kSFull = 24;      // [2] score
  static constexpr int kSFree = 26;      // [2] score, 256 arrivals
  static constexpr int kPFull = 28;      // [4] value: 1 arrival (armed locally) + transaction bytes from the score CTA
  static constexpr int kPFree = 32;      // [4] score: 1 arrival from the value CTA
  static constexpr int kPvGo = 36;       // [4] value, 128 arrivals
  static constexpr int kPvDone = 40;     // [4] value
  static constexpr int kStageFree = 44;   // value, 4 arrivals: the output rows staged in the V stages have been read back
  static constexpr int kFinalFull = 45;  // value, 128 arrivals from the score CTA
  static constexpr int kQReady = 46;     // score, 256 arrivals
  static constexpr int kQrFull = 47;     // score
  static constexpr int kRowMax = 48;     // [2] score, 256 arrivals: both halves of a row's maximum are posted
  static constexpr int kRowSum = 50;     // score, 128 arrivals
  static constexpr int kFinalFree = 51;  // score, 4 arrivals from the value CTA: the final statistics of a unit have been read
  static constexpr int kNumBars = 52;
  static constexpr int kOffBars = 0;
  static constexpr int kOffSlot = 416;     // TMEM base address
  static constexpr int kOffAbort = 424;
  static constexpr int kOffPartTiles = 432;   // int: KV tiles of all units of this cluster
  static constexpr int kOffScale = 512;    // value: float [2][128] rescale factor per tile parity and head
  static constexpr int kOffFinal = 1536;   // value: float [128][2] (1/rowsum, lse)
  static constexpr int kOffRowMax = 512;   // score (same bytes, other CTA): float [2 bufs][2 halves][128]
  static constexpr int kOffRowSum = 2560;  // score: float [128]
  static constexpr int kSmallBytes = 3072;
  static constexpr int kChunkBytes = kMlaTileN * 128;           // 16384: 128 rows x 64 columns
  static constexpr int kScoreSlots = 4;                         // each slot holds three chunks: a tile is 3 slots
  static constexpr int kQrBytes = kMlaHeads * 128;              // 16384: Q[:, 512:576]
  static constexpr int kSlotBytes = 3 * kChunkBytes;            // 49152
  static constexpr int kScoreTileBytes = kQrBytes + kScoreSlots * kSlotBytes;    // 212992
  static constexpr int kPStageBytes = 8 * 8 * 128;                 // score: per softmax warp 8 rows x 128 B of P on their way out
  static constexpr int kVStageRows = 32;
  static constexpr int kVStages = 5;
  static constexpr int kVStageBytes = kVStageRows * 512 * 2;    // 32768: 8 chunks of 32 rows x 128 B
  static constexpr int kPSlots = 4;
  static constexpr int kPBytes = kMlaHeads * 64 * 2;            // 16384: 128 heads x 64 KV rows
  static constexpr int kValueTileBytes = kVStages * kVStageBytes + kPSlots * kPBytes;  // 229376
  static_assert(kNumBars * 8 <= kOffSlot, "barriers overlap");
  static_assert(kSmallBytes + kValueTileBytes <= kMlaSmemBytes, "value CTA does not fit");
};

template <int D, int DV, bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMlaThreads, 1)
mla_split_kernel(const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ CUtensorMap tmKVr,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQr, const MlaParams p) {
  using L = MlaSmem;
  constexpr int N = kMlaTileN, M = kMlaHeads;
  static_assert(D == 576 && DV == 512, "tile bookkeeping below is written for 576/512");
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColQ = 0, kColS = 256;   // score CTA: Q[:, :512] in [0,256), S buffers [256,384) [384,512)

  extern __shared__ uint8_t smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + L::kOffBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L::kOffSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L::kOffAbort);
  float* s_scale = reinterpret_cast<float*>(smem_raw + L::kOffScale);
  float* s_final = reinterpret_cast<float*>(smem_raw + L::kOffFinal);
  float* s_rowmax = reinterpret_cast<float*>(smem_raw + L::kOffRowMax);
  float* s_rowsum = reinterpret_cast<float*>(smem_raw + L::kOffRowSum);
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + L::kSmallBytes + 1023) & ~uintptr_t(1023));
  // score CTA: [Q rope tile][12 KV chunks];  value CTA: [5 V stages][4 P slots]
  uint8_t* sQr = tiles;
  uint8_t* sChunk = tiles + L::kQrBytes;
  uint8_t* sPStage = tiles + L::kScoreTileBytes;
  uint8_t* sV = tiles;
  uint8_t* sP = tiles + L::kVStages * L::kVStageBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = score CTA, 1 = value CTA
  const AbortState ab{abort_flag, p.status};
  // scheduled mode: blockIdx.y = head block * parts + part; uniform splits: blockIdx.y = head block * splits + split
  const int per_hb = p.sched != nullptr ? p.num_parts : p.num_splits;
  const int part = blockIdx.y % per_hb;
  const int hb = blockIdx.y / per_hb;
  const int head0 = hb * M;
  volatile int* part_tiles_s = reinterpret_cast<volatile int*>(smem_raw + L::kOffPartTiles);
  auto make_walk = [&]() { return MlaWalk(p, part, static_cast<int>(blockIdx.z), part); };
  // pool coordinates of logical token row `r` of a sequence with a paged cache (rows past the end are redirected to
  // the last token's 64-row block: they are masked, but must be read from mapped memory)
  auto locate = [&](const MlaUnit& u, int r, int& row_in_page, int& page) {
    r = min(r, ((u.seq_len - 1) >> 6) << 6 | (r & 63));
    const int blk = r / p.page_rows;
    page = p.block_table[static_cast<long long>(u.b) * p.bt_stride + blk];
    row_in_page = r - blk * p.page_rows;
  };
  const bool paged = p.block_table != nullptr;
  constexpr uint32_t kPTxEven = L::kPBytes + M * 4;   // half 0 of a tile also carries the rescale factors
  constexpr uint32_t kPTxOdd = L::kPBytes;

  if (threadIdx.x == 0) {
    int bad = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    // the operand tiles must end inside the dynamic shared memory that was requested
    const size_t used = static_cast<size_t>(tiles - smem_raw) + (rank == 0 ? L::kScoreTileBytes + L::kPStageBytes : L::kValueTileBytes);
    if (used > static_cast<size_t>(kMlaSmemBytes)) {
      atomicCAS(p.status, 0, kStatusTimeoutBase + kMlaSmemLayout);
      bad = 1;
    }
    *abort_flag = bad;
    {
      MlaWalk count = make_walk();
      MlaUnit u;
      int tiles = 0;
      while (count.next(u)) tiles += u.n;
      *part_tiles_s = tiles;
    }
    for (int i = 0; i < 12; ++i) {
      mbar_init(&bars[L::kSlotFull + i], 1);
      mbar_init(&bars[L::kSlotEmpty + i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[L::kSFull + i], 1);
      mbar_init(&bars[L::kSFree + i], 256);
      mbar_init(&bars[L::kRowMax + i], 256);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars[L::kPFull + i], 1);
      mbar_init(&bars[L::kPFree + i], 1);
      mbar_init(&bars[L::kPvGo + i], 128);
      mbar_init(&bars[L::kPvDone + i], 1);
    }
    mbar_init(&bars[L::kStageFree], 4);
    mbar_init(&bars[L::kFinalFree], 4);
    mbar_init(&bars[L::kFinalFull], 128);
    mbar_init(&bars[L::kQReady], 256);
    mbar_init(&bars[L::kQrFull], 1);
    mbar_init(&bars[L::kRowSum], 128);
    fence_barrier_init();
    if (rank == 1) {
      // every P slot expects its first half tile before the score CTA can send anything
      for (int i = 0; i < 4; ++i) mbar_arrive_expect_tx(&bars[L::kPFull + i], (i & 1) ? kPTxOdd : kPTxEven);
    }
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tmKV);
    tma_prefetch_desc(&tmKVr);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmQr);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs have initialised (and armed) their barriers before any remote traffic
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int part_tiles = *part_tiles_s;
  const bool run = (part_tiles > 0) && !*abort_flag && (*reinterpret_cast<volatile int*>(p.status) == 0);

  if (rank == 0) {
    // ===================================== score CTA =====================================
    if (warp == 8) {
      if (lane == 0 && run) {
        MlaWalk walk = make_walk();
        MlaUnit u;
        int J = 0;     // KV tiles of the units before this one: ring positions and barrier phases run on across units
        bool ok = true;
        for (int ui = 0; ok && walk.next(u); ++ui, J += u.n) {
          if (ui > 0) {
            // the rope tile of the previous unit is read by the MMAs of its last slot load
            const int gl = 3 * J - 1;
            ok = mbar_wait(&bars[L::kSlotEmpty + gl % L::kScoreSlots], (gl / L::kScoreSlots) & 1, ab, kMlaSlotEmpty);
            if (!ok) break;
          }
          mbar_arrive_expect_tx(&bars[L::kQrFull], L::kQrBytes);
          tma_load_3d(sQr, &tmQr, &bars[L::kQrFull], 0, head0, u.b);
          for (int g = 0; g < u.n * 3; ++g) {   // slot loads: three 64-column chunks of one 128-row tile each
            const int gg = 3 * J + g;
            const int j = g / 3, c0 = (g - j * 3) * 3, slot = gg % L::kScoreSlots;
            ok = mbar_wait(&bars[L::kSlotEmpty + slot], ((gg / L::kScoreSlots) & 1) ^ 1, ab, kMlaSlotEmpty);
            if (!ok) break;
            mbar_arrive_expect_tx(&bars[L::kSlotFull + slot], L::kSlotBytes);
            if (!paged) {
              for (int c = c0; c < c0 + 3; ++c)
                tma_load_3d(sChunk + slot * L::kSlotBytes + (c - c0) * L::kChunkBytes, c < 8 ? &tmKV : &tmKVr, &bars[L::kSlotFull + slot],
                            c < 8 ? c * 64 : 0, (u.t0 + j) * N, u.b);
            } else {
              // paged cache: the maps have 64-row boxes over [pool page][row in page]; a tile is two boxes
              for (int hf = 0; hf < 2; ++hf) {
                int rin, pg;
                locate(u, (u.t0 + j) * N + hf * 64, rin, pg);
                for (int c = c0; c < c0 + 3; ++c)
                  tma_load_3d(sChunk + slot * L::kSlotBytes + (c - c0) * L::kChunkBytes + hf * (64 * 128), c < 8 ? &tmKV : &tmKVr,
                              &bars[L::kSlotFull + slot], c < 8 ? c * 64 : 0, rin, pg);
              }
            }
          }
        }
      }
    } else if (warp == 9) {
      // The whole warp runs this loop converged and one elected lane issues each batch of twelve MMAs with its
      // commits: descriptors and loop state then live in uniform registers and a batch leaves at the tensor pipe's
      // rate (issued from inside an `if (lane == 0)` region an MMA with N = 128 took ~90 cycles beside the busy
      // softmax warps, against the 64 the pipe needs for it: 36 of them per tile).
      if (__all_sync(0xffffffffu, run)) {
        constexpr uint32_t idesc = make_idesc_f16(M, N, kBf16, false, false);
        const uint64_t chunk_desc0 = make_smem_desc(smem_u32(sChunk), 16, 1024);
        const uint64_t qr_desc0 = make_smem_desc(smem_u32(sQr), 16, 1024);
        auto wait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
          return __all_sync(0xffffffffu, mbar_wait(bar, parity, ab, site));
        };
        MlaWalk walk = make_walk();
        MlaUnit unit;
        int J = 0;
        bool ok = true;
        for (int ui = 0; ok && walk.next(unit); ++ui, J += unit.n) {
        ok = wait(&bars[L::kQReady], ui & 1, kMlaQReady) && wait(&bars[L::kQrFull], ui & 1, kMlaQrFull);
        for (int jl = 0; jl < unit.n && ok; ++jl) {
          const int j = J + jl;
          const int buf = j & 1;
          ok = wait(&bars[L::kSFree + buf], ((j >> 1) & 1) ^ 1, kMlaSFree);
          for (int u = 0; u < 3 && ok; ++u) {
            const int g = j * 3 + u, slot = g % L::kScoreSlots;
            ok = wait(&bars[L::kSlotFull + slot], (g / L::kScoreSlots) & 1, kMlaSlotFull);
            if (!ok) break;
            tc_fence_after_sync();
            // three 64-column chunks, four K steps each: operands advance by 32 bytes (A: 8 TMEM columns);
            // one barrier check and one commit per twelve MMAs
            const uint64_t bdesc = chunk_desc0 + static_cast<uint64_t>(slot * (L::kSlotBytes >> 4));
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < 3; ++k) {
                const int c = u * 3 + k;
                const uint64_t bd = bdesc + static_cast<uint64_t>(k * (L::kChunkBytes >> 4));
                if (c < 8)
                  umma_ts_x4<8, 2>(tmem_base + kColS + buf * N, tmem_base + kColQ + c * 32, bd, idesc, c > 0 ? 1u : 0u);
                else
                  umma_ss_x4<2, 2>(tmem_base + kColS + buf * N, qr_desc0, bd, idesc, 1u);
              }
              umma_commit(&bars[L::kSlotEmpty + slot]);
              if (u == 2) umma_commit(&bars[L::kSFull + buf]);
            }
          }
        }
        }
      }
    } else {
      // 256 threads: thread (wg, row) owns columns [64*wg, 64*wg+64) of its head's score row
      const int wg = warp >> 2;
      const int row = (warp & 3) * 32 + lane;
      const int head = head0 + row;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t stage_w = smem_u32(sPStage) + warp * 1024;
      const uint32_t peer_p = map_to_cta(smem_u32(sP), 1) + (warp & 3) * (32 * 128) + lane * 16;
      const uint32_t peer_scale = map_to_cta(smem_u32(s_scale), 1) + row * 4;
      const uint32_t peer_pfull = map_to_cta(smem_u32(&bars[L::kPFull]), 1);
      MlaWalk walk = make_walk();
      MlaUnit unit;
      int J = 0;
      bool ok = run;
      for (int ui = 0; ok && walk.next(unit); ++ui, J += unit.n) {
        const int b = unit.b, n = unit.n, seq_len = unit.seq_len, tile_begin = unit.t0;
        // ---- this head's query row, columns [256*wg, 256*wg+256) -> TMEM as 16-bit pairs (every score MMA of the
        //      previous unit has completed: this thread has seen its last score tile) ----
        const bool valid = head < p.heads;
        const uint4* qm = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.q) + b * p.q_sb +
                                                         static_cast<long long>(head) * p.q_sh + wg * 256);
        // a thread reads its own row (rows are a kilobyte apart): the loads of half a row are issued together,
        // so that the copy costs two memory round trips instead of one per 128 bytes
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t w[64];
#pragma unroll
          for (int v = 0; v < 16; ++v) {
            const uint4 x = valid ? qm[hf * 16 + v] : make_uint4(0u, 0u, 0u, 0u);
            w[4 * v + 0] = x.x;
            w[4 * v + 1] = x.y;
            w[4 * v + 2] = x.z;
            w[4 * v + 3] = x.w;
          }
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t wc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) wc[i] = w[c * 32 + i];
            tmem_st32(tmem_base + lane_base + kColQ + wg * 128 + (hf * 2 + c) * 32, wc);
          }
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&bars[L::kQReady]);

        // ---- online softmax, one 128-row tile at a time; this thread produces half tile `wg` ----
        float m_ref = -1.0e30f, r_sum = 0.0f;
        const float c2 = p.scale_log2;
        // P leaves through an 1 KB staging area per warp: the rows of eight lanes at a time are written there in the
        // (128-byte swizzled) image of the value CTA's tile and sent on as whole 512-byte runs per warp instruction.
        // Sixteen-byte pieces sent row by row (32 rows per instruction) held the tensor pipe of this SM back for
        // about half of every tile.
        for (int jl = 0; jl < n && ok; ++jl) {
          const int j = J + jl;   // position in the cluster's whole run: rings, buffers and phases
          const int buf = j & 1;
          const int pslot = (2 * j + wg) & 3;
          ok = mbar_wait(&bars[L::kSFull + buf], (j >> 1) & 1, ab, kMlaSFull);
          if (!ok) break;
          tc_fence_after_sync();
          float s[64];
          tmem_ld32f(tmem_base + lane_base + kColS + buf * N + wg * 64, &s[0]);
          tmem_ld32f(tmem_base + lane_base + kColS + buf * N + wg * 64 + 32, &s[32]);
          tmem_wait_ld();
          tc_fence_before_sync();
          mbar_arrive(&bars[L::kSFree + buf]);  // this half is in registers
          const int kv0 = (tile_begin + jl) * N + wg * 64;
          if (kv0 + 64 > seq_len) {
#pragma unroll
            for (int i = 0; i < 64; ++i) s[i] = (kv0 + i < seq_len) ? s[i] : -INFINITY;
          }
          float mx0 = s[0], mx1 = s[1];
#pragma unroll
          for (int i = 2; i < 64; i += 2) {
            mx0 = fmaxf(mx0, s[i]);
            mx1 = fmaxf(mx1, s[i + 1]);
          }
          // the row maximum needs the other half too: post mine, wait for both
          s_rowmax[(buf * 2 + wg) * M + row] = fmaxf(mx0, mx1);
          mbar_arrive(&bars[L::kRowMax + buf]);
          ok = mbar_wait(&bars[L::kRowMax + buf], (j >> 1) & 1, ab, kMlaRowMax);
          if (!ok) break;
          const float mx = fmaxf(s_rowmax[(buf * 2) * M + row], s_rowmax[(buf * 2 + 1) * M + row]);
          float o_scale = 1.0f;
          if ((mx - m_ref) * c2 > 8.0f) {   // both halves take the same decision from the same numbers
            o_scale = fast_exp2((m_ref - mx) * c2);
            m_ref = mx;
            r_sum *= o_scale;
          }
          const float neg = -m_ref * c2;
          float a0 = 0.f, a1 = 0.f;
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float e0 = fast_exp2(fmaf(s[i], c2, neg));
            const float e1 = fast_exp2(fmaf(s[i + 1], c2, neg));
            a0 += e0;
            a1 += e1;
            pk[i / 2] = pack2<kBf16>(e0, e1);
          }
          r_sum += a0 + a1;
          // P half tile (128-byte row, swizzled like a TMA-written K-major tile) and, with half 0, the rescale
          // factor go to the value CTA; every byte is counted on its p_full barrier
          ok = mbar_wait_cluster(&bars[L::kPFree + pslot], ((j >> 1) & 1) ^ 1, ab, kMlaPFree);
          if (!ok) break;
          const uint32_t dst = peer_p + pslot * L::kPBytes;
          const uint32_t bar = peer_pfull + pslot * 8;
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            if ((lane >> 3) == pass) {
              const uint32_t mine = stage_w + (lane & 7) * 128;
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4)
                st_shared_v4(mine + ((q4 ^ (lane & 7)) << 4), make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]));
            }
            __syncwarp();
            const uint4 run0 = ld_shared_v4(stage_w + lane * 16);
            const uint4 run1 = ld_shared_v4(stage_w + 512 + lane * 16);
            st_async_v4(dst + pass * 1024, run0, bar);
            st_async_v4(dst + pass * 1024 + 512, run1, bar);
            __syncwarp();
          }
          if (wg == 0) st_async_f32(peer_scale + (j & 1) * (M * 4), o_scale, bar);
        }
        // ---- final row statistics: sum of both halves ----
        if (ok) {
          if (wg == 1) {
            s_rowsum[row] = r_sum;
            mbar_arrive(&bars[L::kRowSum]);
          } else {
            ok = mbar_wait(&bars[L::kRowSum], ui & 1, ab, kMlaRowSum);
            // the value CTA must have read the previous unit's statistics before they are replaced
            if (ok && ui > 0) ok = mbar_wait_cluster(&bars[L::kFinalFree], (ui - 1) & 1, ab, kMlaFinal);
            if (ok) {
              const float total = r_sum + s_rowsum[row];
              const uint32_t peer_final = map_to_cta(smem_u32(s_final), 1) + row * 8;
              st_cluster_f32(peer_final, 1.0f / total);
              st_cluster_f32(peer_final + 4, logf(total) + m_ref * p.scale);
              mbar_arrive_cluster(map_to_cta(smem_u32(&bars[L::kFinalFull]), 1));
            }
          }
        }
      }
    }
  } else {
    // ===================================== value CTA =====================================
    const int part_half = 2 * part_tiles;   // 64-row half tiles of all units
    if (warp == 4) {
      if (lane == 0 && run) {
        MlaWalk walk = make_walk();
        MlaUnit u;
        int J = 0;
        bool ok = true;
        for (int ui = 0; ok && walk.next(u); ++ui, J += u.n) {
          // the output rows of the previous unit are staged in the V stages: wait until they have been read back
          if (ui > 0) ok = mbar_wait(&bars[L::kStageFree], (ui - 1) & 1, ab, kMlaOFinal);
          for (int g = 0; g < u.n * 4 && ok; ++g) {   // 32-row stages
            const int gg = 4 * J + g;
            const int st = gg % L::kVStages;
            ok = mbar_wait(&bars[L::kSlotEmpty + st], ((gg / L::kVStages) & 1) ^ 1, ab, kMlaSlotEmpty);
            if (!ok) break;
            mbar_arrive_expect_tx(&bars[L::kSlotFull + st], L::kVStageBytes);
            uint8_t* dst = sV + st * L::kVStageBytes;
            int vrow = u.t0 * N + g * L::kVStageRows, vz = u.b;
            if (paged) locate(u, vrow, vrow, vz);
            for (int c = 0; c < 8; ++c)
              tma_load_3d(dst + c * (L::kVStageRows * 128), &tmV, &bars[L::kSlotFull + st], c * 64, vrow, vz);
          }
        }
      }
    } else if (warp == 5) {
      if (lane == 0 && run) {
        constexpr uint32_t idesc = make_idesc_f16(M, 256, kBf16, false, true);
        const uint64_t v_desc0 = make_smem_desc(smem_u32(sV), L::kVStageRows * 128, 1024);
        const uint64_t p_desc0 = make_smem_desc(smem_u32(sP), 16, 1024);
        MlaWalk walk = make_walk();
        MlaUnit u;
        int J = 0;
        bool ok = true;
        for (int ui = 0; ok && walk.next(u); ++ui, J += u.n) {
        for (int hl = 0; hl < 2 * u.n && ok; ++hl) {
          const int h = 2 * J + hl;    // position in the cluster's whole run
          const int pslot = h & 3;
          ok = mbar_wait(&bars[L::kPvGo + pslot], (h >> 2) & 1, ab, kMlaPvGo);
          for (int s2 = 0; s2 < 2 && ok; ++s2) {
            const int g = h * 2 + s2, st = g % L::kVStages;
            ok = mbar_wait(&bars[L::kSlotFull + st], (g / L::kVStages) & 1, ab, kMlaSlotFull);
            if (!ok) break;
            tc_fence_after_sync();
            // two K steps of 16 KV rows; each feeds the two 256-column halves of O.  V columns [256*hh, +256):
            // four 64-column chunks of 32 rows (4096 B apart); a K step is 2048 B further
            const uint64_t adesc = p_desc0 + static_cast<uint64_t>(pslot * (L::kPBytes >> 4) + s2 * 4);
            const uint64_t bdesc = v_desc0 + static_cast<uint64_t>(st * (L::kVStageBytes >> 4));
            constexpr uint64_t kHalf = (4 * L::kVStageRows * 128) >> 4;
            umma_ss_2d(tmem_base, tmem_base + 256, adesc, bdesc, bdesc + kHalf, idesc, (hl > 0 || s2 > 0) ? 1u : 0u);
            umma_ss_2d(tmem_base, tmem_base + 256, adesc + 2, bdesc + 128, bdesc + kHalf + 128, idesc, 1u);
            umma_commit(&bars[L::kSlotEmpty + st]);
          }
          if (ok) umma_commit(&bars[L::kPvDone + pslot]);
        }
        }
      }
    } else if (warp == 6) {
      if (lane == 0 && run) {
        const uint32_t peer_pfree = map_to_cta(smem_u32(&bars[L::kPFree]), 0);
        for (int h = 0; h < part_half; ++h) {
          const int pslot = h & 3;
          if (!mbar_wait(&bars[L::kPvDone + pslot], (h >> 2) & 1, ab, kMlaPvDone)) break;
          // arm the slot for its next half tile BEFORE the score CTA learns that it is free
          if (h + 4 < part_half) mbar_arrive_expect_tx(&bars[L::kPFull + pslot], (pslot & 1) ? kPTxOdd : kPTxEven);
          mbar_arrive_cluster(peer_pfree + pslot * 8);
        }
      }
    } else if (warp < 4) {
      const int row = warp * 32 + lane;
      const int head = head0 + row;
      const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
      const uint32_t tO = tmem_base + lane_base;
      const uint32_t peer_final_free = map_to_cta(smem_u32(&bars[L::kFinalFree]), 0);
      MlaWalk walk = make_walk();
      MlaUnit unit;
      int J = 0;
      bool ok = run;
      bool any_unit = false;
      for (int ui = 0; ok && walk.next(unit); ++ui, J += unit.n) {
      any_unit = true;
      const int b = unit.b, n = unit.n, n_half = 2 * unit.n;
      for (int hl = 0; hl < n_half && ok; ++hl) {
        const int h = 2 * J + hl;   // position in the cluster's whole run
        const int pslot = h & 3;
        ok = mbar_wait_cluster(&bars[L::kPFull + pslot], (h >> 2) & 1, ab, kMlaPFull);
        if (!ok) break;
        const float o_scale = (h & 1) ? 1.0f : s_scale[((h >> 1) & 1) * M + row];
        if (hl > 0 && __any_sync(0xffffffffu, o_scale != 1.0f)) {
          // O must hold everything up to half tile h-1.  A parity wait is only unambiguous if the barrier
          // cannot be two phases away: these threads run far ahead of the MMAs, so they wait on the ring of
          // per-slot barriers (slot (h-1)&3 was last completed for half tile h-5, which p_full(h) implies).
          ok = mbar_wait(&bars[L::kPvDone + ((h - 1) & 3)], ((h - 1) >> 2) & 1, ab, kMlaODone);
          if (ok) {
            tc_fence_after_sync();
#pragma unroll 4
            for (int c = 0; c < DV / 32; ++c) {
              float o[32];
              tmem_ld32f(tO + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= o_scale;
              tmem_st32f(tO + c * 32, o);
            }
            tmem_wait_st();
          }
        }
        fence_proxy_async_smem();   // P arrived through generic-proxy stores; the MMA reads it through the async proxy
        tc_fence_before_sync();
        mbar_arrive(&bars[L::kPvGo + pslot]);
      }
      if (ok) {
        const int h_last = 2 * J + n_half - 1;
        ok = mbar_wait_cluster(&bars[L::kFinalFull], ui & 1, ab, kMlaFinal) &&
             mbar_wait(&bars[L::kPvDone + (h_last & 3)], (h_last >> 2) & 1, ab, kMlaOFinal);
        if (ok) {
          tc_fence_after_sync();
          const bool in_range = head < p.heads;
          const float inv = s_final[row * 2];
          const float lse = s_final[row * 2 + 1];
          // the statistics are in registers: the score CTA may send the next unit's
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(peer_final_free);
          // Rows leave through the V stages (all consumed by now), 1024 bytes of a row at a time: the whole 16-bit
          // output row of a unit that is its whole sequence, or half of the fp32 row of a partial result (two
          // passes).  Each warp stages the 32 rows it holds (16-byte pieces, piece index xor row: conflict-free) and
          // then stores them as 512 contiguous bytes per instruction; a thread storing its own row scatters every
          // warp instruction over 32 rows (and 16 bytes into each 32-byte sector).
          static_assert(4 * 32 * 1024 <= L::kVStages * L::kVStageBytes && DV == 512, "row staging is laid out for 1 KB pieces of 512-wide rows");
          const bool partial = unit.slot >= 0;
          const uint32_t stage = smem_u32(sV) + warp * (32 * 1024);
          const uint32_t mine = stage + lane * 1024;
          uint8_t* gbase = partial
              ? reinterpret_cast<uint8_t*>(p.part_o + (static_cast<long long>(unit.slot) * p.heads + head0 + warp * 32) * DV)
              : reinterpret_cast<uint8_t*>(p.o) + 2 * ((static_cast<long long>(b) * p.heads + head0 + warp * 32) * DV);
          const long long grow = partial ? DV * 4 : DV * 2;   // bytes between rows
          for (int pass = 0; pass < (partial ? 2 : 1); ++pass) {
            if (pass > 0) __syncwarp();   // the first half has been read back
            if (!partial) {
#pragma unroll 2
              for (int c = 0; c < DV / 32; ++c) {
                float o[32];
                tmem_ld32f(tO + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  uint4 pk;
                  pk.x = pack2<kBf16>(o[8 * v + 0] * inv, o[8 * v + 1] * inv);
                  pk.y = pack2<kBf16>(o[8 * v + 2] * inv, o[8 * v + 3] * inv);
                  pk.z = pack2<kBf16>(o[8 * v + 4] * inv, o[8 * v + 5] * inv);
                  pk.w = pack2<kBf16>(o[8 * v + 6] * inv, o[8 * v + 7] * inv);
                  st_shared_v4(mine + (((c * 4 + v) ^ (lane & 7)) << 4), pk);
                }
              }
            } else {
#pragma unroll 2
              for (int c = 0; c < 8; ++c) {
                float o[32];
                tmem_ld32f(tO + (pass * 8 + c) * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  uint4 pk;
                  pk.x = __float_as_uint(o[4 * v + 0] * inv);
                  pk.y = __float_as_uint(o[4 * v + 1] * inv);
                  pk.z = __float_as_uint(o[4 * v + 2] * inv);
                  pk.w = __float_as_uint(o[4 * v + 3] * inv);
                  st_shared_v4(mine + (((c * 8 + v) ^ (lane & 7)) << 4), pk);
                }
              }
            }
            __syncwarp();
            uint8_t* obase = gbase + pass * 1024 + lane * 16;
#pragma unroll 1
            for (int r0 = 0; r0 < 32; r0 += 8) {
              uint4 val[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int r = r0 + i / 2, piece = (i % 2) * 32 + lane;
                val[i] = ld_shared_v4(stage + r * 1024 + ((piece ^ (r & 7)) << 4));
              }
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int r = r0 + i / 2;
                if (head0 + warp * 32 + r < p.heads)
                  *reinterpret_cast<uint4*>(obase + static_cast<long long>(r) * grow + (i % 2) * 512) = val[i];
              }
            }
          }
          if (in_range) {
            if (partial) p.part_lse[static_cast<long long>(unit.slot) * p.heads + head] = lse;
            else if (p.lse != nullptr) p.lse[static_cast<long long>(b) * p.heads + head] = lse;
          }
          // the staged rows have been read back (or none were staged): the V stages may be refilled
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[L::kStageFree]);
        }
      }
      }
      if (!any_unit && p.sched == nullptr && p.num_splits > 1 && head < p.heads && !*abort_flag) {
        // uniform splits: a split with no KV rows contributes nothing
        p.part_lse[(static_cast<long long>(blockIdx.z) * p.num_splits + part) * p.heads + head] = -INFINITY;
      }
    }
  }

  // teardown: neither CTA may leave while its peer can still touch its shared memory or barriers
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// o[b,h,:] = sum_i exp(lse_i - lse) * part_o[b,i,h,:],  lse = log sum_i exp(lse_i).
// One warp per (b, h); each lane owns DV/32 columns spread in float4 groups.
// The partial rows of sequence b are rows [cum[b], cum[b+1]) of part_o / part_lse (scheduled mode; a sequence with one
// row was written directly by the decode kernel and is skipped), or rows [b*num_splits, (b+1)*num_splits) (cum == null).
template <int DV, bool kBf16>
__global__ void __launch_bounds__(256) mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                                        void* __restrict__ o, float* __restrict__ lse_out, int batch,
                                                        int heads, int uniform_splits, const int* __restrict__ cum) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= batch * heads) return;
  const int b = warp / heads, h = warp % heads;
  const int row0 = cum != nullptr ? cum[b] : b * uniform_splits;
  const int num_splits = cum != nullptr ? cum[b + 1] - row0 : uniform_splits;
  if (cum != nullptr && num_splits <= 1) return;
  part_o += static_cast<long long>(row0) * heads * DV;
  part_lse += static_cast<long long>(row0) * heads;
  float mx = -INFINITY;
  for (int i = 0; i < num_splits; ++i) mx = fmaxf(mx, part_lse[static_cast<long long>(i) * heads + h]);
  float den = 0.f;
  for (int i = 0; i < num_splits; ++i) den += __expf(part_lse[static_cast<long long>(i) * heads + h] - mx);
  const float lse = mx + __logf(den);
  constexpr int V4 = DV / 128;  // float4 groups per lane
  float4 acc[V4];
#pragma unroll
  for (int v = 0; v < V4; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < num_splits; ++i) {
    const long long row = static_cast<long long>(i) * heads + h;
    const float li = part_lse[row];
    if (li == -INFINITY) continue;
    const float w = __expf(li - lse);
    const float4* src = reinterpret_cast<const float4*>(part_o + row * DV);
#pragma unroll
    for (int v = 0; v < V4; ++v) {
      const float4 x = src[v * 32 + lane];
      acc[v].x += w * x.x;
      acc[v].y += w * x.y;
      acc[v].z += w * x.z;
      acc[v].w += w * x.w;
    }
  }
  uint8_t* orow = reinterpret_cast<uint8_t*>(o) + 2 * (static_cast<long long>(b) * heads + h) * DV;
#pragma unroll
  for (int v = 0; v < V4; ++v) {
    uint2 pk;
    pk.x = pack2<kBf16>(acc[v].x, acc[v].y);
    pk.y = pack2<kBf16>(acc[v].z, acc[v].w);
    *reinterpret_cast<uint2*>(orow + (v * 32 + lane) * 8) = pk;
  }
  if (lane == 0 && lse_out != nullptr) lse_out[static_cast<long long>(b) * heads + h] = lse;
}

// Scheduler: cuts the KV tiles of all sequences (each sequence, and each part of a sequence, charged
// kMlaSchedOverhead tiles on top of its own) into `parts` equal payloads, one per cluster.  The greedy of the reference
// (kernels/get_mla_metadata.cu:8-82) in this kernel's units: a part takes whole sequences while they fit its
// remaining payload and then as many tiles of the next one as are left beyond the overhead.  Record of a part: first
// sequence, first token, last sequence (inclusive), end token (exclusive), split index of its first unit, KV tiles.
// cum[b] = partial-result rows in front of sequence b.  One warp; the walk itself is serial.
__global__ void __launch_bounds__(32) mla_schedule_kernel(const int* __restrict__ seq_lens, int batch, int seq_kv, int parts,
                                                        int* __restrict__ sched, int* __restrict__ cum) {
  auto tiles_of = [&](int b) {
    const int len = seq_lens != nullptr ? max(1, min(seq_lens[b], seq_kv)) : seq_kv;
    return (len + kMlaTileN - 1) / kMlaTileN;
  };
  auto len_of = [&](int b) { return seq_lens != nullptr ? max(1, min(seq_lens[b], seq_kv)) : seq_kv; };
  int total = 0;
  for (int b = threadIdx.x; b < batch; b += 32) total += tiles_of(b) + kMlaSchedOverhead;
  for (int off = 16; off >= 1; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
  if (threadIdx.x != 0) return;
  const int payload = max((total + parts - 1) / parts + kMlaSchedOverhead, 2 * kMlaSchedOverhead);
  int seq = 0, tile = 0, split = 0, rows = 0;
  cum[0] = 0;
  for (int part = 0; part < parts; ++part) {
    int* rec = sched + part * kMlaSchedInts;
    rec[0] = seq;
    rec[1] = tile * kMlaTileN;
    rec[4] = split;
    int budget = payload, taken = 0;
    while (seq < batch) {
      const int rest = tiles_of(seq) - tile;
      if (budget >= rest + kMlaSchedOverhead) {   // the rest of this sequence fits
        rows += split + 1;
        cum[seq + 1] = rows;
        budget -= rest + kMlaSchedOverhead;
        taken += rest;
        ++seq;
        tile = 0;
        split = 0;
      } else {
        if (budget > kMlaSchedOverhead) {          // a piece of it does
          tile += budget - kMlaSchedOverhead;
          taken += budget - kMlaSchedOverhead;
          ++split;
        }
        break;
      }
    }
    rec[2] = tile > 0 ? seq : seq - 1;
    rec[3] = tile > 0 ? tile * kMlaTileN : (seq > 0 ? len_of(seq - 1) : 0);
    rec[5] = taken;
    rec[6] = rec[7] = 0;
  }
}

// Clusters that share the KV of all sequences: SM pairs, divided among the head blocks (each head block walks the
// same schedule on its own clusters).
inline int mla_num_parts(int heads_q, int sm_count) {
  const int head_blocks = (heads_q + kMlaHeads - 1) / kMlaHeads;
  return std::max(1, sm_count / 2 / head_blocks);
}

inline int current_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

// Scheduled mode: layout of the workspace -- scheduler records, cumulative split counts, then the partial rows.
struct MlaSchedLayout {
  int parts;
  long long max_rows, off_cum, off_part_o, off_part_lse, bytes;
  MlaSchedLayout(const AttnB200MlaShape& s, int parts_) : parts(parts_) {
    max_rows = static_cast<long long>(s.batch) + parts;   // every part boundary cuts at most one sequence
    off_cum = static_cast<long long>(parts) * kMlaSchedInts * 4;
    off_part_o = (off_cum + (static_cast<long long>(s.batch) + 1) * 4 + 255) / 256 * 256;
    off_part_lse = off_part_o + max_rows * s.heads_q * s.dim_v * 4;
    bytes = off_part_lse + max_rows * s.heads_q * 4;
  }
};

// 3-D map over a 16-bit [batch][rows][cols] tensor view with element strides (batch, row), cols contiguous.
inline int encode_3d(CUtensorMap* tm, const void* base, int dtype, uint64_t cols, uint64_t rows, uint64_t batch,
                     int64_t stride_batch, int64_t stride_row, uint32_t box_rows) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return ATTN_B200_E_LAUNCH;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  if (stride_row <= 0 || stride_row % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  if (batch <= 1) stride_batch = stride_row * static_cast<int64_t>(rows);
  if (stride_batch <= 0 || stride_batch % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  cuuint64_t gdim[3] = {cols, rows, batch};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(stride_row) * 2, static_cast<cuuint64_t>(stride_batch) * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == ATTN_B200_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(tm, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ATTN_B200_OK : ATTN_B200_E_UNSUPPORTED;
}

inline int validate_mla_shape(const AttnB200MlaShape* s) {
  if (s == nullptr) return ATTN_B200_E_INVALID_ARG;
  if (s->batch <= 0 || s->heads_q <= 0 || s->seq_kv <= 0) return ATTN_B200_E_INVALID_ARG;
  if (s->dim_qk != 576 || s->dim_v != 512) return ATTN_B200_E_UNSUPPORTED;
  if (s->batch > 65535) return ATTN_B200_E_UNSUPPORTED;
  return ATTN_B200_OK;
}

template <bool kBf16>
int launch_mla(const AttnB200MlaArgs* a, cudaStream_t stream, int* status) {
  constexpr int D = 576, DV = 512;
  const AttnB200MlaShape& s = a->shape;
  CUtensorMap tmKV, tmKVr, tmV, tmQr;
  const int esz = 2;
  // rope columns: a separate tensor, or columns [DV, D) of the fused rows
  const void* q_rope = a->q_rope != nullptr ? a->q_rope : static_cast<const uint8_t*>(a->q) + DV * esz;
  const void* kv_rope = a->kv_rope != nullptr ? a->kv_rope : static_cast<const uint8_t*>(a->kv) + DV * esz;
  const int64_t* qr_st = a->q_rope != nullptr ? a->q_rope_stride : a->q_stride;
  const int64_t* kr_st = a->kv_rope != nullptr ? a->kv_rope_stride : a->kv_stride;
  // the first DV columns of a q row are read with 16-byte loads straight into tensor memory
  if ((reinterpret_cast<uintptr_t>(a->q) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  for (int i = 0; i < 2; ++i)
    if (a->q_stride[i] % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  // dense cache: maps over [batch][token]; paged cache: maps over [pool page][row in page], score-side boxes of 64 rows
  const bool paged = a->block_table != nullptr;
  if (paged) {
    if (a->page_size <= 0 || a->page_size % 64 != 0 || a->num_pages <= 0) return ATTN_B200_E_INVALID_ARG;
    if (a->block_table_stride < (s.seq_kv + a->page_size - 1) / a->page_size) return ATTN_B200_E_INVALID_ARG;
  }
  const uint64_t map_rows = paged ? a->page_size : s.seq_kv, map_outer = paged ? a->num_pages : s.batch;
  const uint32_t score_box = paged ? 64 : kMlaTileN;
  int rc = encode_3d(&tmKV, a->kv, a->dtype, DV, map_rows, map_outer, a->kv_stride[0], a->kv_stride[1], score_box);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmKVr, kv_rope, a->dtype, D - DV, map_rows, map_outer, kr_st[0], kr_st[1], score_box);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmV, a->kv, a->dtype, DV, map_rows, map_outer, a->kv_stride[0], a->kv_stride[1], MlaSmem::kVStageRows);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmQr, q_rope, a->dtype, D - DV, s.heads_q, s.batch, qr_st[0], qr_st[1], kMlaHeads);
  if (rc != ATTN_B200_OK) return rc;
  MlaParams p;
  std::memset(&p, 0, sizeof(p));
  const int total_tiles = (s.seq_kv + kMlaTileN - 1) / kMlaTileN;
  p.q = a->q;
  p.q_sb = a->q_stride[0];
  p.q_sh = a->q_stride[1];
  p.head_blocks = (s.heads_q + kMlaHeads - 1) / kMlaHeads;
  p.o = a->o;
  p.lse = a->lse;
  p.batch = s.batch;
  p.heads = s.heads_q;
  p.seq_kv = s.seq_kv;
  p.seq_lens = a->seq_lens;
  p.block_table = a->block_table;
  p.bt_stride = a->block_table_stride;
  p.page_rows = paged ? a->page_size : 0;
  const bool scheduled = a->num_splits == 0;
  const int splits = scheduled ? 1 : a->num_splits;
  p.num_splits = splits;
  p.tiles_per_split = (total_tiles + splits - 1) / splits;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(2, splits * p.head_blocks, s.batch);  // x = the two CTAs of a cluster
  if (scheduled) {
    // one cluster per SM pair and head block runs the units the scheduler gives it
    const int parts = a->sched_meta != nullptr ? a->sched_parts : mla_num_parts(s.heads_q, current_sm_count());
    if (parts <= 0) return ATTN_B200_E_INVALID_ARG;
    const MlaSchedLayout lay(s, parts);
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    int* sched = reinterpret_cast<int*>(ws);
    int* cum = reinterpret_cast<int*>(ws + lay.off_cum);
    if (a->sched_meta != nullptr) {
      if (a->sched_num_splits == nullptr) return ATTN_B200_E_INVALID_ARG;
      p.sched = a->sched_meta;
      p.num_splits_cum = a->sched_num_splits;
    } else {
      mla_schedule_kernel<<<1, 32, 0, stream>>>(a->seq_lens, s.batch, s.seq_kv, parts, sched, cum);
      if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
      p.sched = sched;
      p.num_splits_cum = cum;
    }
    p.num_parts = parts;
    p.part_o = reinterpret_cast<float*>(ws + lay.off_part_o);
    p.part_lse = reinterpret_cast<float*>(ws + lay.off_part_lse);
    grid = dim3(2, parts * p.head_blocks, 1);
  } else if (splits > 1) {
    p.part_o = static_cast<float*>(a->workspace);
    p.part_lse = p.part_o + static_cast<long long>(s.batch) * splits * s.heads_q * DV;
  }
  auto kernel = mla_split_kernel<D, DV, kBf16>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  if (grid.y > 65535) return ATTN_B200_E_UNSUPPORTED;
  kernel<<<grid, kMlaThreads, kMlaSmemBytes, stream>>>(tmKV, tmKVr, tmV, tmQr, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  if (scheduled || splits > 1) {
    const long long warps = static_cast<long long>(s.batch) * s.heads_q;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    mla_combine_kernel<DV, kBf16><<<blocks, 256, 0, stream>>>(p.part_o, p.part_lse, a->o, a->lse, s.batch, s.heads_q, splits,
                                                             scheduled ? p.num_splits_cum : nullptr);
    if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  }
  return ATTN_B200_OK;
}

}  // namespace b200

extern "C" {

int attn_b200_mla_plan(const AttnB200MlaShape* shape, int32_t sm_count, int32_t* num_splits_out) {
  int rc = b200::validate_mla_shape(shape);
  if (rc != ATTN_B200_OK) return rc;
  if (num_splits_out == nullptr || sm_count <= 0) return ATTN_B200_E_INVALID_ARG;
  // One cluster (two SMs) per (sequence, split, head block): sm_count / 2 clusters run at a time.
  // Pick the split count that fills whole waves best; every split keeps at least 4 KV tiles of 128 rows (each
  // cluster re-reads Q, and the combine pass costs one more sweep over the partial outputs).
  const long long base = static_cast<long long>((shape->heads_q + b200::kMlaHeads - 1) / b200::kMlaHeads) * shape->batch;
  const int total_tiles = (shape->seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  sm_count = sm_count / 2 > 0 ? sm_count / 2 : 1;
  // Cost model fitted to measurements on B200: a cluster spends about 14 tile-times per work unit on
  // set-up and tear-down (barriers, TMEM, Q into TMEM, pipeline fill, final exchange and store), and
  // split-KV adds the combine pass over the fp32 partials (about one tile-time per unit per 8 splits).
  int best = 1;
  double best_cost = 1e300;
  for (int s = 1; s <= 64; ++s) {
    const int tiles = (total_tiles + s - 1) / s;
    if (s > 1 && tiles < 4) break;
    if ((s - 1) * tiles >= total_tiles) continue;  // last split would be empty
    const long long units = base * s;
    const long long waves = (units + sm_count - 1) / sm_count;
    const double cost = static_cast<double>(waves) * (tiles + 14.0) + (s > 1 ? 0.125 * s * waves : 0.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  // Uniform splits against the scheduled mode (0), in tile-times, from measurements on B200 at 8192 and 2048 tokens
  // and 8..200 sequences: a cluster of the uniform mode spends its tiles + 4 per round (+ 4 more when there are
  // partial results to write and combine); a cluster of the scheduled mode walks an equal share of all tiles and pays
  // about 6.5 per piece of a sequence it touches, plus the combine pass when sequences are cut.  The scheduled mode
  // wins when the uniform rounds do not come out even (100 / 128 / 200 sequences: -12 % / -5 % / -8 %) and loses
  // when they do (64 / 74 / 148 sequences: +7 % / +2 % / +6 %).
  {
    const int tiles = (total_tiles + best - 1) / best;
    const long long units = base * best;
    const long long waves = (units + sm_count - 1) / sm_count;
    const double cost_uniform = static_cast<double>(waves) * (tiles + 4.0 + (best > 1 ? 4.0 : 0.0));
    const long long all_tiles = static_cast<long long>(shape->batch) * total_tiles;   // per head block
    const long long parts = sm_count;   // clusters (SM pairs); head blocks divide them, and the tiles alike
    const long long head_blocks = base / shape->batch;
    const long long per_part = (all_tiles * head_blocks + parts - 1) / parts;
    const bool even = per_part % total_tiles == 0;
    const long long pieces = even ? per_part / total_tiles : per_part / total_tiles + 2;
    const double cost_sched = static_cast<double>(per_part) + 6.5 * static_cast<double>(pieces) + (even ? 1.0 : 3.0);
    if (cost_sched < cost_uniform) best = 0;
  }
  *num_splits_out = best;
  return ATTN_B200_OK;
}

int32_t attn_b200_mla_num_parts(int32_t heads_q, int32_t sm_count) {
  if (heads_q <= 0 || sm_count <= 0) return -1;
  return b200::mla_num_parts(heads_q, sm_count);
}

int attn_b200_mla_metadata(const int32_t* cache_seqlens, int32_t batch, int32_t seq_kv, int32_t num_parts,
                           int32_t* tile_scheduler_metadata, int32_t* num_splits, void* cuda_stream) {
  if (tile_scheduler_metadata == nullptr || num_splits == nullptr || batch <= 0 || seq_kv <= 0 || num_parts <= 0)
    return ATTN_B200_E_INVALID_ARG;
  b200::mla_schedule_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(cache_seqlens, batch, seq_kv, num_parts,
                                                                                 tile_scheduler_metadata, num_splits);
  return cudaGetLastError() == cudaSuccess ? ATTN_B200_OK : ATTN_B200_E_LAUNCH;
}

int64_t attn_b200_mla_workspace_bytes(const AttnB200MlaShape* shape, int32_t num_splits) {
  if (b200::validate_mla_shape(shape) != ATTN_B200_OK || num_splits < 0) return -1;
  if (num_splits == 0) {   // scheduled mode on the current device
    const int sms = b200::current_sm_count();
    if (sms <= 0) return -1;
    return b200::MlaSchedLayout(*shape, b200::mla_num_parts(shape->heads_q, sms)).bytes;
  }
  if (num_splits == 1) return 0;
  const int64_t rows = static_cast<int64_t>(shape->batch) * num_splits * shape->heads_q;
  return rows * shape->dim_v * 4 + rows * 4;
}

int attn_b200_mla_decode(const AttnB200MlaArgs* a, void* cuda_stream) {
  if (a == nullptr || a->q == nullptr || a->kv == nullptr || a->o == nullptr) return ATTN_B200_E_INVALID_ARG;
  int rc = b200::validate_mla_shape(&a->shape);
  if (rc != ATTN_B200_OK) return rc;
  if (a->dtype != ATTN_B200_DTYPE_FP16 && a->dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a->num_splits < 0 || a->num_splits > 32767) return ATTN_B200_E_INVALID_ARG;
  const int total_tiles = (a->shape.seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  if (a->num_splits > total_tiles) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  int64_t need = attn_b200_mla_workspace_bytes(&a->shape, a->num_splits);
  if (a->num_splits == 0 && a->sched_meta != nullptr) {
    if (a->sched_parts <= 0) return ATTN_B200_E_INVALID_ARG;
    need = b200::MlaSchedLayout(a->shape, a->sched_parts).bytes;
  }
  if (need < 0) return ATTN_B200_E_LAUNCH;
  if (need > 0 && (a->workspace == nullptr || a->workspace_bytes < need)) return ATTN_B200_E_WORKSPACE;
  if (need > 0 && (reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0) return ATTN_B200_E_WORKSPACE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ATTN_B200_E_LAUNCH;
  int* status = b200::device_status_word(dev);
  if (status == nullptr) return ATTN_B200_E_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  return a->dtype == ATTN_B200_DTYPE_BF16 ? b200::launch_mla<true>(a, stream, status) : b200::launch_mla<false>(a, stream, status);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the MLA decode entry point.
//
// Who needs it: hosts that must not call cudaMalloc (or anything that does) around the decode.
// Typical cases are a serving process whose own arena already owns all of the device memory, so
// that a further cudaMalloc either fails or has to be carved out of that arena by hand, and
// latency-critical loops that cannot afford the implicit device-wide synchronisation and the
// unpredictable duration of a driver allocation.  The regular entry point needs two pieces of
// device memory besides inputs and outputs: the split-KV scratch (fp32 partial outputs and partial
// log-sum-exps, normally handed in by the caller as `workspace`) and the library's status word
// (allocated with cudaMalloc on first use).  Here the scratch is a fixed array in the library's
// own device data segment and the status word is supplied by the caller, so the call performs no
// allocation of any kind.
//
// Cost and limits: every GPU on which the library gets loaded carries the array (32 MiB) until the
// process exits, used or not.  Problems whose scratch does not fit are refused with
// ATTN_B200_E_SCRATCH_LIMIT; nothing is launched in that case.  All calls on one device share the
// one array, and it keeps whatever the previous call left in it.  Nothing in it has to start at
// zero: every row the combine pass reads was written by the split pass of the same call, and rows
// it does not read are ignored.  The only word that must start at zero is the caller's status
// word, which the call clears itself (a memset on the same stream, ahead of the kernels).  Two calls
// that overlap on the GPU -- different streams, or one stream from two threads without ordering --
// race on the array and produce garbage; serialise them.
//
// Set-up: the address of the array is looked up once per device, on the first call made while
// that device is current (cudaGetSymbolAddress; the name of the array is only a host-side handle,
// not a device address, so it cannot be passed to a kernel directly).  Make that first call
// before any stream capture is started on the device.
// ---------------------------------------------------------------------------------------------
namespace b200 {

constexpr size_t kMlaStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_mla_static_scratch[kMlaStaticScratchBytes];

// Device address of the array for the current device; null on failure.  Looked up once per device.
static void* mla_static_scratch_ptr() {
  constexpr int kMaxDevices = 64;
  static void* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_mla_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace b200

extern "C" int attn_b200_mla_decode_static(const AttnB200MlaArgs* a, int32_t* status_word, void* cuda_stream) {
  if (a == nullptr || a->q == nullptr || a->kv == nullptr || a->o == nullptr || status_word == nullptr)
    return ATTN_B200_E_INVALID_ARG;
  int rc = b200::validate_mla_shape(&a->shape);
  if (rc != ATTN_B200_OK) return rc;
  if (a->dtype != ATTN_B200_DTYPE_FP16 && a->dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a->num_splits < 0 || a->num_splits > 32767) return ATTN_B200_E_INVALID_ARG;
  const int total_tiles = (a->shape.seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  if (a->num_splits > total_tiles) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0 || (reinterpret_cast<uintptr_t>(status_word) & 3) != 0)
    return ATTN_B200_E_UNSUPPORTED;
  int64_t need = attn_b200_mla_workspace_bytes(&a->shape, a->num_splits);
  if (a->num_splits == 0 && a->sched_meta != nullptr && a->sched_parts > 0) need = b200::MlaSchedLayout(a->shape, a->sched_parts).bytes;
  if (need < 0) return ATTN_B200_E_UNSUPPORTED;
  if (static_cast<uint64_t>(need) > b200::kMlaStaticScratchBytes) return ATTN_B200_E_SCRATCH_LIMIT;
  void* scratch = b200::mla_static_scratch_ptr();
  if (scratch == nullptr) return ATTN_B200_E_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // the kernels give up at once when they find a non-zero status word: start every call from zero
  if (cudaMemsetAsync(status_word, 0, sizeof(int32_t), stream) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  AttnB200MlaArgs local = *a;  // the caller's workspace fields are ignored
  local.workspace = need > 0 ? scratch : nullptr;
  local.workspace_bytes = need;
  return a->dtype == ATTN_B200_DTYPE_BF16 ? b200::launch_mla<true>(&local, stream, status_word)
                                          : b200::launch_mla<false>(&local, stream, status_word);
}
