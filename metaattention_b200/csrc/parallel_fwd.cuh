// Kernel family (1): parallel-pattern attention forward for sm_100a.
//
//   O = epilogue( sum over KV tiles of  o_scale-rescaled  P.V ),
//   P = online_fwd( score_mod( mask + Q.K^T ) )
//
// with score_mod / online_fwd / epilogue supplied by a device functor F (the
// lowered form of the user's score_mod and OnlineFunc).  Replaces the
// generated TileLang kernel of the reference
// (attention_engine/core/template/tl_template/attn/attn_tl.py:93-190) and its
// CuTe warp-specialised forward (core/template/cute_template/flash_fwd_kernel.h:28-199).
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the KV
// sequence in 128-row tiles:
//   warp 8      TMA producer: Q once, then K and V tiles into 2-stage rings
//   warp 9      tcgen05.mma issuer (one thread): S_t = Q_t.K^T into TMEM,
//               O_t += P_t.V with P_t read from TMEM (aliasing S_t)
//   warps 0-3   row-per-thread functor stage for query tile 0
//   warps 4-7   same for query tile 1
// The two query tiles ping-pong: while the functor stage of one tile runs on
// the CUDA cores, the tensor pipe works on the other tile.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+DV) O1 [256+DV,256+2DV).
// Masks are bands kv_idx in [q_idx - left, q_idx + right] (none / causal / explicit bounds): a query tile
// walks only the KV tiles its band touches, the CTA loads the union of its two tiles' ranges, and tiles
// that cross an edge of the band are masked element by element.  K/V heads may be shared by groups of
// query heads (kv_group).  The same kernel serves q_len != kv_len (decode patterns).
// Start and end of a CTA: the producer lane initialises the barriers and issues the query tiles and the first K/V
// tiles before the tensor-memory allocation and the CTA-wide sync; the output rows of a tile are staged in its
// query buffer and stored as whole rows.
#pragma once

#include <type_traits>

#include "sm100.cuh"

namespace b200 {

constexpr int kMaxCustom = 4;
constexpr int kNoBound = 0x3fffffff;   // an open side of the mask band
constexpr int kMaxRowScales = 4;

struct FunctorArgs {
  float f[8];
  const void* custom[kMaxCustom];
  long long cstride[kMaxCustom][4];  // element strides of (batch, heads, seq_len, seq_len_kv)
};

// What a functor knows about the row it is working on.
// A functor may offer tile_halves<N>() (see SoftmaxFunctor) beside tile<N>().
template <class F, class = void>
struct functor_half_store : std::false_type {};
template <class F>
struct functor_half_store<F, std::void_t<decltype(F::kHalfStore)>> : std::integral_constant<bool, F::kHalfStore> {};

struct RowCtx {
  int b, h, q_idx;   // batch, head, query position of this thread's row
  int kv0;           // first KV position of the current tile
  int seq_q, seq_kv;
  const FunctorArgs* fa;
};

// Position (1..3) of the head / sequence / batch coordinate inside a 4-D
// tensor map whose dimension 0 is the feature dimension; the host sorts the
// three outer dimensions by stride.
struct CoordOrder {
  int pos_s, pos_h, pos_b;
};

struct ParallelParams {
  void* o;
  float* final_out[kMaxRowScales];
  int batch, heads, seq_q, seq_kv;
  int kv_group;                // query heads per KV head (1 = one KV head per query head)
  int kv_splits;               // > 1: blockIdx.z = batch * kv_splits + split, each split covers tiles_per_split KV tiles
  int tiles_per_split;
  float* part_o;               // [batch, kv_splits, heads, seq_q, dim_v] fp32 results of the splits (kv_splits > 1)
  float* part_final;           // [kFinal][batch, kv_splits, heads, seq_q] their final row scales
  long long part_final_stride; // elements between two final row scales in part_final
  // Block sparsity (kSparse kernels): per (sparse batch, sparse head, 128-row query tile) a bitmap of the 128-row KV
  // tiles to visit and one of the tiles among them that need the element mask.
  const uint32_t* tile_keep;   // [sparse_batch][sparse_heads][q_tiles][tile_words]
  const uint32_t* tile_partial;
  const int* tile_mask_base;   // [sparse_batch][sparse_heads][q_tiles] first element-mask slot of the query tile, or null
  const uint32_t* elem_mask;   // slots of [elem_mask_rows][4] words (bit = keep), or with elem_mask_rows == 0 one
                               // [4]-word column mask per (sparse batch, sparse head, KV tile)
  int sparse_batch, sparse_heads, tile_words, elem_mask_rows;
  long long o_sb, o_ss, o_sh;  // element strides of o
  int mask_kind;               // 0 none, 1 causal (keep q_idx >= kv_idx), 2 band
  int win_left, win_right;     // band: keep kv_idx in [q_idx - win_left, q_idx + win_right]; kNoBound = open side
  CoordOrder oq, ok, ov;
  int* status;
  FunctorArgs fa;
};

__device__ __forceinline__ void tma_load_rows(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int s, int h,
                                              int b, const CoordOrder& o) {
  const int c1 = (o.pos_s == 1) ? s : (o.pos_h == 1) ? h : b;
  const int c2 = (o.pos_s == 2) ? s : (o.pos_h == 2) ? h : b;
  const int c3 = (o.pos_s == 3) ? s : (o.pos_h == 3) ? h : b;
  tma_load_4d(dst, tm, bar, c0, c1, c2, c3);
}

// wait-site ids reported through the device status word
enum ParallelWaitSite {
  kSiteQFull = 1, kSiteKFull, kSiteVFull, kSiteKEmpty, kSiteVEmpty, kSiteSFull, kSitePReady, kSiteODone, kSiteOFinal
};

// Walks the set bits of one bitmap, or of the union of two, in increasing order (KV tile indices of a sparse walk).
struct TileWalk {
  const uint32_t* a;
  const uint32_t* b;
  int words, w;
  uint32_t bits;
  __device__ TileWalk(const uint32_t* a_, const uint32_t* b_, int words_) : a(a_), b(b_), words(words_), w(-1), bits(0) {}
  __device__ int next() {
    while (bits == 0) {
      if (++w >= words) return -1;
      bits = a[w] | (b != nullptr ? b[w] : 0u);
    }
    const int j = w * 32 + __ffs(bits) - 1;
    bits &= bits - 1;
    return j;
  }
};

constexpr int kMaxTileWords = 128;   // sparse walks: at most 4096 KV tiles (512 k tokens)

// NT = query tiles per CTA: 2 (K/V in two stages, shared by both tiles) or 1 (single-staged K/V; the layout that
// fits dim_qk = 256: one 64 KB query tile, 64 KB of K, 32 KB of V)
template <int D, int DV, int NT = 2>
struct ParallelSmem {
  static constexpr int kBM = 128, kBN = 128, kStages = NT == 2 ? 2 : 1;
  static constexpr int kQBytes = kBM * D * 2;
  static constexpr int kKBytes = kBN * D * 2;
  static constexpr int kVBytes = kBN * DV * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + NT * kQBytes;
  static constexpr int kOffV = kOffK + kStages * kKBytes;
  static constexpr int kOffBar = kOffV + kStages * kVBytes;
  static constexpr int kNumBars = 2 + 4 * kStages + 6;
  static constexpr int kOffMisc = kOffBar + 8 * kNumBars;
  static constexpr int kOffSparse = kOffMisc + 16;     // sparse kernels: keep / partial bitmaps of the two query tiles
  static constexpr int kBytes = kOffMisc + 16 + 1024;  // + slack for manual 1024-byte alignment
  static constexpr int kBytesSparse = kBytes + 4 * kMaxTileWords * 4;
};

template <class F, int D, int DV, bool kBf16, int NT = 2, bool kSparse = false>
__global__ void __launch_bounds__((4 * NT + 2) * 32, 1)
parallel_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const ParallelParams p) {
  using L = ParallelSmem<D, DV, NT>;
  constexpr int BM = L::kBM, BN = L::kBN, ST = L::kStages;
  static_assert(D % 64 == 0 && DV % 64 == 0 && DV <= 128 && (D <= 128 || (D <= 256 && NT == 1)), "unsupported head dims");
  static_assert((kSparse ? L::kBytesSparse : L::kBytes) <= 232448, "shared memory layout exceeds an SM");
  constexpr uint32_t kTmemCols = NT == 2 ? 512 : 256;
  constexpr uint32_t kColS = 0, kColO = NT * 128;
  constexpr int kTmaWarp = 4 * NT, kMmaWarp = 4 * NT + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars;          // [2] one per query tile
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + ST;
  uint64_t* v_full = k_empty + ST;
  uint64_t* v_empty = v_full + ST;
  uint64_t* s_full = v_empty + ST;   // [2] one per query tile
  uint64_t* p_ready = s_full + 2;    // [2]
  uint64_t* o_done = p_ready + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortState ab{abort_flag, p.status};

  // Every mask is a band kv_idx in [q_idx - left, q_idx + right]: none = open on both sides, causal = open
  // to the left with right = 0, sliding windows bound the left side as well.
  const bool causal = p.mask_kind == 1;
  const int left = p.mask_kind == 2 ? p.win_left : kNoBound;
  const int right = p.mask_kind == 0 ? kNoBound : (p.mask_kind == 1 ? 0 : p.win_right);
  const bool banded = p.mask_kind != 0;
  // heaviest query tiles (largest KV range under a causal mask) are launched first
  const int m_pair = causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int h = blockIdx.y;
  const int b = p.kv_splits > 1 ? blockIdx.z / p.kv_splits : blockIdx.z;
  const int split = p.kv_splits > 1 ? blockIdx.z % p.kv_splits : 0;
  const int m0 = m_pair * NT * BM;
  const int n_kv_tiles = (p.seq_kv + BN - 1) / BN;
  // KV tiles [j_lo, j_hi) of each query tile; the CTA walks the union [j_min, j_max)
  int j_lo[2], j_hi[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int row0 = m0 + t * BM;
    j_lo[t] = j_hi[t] = 0;
    if (t < NT && row0 < p.seq_q) {
      j_lo[t] = (left >= kNoBound || row0 <= left) ? 0 : (row0 - left) / BN;
      j_hi[t] = right >= kNoBound ? n_kv_tiles : min(n_kv_tiles, (row0 + BM - 1 + right) / BN + 1);
      if (p.kv_splits > 1) {   // this CTA's share of the KV tiles
        j_lo[t] = max(j_lo[t], split * p.tiles_per_split);
        j_hi[t] = min(j_hi[t], (split + 1) * p.tiles_per_split);
      }
      if (j_hi[t] < j_lo[t]) j_hi[t] = j_lo[t];
    }
  }
  bool act0 = j_hi[0] > j_lo[0], act1 = j_hi[1] > j_lo[1];
  const int j_min = act0 ? (act1 ? min(j_lo[0], j_lo[1]) : j_lo[0]) : j_lo[1];
  const int j_max = max(act0 ? j_hi[0] : 0, act1 ? j_hi[1] : 0);
  int n_max = (act0 || act1) ? j_max - j_min : 0;
  // Sparse walk: the bitmaps of this CTA's two query tiles are copied to shared memory (a query tile past the end of
  // the sequence gets an empty one); n_tiles[t] = KV tiles of tile t, n_max = tiles of the union.
  uint32_t* sp_keep = reinterpret_cast<uint32_t*>(smem + L::kOffSparse);      // [2][kMaxTileWords]
  uint32_t* sp_part = sp_keep + 2 * kMaxTileWords;                           // [2][kMaxTileWords]
  int n_tiles[2] = {0, 0};
  int sp_row[2] = {0, 0};       // index of (sparse batch, sparse head, query tile) for each of the two tiles
  if constexpr (kSparse) {
    const int sb = p.sparse_batch > 1 ? b : 0;
    const int sh = p.sparse_heads <= 1 ? 0 : (p.sparse_heads == p.heads ? h : h / (p.heads / p.sparse_heads));
    const int q_tiles = (p.seq_q + BM - 1) / BM;
    for (int t = 0; t < 2; ++t) {
      const int qt = m_pair * NT + t;
      const bool exists = t < NT && qt < q_tiles;
      sp_row[t] = (sb * p.sparse_heads + sh) * q_tiles + (exists ? qt : 0);
      for (int w = threadIdx.x; w < p.tile_words; w += blockDim.x) {
        sp_keep[t * kMaxTileWords + w] = exists ? p.tile_keep[static_cast<long long>(sp_row[t]) * p.tile_words + w] : 0u;
        sp_part[t * kMaxTileWords + w] = exists ? p.tile_partial[static_cast<long long>(sp_row[t]) * p.tile_words + w] : 0u;
      }
    }
    __syncthreads();
    n_max = 0;
    for (int w = 0; w < p.tile_words; ++w) {
      n_tiles[0] += __popc(sp_keep[w]);
      n_tiles[1] += __popc(sp_keep[kMaxTileWords + w]);
      n_max += __popc(sp_keep[w] | sp_keep[kMaxTileWords + w]);
    }
    act0 = n_tiles[0] > 0;
    act1 = n_tiles[1] > 0;
  }
  auto active = [&](int t, int j) {
    if constexpr (kSparse) return j >= 0 && ((sp_keep[t * kMaxTileWords + (j >> 5)] >> (j & 31)) & 1u) != 0;
    else return j >= j_lo[t] && j < j_hi[t];
  };

  // ---------------- setup ----------------
  // The producer lane initialises the barriers and sends off the query tiles and the first K and V tiles at once:
  // their ~2800 cycles of latency start before the tensor-memory allocation and the CTA-wide sync, not after.
  auto load_k_tile = [&](int i, int j) {   // KV tile j into the stage of step i
    const int st = i % ST;
    mbar_arrive_expect_tx(&k_full[st], L::kKBytes);
    for (int c = 0; c < D / 64; ++c)
      tma_load_rows(sK + st * L::kKBytes + c * (BN * 128), &tmK, &k_full[st], c * 64, j * BN, h / p.kv_group, b, p.ok);
  };
  auto load_v_tile = [&](int i, int j) {
    const int st = i % ST;
    mbar_arrive_expect_tx(&v_full[st], L::kVBytes);
    for (int c = 0; c < DV / 64; ++c)
      tma_load_rows(sV + st * L::kVBytes + c * (BN * 128), &tmV, &v_full[st], c * 64, j * BN, h / p.kv_group, b, p.ov);
  };
  auto load_k = [&](int i) { load_k_tile(i, j_min + i); };
  auto load_v = [&](int i) { load_v_tile(i, j_min + i); };
  auto load_q = [&](int t) {
    mbar_arrive_expect_tx(&q_full[t], L::kQBytes);
    for (int c = 0; c < D / 64; ++c)
      tma_load_rows(sQ + t * L::kQBytes + c * (BM * 128), &tmQ, &q_full[t], c * 64, m0 + t * BM, h, b, p.oq);
  };
  bool early_loads = false;
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], 128);
      mbar_init(&o_done[t], 1);
    }
    fence_barrier_init();
    if (n_max > 0 && !kSparse) {
      // in the order of first use: query tile 0 and K so that its scores can start, then query tile 1, then V
      const int nq = act1 ? 2 : 1;
      load_q(0);
      load_k(0);
      if (nq > 1) load_q(1);
      load_v(0);
      early_loads = true;
    }
  }
  // The device status word (set by a CTA whose wait ran out) is read by another thread meanwhile: a global-memory
  // round trip that the first loads do not wait for.  If it is set, nobody consumes those loads and the teardown
  // below gives them time to land.
  if (threadIdx.x == 0) *abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kTmaWarp) {
    // =============== TMA producer ===============
    if constexpr (kSparse) {
      if (lane == 0 && n_max > 0 && !*abort_flag) {
        TileWalk walk(sp_keep, sp_keep + kMaxTileWords, p.tile_words);
        load_q(0);
        if (NT > 1 && act1) load_q(1);
        for (int i = 0; i < n_max; ++i) {
          const int j = walk.next();
          const int st = i % ST;
          const uint32_t ph = (i / ST) & 1;
          if (i >= ST && !mbar_wait(&k_empty[st], ph ^ 1, ab, kSiteKEmpty)) break;
          load_k_tile(i, j);
          if (i >= ST && !mbar_wait(&v_empty[st], ph ^ 1, ab, kSiteVEmpty)) break;
          load_v_tile(i, j);
        }
      }
    } else if (lane == 0 && early_loads && !*abort_flag) {
      for (int i = 1; i < n_max; ++i) {
        const int st = i % ST;
        const uint32_t ph = (i / ST) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, ab, kSiteKEmpty)) break;
        load_k(i);
        if (!mbar_wait(&v_empty[st], ph ^ 1, ab, kSiteVEmpty)) break;
        load_v(i);
      }
    }
  } else if (warp == kMmaWarp) {
    // =============== MMA issuer ===============
    // The whole warp runs this code converged; one elected lane issues each batch of MMAs with its commit.  The
    // descriptors then live in uniform registers and a batch leaves at the tensor pipe's rate whatever the functor
    // warps do: issued from inside an `if (lane == 0)` region an MMA with N = 128 took ~90 cycles beside busy warps,
    // against the 64 the pipe needs for it.
    if (n_max > 0 && __all_sync(0xffffffffu, !*abort_flag)) {
      auto wait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, ab, site));
      };
      auto wait_poll = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
        return __all_sync(0xffffffffu, mbar_wait_poll(bar, parity, ab, site));
      };
      auto commit2 = [&](uint64_t* c1, uint64_t* c2) {
        if (elect_one()) {
          umma_commit(c1);
          if (c2 != nullptr) umma_commit(c2);
        }
      };
      constexpr uint32_t idesc_qk = make_idesc_f16(BM, BN, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(BM, DV, kBf16, false, true);
      // Descriptors are built once; per MMA only the start-address field moves (units of 16 bytes), and four
      // K steps go out per asm block: the issuing lane's instruction count is latency in front of the tensor pipe.
      const uint64_t q_desc0 = make_smem_desc(smem_u32(sQ), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc(smem_u32(sK), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc(smem_u32(sV), BN * 128, 1024);
      auto issue_qk = [&](int t, int st) {
        const uint64_t a = q_desc0 + static_cast<uint64_t>(t * (L::kQBytes >> 4));
        const uint64_t bq = k_desc0 + static_cast<uint64_t>(st * (L::kKBytes >> 4));
        if (elect_one()) {
#pragma unroll
          for (int ch = 0; ch < D / 64; ++ch)
            umma_ss_x4<2, 2>(tmem_base + kColS + t * BN, a + ch * ((BM * 128) >> 4), bq + ch * ((BN * 128) >> 4), idesc_qk, ch > 0 ? 1u : 0u);
          umma_commit(&s_full[t]);
        }
      };
      auto issue_pv = [&](int t, int st, bool first) {
        const uint64_t bv = v_desc0 + static_cast<uint64_t>(st * (L::kVBytes >> 4));
        if (elect_one()) {
#pragma unroll
          for (int g = 0; g < BN / 64; ++g)   // 16 KV rows (2048 B) per K step, P advances 8 TMEM columns
            umma_ts_x4<8, 128>(tmem_base + kColO + t * DV, tmem_base + kColS + t * BN + g * 32, bv + g * 512, idesc_pv,
                               (!first || g > 0) ? 1u : 0u);
          umma_commit(&o_done[t]);
        }
      };
      bool ok = wait(&q_full[0], 0, kSiteQFull);
      ok = ok && wait(&k_full[0], 0, kSiteKFull);
      if constexpr (kSparse) {
        // the same schedule over the union of the two tiles' KV tile sets; a tile takes part in a step when the
        // step's KV tile is in its own set, and its barrier phases count its own tiles
        TileWalk walk(sp_keep, sp_keep + kMaxTileWords, p.tile_words);
        int j = walk.next();
        int done[2] = {0, 0};
        if (ok) {
          tc_fence_after_sync();
          if (active(0, j)) issue_qk(0, 0);
          if (NT > 1 && act1) {
            ok = wait(&q_full[1], 0, kSiteQFull);
            tc_fence_after_sync();
            if (ok && active(1, j)) issue_qk(1, 0);
          }
          commit2(&k_empty[0], nullptr);
        }
        for (int i = 0; i < n_max && ok; ++i) {
          const int jn = walk.next();
          const int st = i % ST;
          const int stn = (i + 1) % ST;
          ok = wait(&v_full[st], (i / ST) & 1, kSiteVFull);
          if (ok && jn >= 0) ok = wait(&k_full[stn], ((i + 1) / ST) & 1, kSiteKFull);
          if (!ok) break;
          for (int t = 0; t < NT; ++t) {
            if (active(t, j)) {
              ok = wait_poll(&p_ready[t], done[t] & 1, kSitePReady);
              if (!ok) break;
              tc_fence_after_sync();
              issue_pv(t, st, done[t] == 0);
              ++done[t];
            }
            if (active(t, jn)) issue_qk(t, stn);
          }
          if (!ok) break;
          commit2(&v_empty[st], jn >= 0 ? &k_empty[stn] : nullptr);
          j = jn;
        }
      } else if (ok) {
        tc_fence_after_sync();
        if (active(0, j_min)) issue_qk(0, 0);
        if (NT > 1 && act1) {
          ok = wait(&q_full[1], 0, kSiteQFull);
          tc_fence_after_sync();
          if (ok && active(1, j_min)) issue_qk(1, 0);
        }
        commit2(&k_empty[0], nullptr);
        for (int i = 0; i < n_max && ok; ++i) {
          const int j = j_min + i;
          const int st = i % ST;
          const int stn = (i + 1) % ST;
          ok = wait(&v_full[st], (i / ST) & 1, kSiteVFull);
          if (ok && i + 1 < n_max) ok = wait(&k_full[stn], ((i + 1) / ST) & 1, kSiteKFull);
          if (!ok) break;
          for (int t = 0; t < NT; ++t) {
            if (active(t, j)) {
              // on the serial chain of the tile: polled, a suspended wait wakes up ~150 cycles late
              ok = wait_poll(&p_ready[t], (j - j_lo[t]) & 1, kSitePReady);
              if (!ok) break;
              tc_fence_after_sync();
              issue_pv(t, st, j == j_lo[t]);
            }
            // the tile's next scores; also its first ones when its KV range starts later than the other tile's
            if (active(t, j + 1)) issue_qk(t, stn);
          }
          if (!ok) break;
          commit2(&v_empty[st], i + 1 < n_max ? &k_empty[stn] : nullptr);
        }
      }
    }
  } else {
    // =============== functor stage: one query row per thread ===============
    const int t = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int q_idx = m0 + t * BM + row;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + t * BN;
    const uint32_t tO = tmem_base + lane_base + kColO + t * DV;
    const int n = kSparse ? n_tiles[t] : j_hi[t] - j_lo[t];
    const int row0 = m0 + t * BM;
    TileWalk walk(sp_keep + t * kMaxTileWords, nullptr, kSparse ? p.tile_words : 0);
    int mask_slot = (kSparse && p.tile_mask_base != nullptr) ? p.tile_mask_base[sp_row[t]] : 0;
    float rs[F::kRowScales > 0 ? F::kRowScales : 1];
    RowCtx ctx{b, h, q_idx, 0, p.seq_q, p.seq_kv, &p.fa};
    F::init(rs, ctx);
    bool ok = (n > 0) && !*abort_flag;
    for (int j = 0; j < n && ok; ++j) {   // j counts this query tile's own KV tiles
      ok = mbar_wait(&s_full[t], j & 1, ab, kSiteSFull);
      if (!ok) break;
      tc_fence_after_sync();
      float s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld32f(tS + c * 32, &s[c * 32]);
      tmem_wait_ld();
      const int jt = kSparse ? walk.next() : j_lo[t] + j;   // KV tile of this step
      const int kv0 = jt * BN;
      ctx.kv0 = kv0;
      if constexpr (kSparse) {
        // element mask of a partial tile: 128 keep bits for this thread's row (or one column mask for all rows)
        if (F::kNegInfMask && ((sp_part[t * kMaxTileWords + (jt >> 5)] >> (jt & 31)) & 1u) != 0) {
          const uint32_t* mrow;
          if (p.elem_mask_rows > 0) {
            mrow = p.elem_mask + (static_cast<long long>(mask_slot) * p.elem_mask_rows + row) * 4;
            ++mask_slot;
          } else {
            const int n_kv = (p.seq_kv + BN - 1) / BN;
            mrow = p.elem_mask + ((static_cast<long long>(sp_row[t]) / ((p.seq_q + BM - 1) / BM)) * n_kv + jt) * 4;
          }
          const uint4 mw = *reinterpret_cast<const uint4*>(mrow);
          const uint32_t words[4] = {mw.x, mw.y, mw.z, mw.w};
#pragma unroll
          for (int i = 0; i < BN; ++i) s[i] = ((words[i >> 5] >> (i & 31)) & 1u) ? s[i] : -INFINITY;
        }
      }
      // a tile needs element masking when it crosses an edge of the mask band or the end of the KV sequence
      const bool crosses = (banded && ((right < kNoBound && kv0 + BN - 1 > row0 + right) ||
                                       (left < kNoBound && kv0 < row0 + BM - 1 - left))) || (kv0 + BN > p.seq_kv);
      if (crosses) {
        if (F::kNegInfMask) {
          const int kv_first = left < kNoBound ? q_idx - left : -kNoBound;
          const int kv_last = right < kNoBound ? min(q_idx + right, p.seq_kv - 1) : p.seq_kv - 1;
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            const int kv = kv0 + i;
            const bool keep = (kv >= kv_first) && (kv <= kv_last);
            s[i] = keep ? s[i] : -INFINITY;
          }
        }
      }
      // P (16-bit, two per column) overwrites the first BN/2 columns of S
      auto store_half = [&](int c) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = pack2<kBf16>(s[c * 64 + 2 * i], s[c * 64 + 2 * i + 1]);
        tmem_st32(tS + c * 32, pk);
      };
      float o_scale;
      if constexpr (functor_half_store<F>::value && BN == 128) {
        // the functor hands over a piece of the row (BN / kPieces columns) as soon as its probabilities are final: the
        // piece is on its way to tensor memory while the exponentials of the next one run
        o_scale = F::template tile_pieces<BN>(s, rs, ctx, [&](int c) {
          constexpr int W = BN / F::kPieces / 2;   // packed columns per piece
          uint32_t pk[W];
#pragma unroll
          for (int i = 0; i < W; ++i) pk[i] = pack2<kBf16>(s[c * 2 * W + 2 * i], s[c * 2 * W + 2 * i + 1]);
          if constexpr (W == 32) tmem_st32(tS + c * W, reinterpret_cast<const uint32_t(&)[32]>(pk));
          else if constexpr (W == 16) tmem_st16(tS + c * W, pk);
          else tmem_st8(tS + c * W, pk);
        });
      } else if constexpr (F::kUnitOScale && BN == 128) {
        // no rescale: the row can be handed to the functor as four narrower tiles, each stored as soon as it is done
        o_scale = 1.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          ctx.kv0 = kv0 + c * 32;
          F::template tile<32>(reinterpret_cast<float(&)[32]>(s[c * 32]), rs, ctx);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack2<kBf16>(s[c * 32 + 2 * i], s[c * 32 + 2 * i + 1]);
          tmem_st16(tS + c * 16, pk);
        }
        ctx.kv0 = kv0;
      } else {
        o_scale = F::template tile<BN>(s, rs, ctx);
#pragma unroll
        for (int c = 0; c < BN / 64; ++c) store_half(c);
      }
      if (!F::kUnitOScale && j > 0) {
        const bool need = (o_scale != 1.0f);
        if (__any_sync(0xffffffffu, need)) {
          ok = mbar_wait(&o_done[t], (j - 1) & 1, ab, kSiteODone);
          if (ok) {
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < DV / 32; ++c) {
              float o[32];
              tmem_ld32f(tO + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= o_scale;
              tmem_st32f(tO + c * 32, o);
            }
          }
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[t]);
    }
    // a query tile of a sparse walk that visits no KV tile at all still owes its output rows: the epilogue of an
    // empty accumulator (what the reference's kernel leaves there as well)
    const bool empty_tile = kSparse && n == 0 && t < NT && row0 < p.seq_q && !*abort_flag;
    if ((ok && n > 0) || empty_tile) {
      ok = n > 0 ? mbar_wait(&o_done[t], (n - 1) & 1, ab, kSiteOFinal) : true;
      if (ok) {
        tc_fence_after_sync();
        const bool in_range = q_idx < p.seq_q;
        float o[DV];
        if (n > 0) {
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) tmem_ld32f(tO + c * 32, &o[c * 32]);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < DV; ++i) o[i] = 0.0f;
        }
        F::template epilogue<DV>(o, rs, ctx);
        if (p.kv_splits > 1) {
          // split-KV: the normalised rows and their log-sum-exp go to the scratch the combine kernel reads
          if (in_range) {
            const long long prow = ((static_cast<long long>(b) * p.kv_splits + split) * p.heads + h) * p.seq_q + q_idx;
            float4* dst = reinterpret_cast<float4*>(p.part_o + prow * DV);
#pragma unroll
            for (int v = 0; v < DV / 4; ++v) dst[v] = make_float4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
#pragma unroll
            for (int i = 0; i < F::kFinal; ++i) p.part_final[i * p.part_final_stride + prow] = F::final_rowscale(i, rs, ctx);
          }
        } else {
          // Output rows leave through the tile's own Q buffer (free: its last Q.K^T ran before the P.V that o_done
          // reports).  Each warp owns the 32 rows it computed, so a warp-level sync is enough: every lane writes its
          // row in 16-byte pieces (piece index xor row: conflict-free), then the warp stores whole rows, DV*2
          // contiguous bytes per row and 512 bytes per instruction.  A thread storing its own row put 32 pieces
          // into 32 different rows with every instruction, and the tile's last output took ~3100 cycles.
          static_assert(DV <= D, "the output tile is staged in the query tile's buffer");
          constexpr int PR = DV / 8;     // 16-byte pieces per row
          constexpr int RPI = 32 / PR;   // rows per warp instruction
          const uint32_t stage = smem_u32(sQ + t * L::kQBytes) + (warp & 3) * (32 * DV * 2);
          const uint32_t mine = stage + lane * (DV * 2);
#pragma unroll
          for (int v = 0; v < PR; ++v) {
            uint4 pk;
            pk.x = pack2<kBf16>(o[8 * v + 0], o[8 * v + 1]);
            pk.y = pack2<kBf16>(o[8 * v + 2], o[8 * v + 3]);
            pk.z = pack2<kBf16>(o[8 * v + 4], o[8 * v + 5]);
            pk.w = pack2<kBf16>(o[8 * v + 6], o[8 * v + 7]);
            st_shared_v4(mine + ((v ^ (lane & (PR - 1))) << 4), pk);
          }
          __syncwarp();
          const int c = lane & (PR - 1), rsub = lane / PR;
          const int row_first = row0 + (warp & 3) * 32;
          uint8_t* obase = reinterpret_cast<uint8_t*>(p.o) +
                           2 * (static_cast<long long>(b) * p.o_sb + static_cast<long long>(h) * p.o_sh) + c * 16;
          uint4 val[PR];   // all loads first, then all stores: one after the other each pair costs a shared-memory round trip
#pragma unroll
          for (int i = 0; i < PR; ++i) {
            const int r = i * RPI + rsub;
            val[i] = ld_shared_v4(stage + r * (DV * 2) + ((c ^ (r & (PR - 1))) << 4));
          }
#pragma unroll
          for (int i = 0; i < PR; ++i) {
            const int r = i * RPI + rsub;
            if (row_first + r < p.seq_q)
              *reinterpret_cast<uint4*>(obase + 2 * static_cast<long long>(row_first + r) * p.o_ss) = val[i];
          }
        }
        if (in_range && p.kv_splits <= 1) {
#pragma unroll
          for (int i = 0; i < F::kFinal; ++i) {
            if (p.final_out[i] != nullptr) {
              p.final_out[i][(static_cast<long long>(b) * p.heads + h) * p.seq_q + q_idx] = F::final_rowscale(i, rs, ctx);
            }
          }
        }
      }
    }
  }

  // a split whose share of the KV tiles is empty for a query tile contributes nothing
  if (p.kv_splits > 1 && warp < 4 * NT) {
    const int t = warp >> 2;
    const int q_idx = m0 + t * BM + (warp & 3) * 32 + lane;
    if (j_hi[t] <= j_lo[t] && q_idx < p.seq_q)
      p.part_final[((static_cast<long long>(b) * p.kv_splits + split) * p.heads + h) * p.seq_q + q_idx] = -INFINITY;
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // a wait was abandoned: give copies and MMAs still in flight time to land before the CTA's
    // shared and tensor memory are released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// Split-KV combine: o[b,q,h,:] = sum_i w_i part_o[b,i,h,q,:] with w_i = F::combine(i, splits, final row scales of
// all splits) -- the lowered OnlineFunc.combine of the reference (core/lower/lower_decode.py:287-302, combine kernel
// of attn_decode_tl.py:158-206).  For the built-in softmax that is exp(lse_i - lse), lse = log sum_i exp(lse_i), and
// the combined lse is written out as the call's final row scale.  One warp per (batch, head, query row).
template <class F, int DV, bool kBf16>
__global__ void __launch_bounds__(256) parallel_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_final,
                                                             long long part_final_stride, void* __restrict__ o,
                                                             float* __restrict__ final_out, int batch, int heads, int seq_q,
                                                             int splits, long long o_sb, long long o_ss, long long o_sh) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(batch) * heads * seq_q) return;
  const int q = static_cast<int>(row % seq_q);
  const int h = static_cast<int>((row / seq_q) % heads);
  const int b = static_cast<int>(row / (static_cast<long long>(seq_q) * heads));
  const long long split_stride = static_cast<long long>(heads) * seq_q;
  const long long prow0 = (static_cast<long long>(b) * splits * heads + h) * seq_q + q;   // split 0
  const float* fin = part_final + prow0;
  constexpr int E = DV / 32;   // columns per lane
  float acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  for (int i = 0; i < splits; ++i) {
    const float w = F::combine(i, splits, fin, split_stride, part_final_stride);
    if (w == 0.0f) continue;   // an empty split (its partial rows were never written)
    const float* src = part_o + (prow0 + i * split_stride) * DV + lane * E;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] += w * src[e];
  }
  uint8_t* orow = reinterpret_cast<uint8_t*>(o) + 2 * (b * o_sb + q * o_ss + h * o_sh + lane * E);
#pragma unroll
  for (int e = 0; e < E; e += 2) *reinterpret_cast<uint32_t*>(orow + 2 * e) = pack2<kBf16>(acc[e], acc[e + 1]);
  if constexpr (F::kCombinedFinal) {
    if (lane == 0 && final_out != nullptr)
      final_out[(static_cast<long long>(b) * heads + h) * seq_q + q] = F::combined_final(splits, fin, split_stride, part_final_stride);
  }
}

}  // namespace b200
