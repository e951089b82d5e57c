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
// Split kernel: one CTA per (half of dim_v, KV split, block of 128 heads, sequence).  The 128
// heads are the M dimension of the MMAs, so the latent KV is streamed once per CTA for all heads:
//   warp 4      TMA producer: Q (128 x dim_qk) once, then 32-row KV tiles into a 2-stage ring
//   warp 5      tcgen05.mma issuer: S = Q.KV^T (K = dim_qk) into a double-buffered TMEM tile,
//               O += P.V with P read from TMEM and V addressed inside the SAME shared-memory KV
//               tile (the K-major 64-column chunks of a KV tile are exactly the MN-major chunks
//               of V), so V is never loaded separately
//   warps 0-3   one head per thread: online softmax in the exp2 domain with lazy accumulator rescale
// The fp32 accumulator of 128 heads x 512 columns would fill all 512 TMEM columns and leave none
// for S, hence the split of dim_v over two CTAs (each recomputes S).
// Combine kernel: log-sum-exp weighted sum of the per-split fp32 partial outputs.
#include <algorithm>
#include <cstring>
#include <mutex>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "parallel_launch.cuh"  // tensor_map_encoder()
#include "sm100.cuh"

namespace b200 {

constexpr int kMlaHeads = 128;     // heads per CTA (MMA M)
constexpr int kMlaTileN = 32;      // KV rows per tile
constexpr int kMlaStages = 2;
constexpr int kMlaThreads = 192;

struct MlaParams {
  void* o;            // [B, H, DV] 16-bit, written when num_splits == 1
  float* lse;         // [B, H] or null
  float* part_o;      // [B, splits, H, DV] fp32 (num_splits > 1)
  float* part_lse;    // [B, splits, H]
  int batch, heads, seq_kv, num_splits, tiles_per_split;
  float scale_log2;   // scale * log2(e)
  float scale;
  int* status;
};

enum MlaWaitSite { kMlaQFull = 21, kMlaKvFull, kMlaKvEmpty, kMlaSFull, kMlaPReady, kMlaODone, kMlaOFinal };

template <int D, int DV>
struct MlaSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kQBytes = kMlaHeads * D * 2;
  static constexpr int kKvBytes = kMlaTileN * D * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKv = kQBytes;
  static constexpr int kOffBar = kOffKv + kMlaStages * kKvBytes;
  static constexpr int kNumBars = 1 + 2 * kMlaStages + 2 + 2 + 1;
  static constexpr int kOffMisc = kOffBar + 8 * kNumBars;
  static constexpr int kBytes = kOffMisc + 16 + 1024;
};

template <int D, int DV, bool kBf16>
__global__ void __launch_bounds__(kMlaThreads, 1)
mla_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmQr,
                 const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ CUtensorMap tmKVr, const MlaParams p) {
  using L = MlaSmem<D, DV>;
  constexpr int N = kMlaTileN, ST = kMlaStages, M = kMlaHeads;
  constexpr int DVH = DV / 2;                 // columns of the output handled by this CTA
  static_assert(D % 64 == 0 && DVH % 64 == 0 && DVH <= 256, "unsupported MLA dims");
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColO = 0, kColS = 256;  // O: [0, DVH), S buffers: 256 + 32*buf

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sKV = smem + L::kOffKv;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + ST;
  uint64_t* s_full = kv_empty + ST;  // [2]
  uint64_t* p_ready = s_full + 2;    // [2]
  uint64_t* o_done = p_ready + 2;    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortState ab{abort_flag, p.status};
  const int half = blockIdx.x & 1;
  const int split = blockIdx.x >> 1;
  const int hb = blockIdx.y;          // block of 128 heads
  const int b = blockIdx.z;
  const int head0 = hb * M;
  const int total_tiles = (p.seq_kv + N - 1) / N;
  const int tile_begin = split * p.tiles_per_split;
  const int n = max(0, min(total_tiles, tile_begin + p.tiles_per_split) - tile_begin);

  if (threadIdx.x == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
    }
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmQr);
    tma_prefetch_desc(&tmKV);
    tma_prefetch_desc(&tmKVr);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // =============== TMA producer ===============
    if (lane == 0 && n > 0 && !*abort_flag) {
      mbar_arrive_expect_tx(q_full, L::kQBytes);
      // the first DV columns come from the main map, the remaining (rope) columns from the second
      for (int c = 0; c < L::kChunks; ++c)
        tma_load_3d(sQ + c * (M * 128), c < DV / 64 ? &tmQ : &tmQr, q_full, c < DV / 64 ? c * 64 : c * 64 - DV, head0, b);
      for (int j = 0; j < n; ++j) {
        const int st = j % ST;
        if (!mbar_wait(&kv_empty[st], ((j / ST) & 1) ^ 1, ab, kMlaKvEmpty)) break;
        mbar_arrive_expect_tx(&kv_full[st], L::kKvBytes);
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_3d(sKV + st * L::kKvBytes + c * (N * 128), c < DV / 64 ? &tmKV : &tmKVr, &kv_full[st],
                      c < DV / 64 ? c * 64 : c * 64 - DV, (tile_begin + j) * N, b);
      }
    }
  } else if (warp == 5) {
    // =============== MMA issuer ===============
    if (lane == 0 && n > 0 && !*abort_flag) {
      constexpr uint32_t idesc_qk = make_idesc_f16(M, N, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(M, DVH, kBf16, false, true);
      const uint32_t q_addr = smem_u32(sQ), kv_addr = smem_u32(sKV);
      auto issue_qk = [&](int st, int buf) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t adesc = make_smem_desc(q_addr + (ks >> 2) * (M * 128) + (ks & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(kv_addr + st * L::kKvBytes + (ks >> 2) * (N * 128) + (ks & 3) * 32, 16, 1024);
          umma_ss(tmem_base + kColS + buf * N, adesc, bdesc, idesc_qk, ks > 0);
        }
        umma_commit(&s_full[buf]);
      };
      auto issue_pv = [&](int st, int buf, bool first) {
        // V half: chunks [half*DVH/64, ...) of the KV tile, MN-major: 64-column chunks N*128 bytes apart
        const uint32_t v_addr = kv_addr + st * L::kKvBytes + half * (DVH / 64) * (N * 128);
#pragma unroll
        for (int ks = 0; ks < N / 16; ++ks) {
          const uint64_t bdesc = make_smem_desc(v_addr + ks * 2048, N * 128, 1024);
          umma_ts(tmem_base + kColO, tmem_base + kColS + buf * N + ks * 8, bdesc, idesc_pv, (!first || ks > 0) ? 1u : 0u);
        }
        umma_commit(o_done);
        umma_commit(&kv_empty[st]);
      };
      bool ok = mbar_wait(q_full, 0, ab, kMlaQFull) && mbar_wait(&kv_full[0], 0, ab, kMlaKvFull);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0, 0);
        for (int j = 0; j < n && ok; ++j) {
          if (j + 1 < n) {
            const int stn = (j + 1) % ST;
            ok = mbar_wait(&kv_full[stn], ((j + 1) / ST) & 1, ab, kMlaKvFull);
            if (!ok) break;
            tc_fence_after_sync();
            issue_qk(stn, (j + 1) & 1);
          }
          ok = mbar_wait(&p_ready[j & 1], (j >> 1) & 1, ab, kMlaPReady);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(j % ST, j & 1, j == 0);
        }
      }
    }
  } else {
    // =============== softmax: one head per thread ===============
    const int row = warp * 32 + lane;
    const int head = head0 + row;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + kColO;
    float m_ref = -1.0e30f, r_sum = 0.0f;
    const float c2 = p.scale_log2;
    bool ok = (n > 0) && !*abort_flag;
    for (int j = 0; j < n && ok; ++j) {
      const int buf = j & 1;
      const uint32_t tS = tmem_base + lane_base + kColS + buf * N;
      ok = mbar_wait(&s_full[buf], (j >> 1) & 1, ab, kMlaSFull);
      if (!ok) break;
      tc_fence_after_sync();
      float s[N];
      tmem_ld32f(tS, s);
      tmem_wait_ld();
      const int kv0 = (tile_begin + j) * N;
      if (kv0 + N > p.seq_kv) {
#pragma unroll
        for (int i = 0; i < N; ++i) s[i] = (kv0 + i < p.seq_kv) ? s[i] : -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < N; ++i) mx = fmaxf(mx, s[i]);
      float o_scale = 1.0f;
      if ((mx - m_ref) * c2 > 8.0f) {
        o_scale = fast_exp2((m_ref - mx) * c2);
        m_ref = mx;
        r_sum *= o_scale;
      }
      const float neg = -m_ref * c2;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        s[i] = fast_exp2(fmaf(s[i], c2, neg));
        s[i + 1] = fast_exp2(fmaf(s[i + 1], c2, neg));
        a0 += s[i];
        a1 += s[i + 1];
      }
      r_sum += a0 + a1;
      uint32_t pk[N / 2];
#pragma unroll
      for (int i = 0; i < N / 2; ++i) pk[i] = pack2<kBf16>(s[2 * i], s[2 * i + 1]);
      tmem_st16(tS, pk);
      if (j > 0 && __any_sync(0xffffffffu, o_scale != 1.0f)) {
        // every MMA that accumulates into O has been committed to o_done: phase j-1 must be complete
        ok = mbar_wait(o_done, (j - 1) & 1, ab, kMlaODone);
        if (ok) {
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < DVH / 32; ++c) {
            float o[32];
            tmem_ld32f(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= o_scale;
            tmem_st32f(tO + c * 32, o);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[buf]);
    }
    if (ok && n > 0) {
      ok = mbar_wait(o_done, (n - 1) & 1, ab, kMlaOFinal);
      if (ok) {
        tc_fence_after_sync();
        const bool in_range = head < p.heads;
        const float inv = 1.0f / r_sum;
        const float lse = logf(r_sum) + m_ref * p.scale;
        if (p.num_splits == 1) {
          uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) + 2 * ((static_cast<long long>(b) * p.heads + head) * DV + half * DVH);
#pragma unroll
          for (int c = 0; c < DVH / 32; ++c) {
            float o[32];
            tmem_ld32f(tO + c * 32, o);
            tmem_wait_ld();
            if (in_range) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 pk;
                pk.x = pack2<kBf16>(o[8 * v + 0] * inv, o[8 * v + 1] * inv);
                pk.y = pack2<kBf16>(o[8 * v + 2] * inv, o[8 * v + 3] * inv);
                pk.z = pack2<kBf16>(o[8 * v + 4] * inv, o[8 * v + 5] * inv);
                pk.w = pack2<kBf16>(o[8 * v + 6] * inv, o[8 * v + 7] * inv);
                *reinterpret_cast<uint4*>(orow + c * 64 + v * 16) = pk;
              }
            }
          }
          if (in_range && half == 0 && p.lse != nullptr) p.lse[static_cast<long long>(b) * p.heads + head] = lse;
        } else {
          float* prow = p.part_o + ((static_cast<long long>(b) * p.num_splits + split) * p.heads + head) * DV + half * DVH;
#pragma unroll
          for (int c = 0; c < DVH / 32; ++c) {
            float o[32];
            tmem_ld32f(tO + c * 32, o);
            tmem_wait_ld();
            if (in_range) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 f = make_float4(o[4 * v] * inv, o[4 * v + 1] * inv, o[4 * v + 2] * inv, o[4 * v + 3] * inv);
                *reinterpret_cast<float4*>(prow + c * 32 + v * 4) = f;
              }
            }
          }
          if (in_range && half == 0) p.part_lse[(static_cast<long long>(b) * p.num_splits + split) * p.heads + head] = lse;
        }
      }
    } else if (n == 0 && p.num_splits > 1 && head < p.heads && half == 0) {
      // a split with no KV rows contributes nothing
      p.part_lse[(static_cast<long long>(b) * p.num_splits + split) * p.heads + head] = -INFINITY;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// o[b,h,:] = sum_i exp(lse_i - lse) * part_o[b,i,h,:],  lse = log sum_i exp(lse_i).
// One warp per (b, h); each lane owns DV/32 columns spread in float4 groups.
template <int DV, bool kBf16>
__global__ void __launch_bounds__(256) mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                                        void* __restrict__ o, float* __restrict__ lse_out, int batch,
                                                        int heads, int num_splits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= batch * heads) return;
  const int b = warp / heads, h = warp % heads;
  float mx = -INFINITY;
  for (int i = 0; i < num_splits; ++i) mx = fmaxf(mx, part_lse[(static_cast<long long>(b) * num_splits + i) * heads + h]);
  float den = 0.f;
  for (int i = 0; i < num_splits; ++i) den += __expf(part_lse[(static_cast<long long>(b) * num_splits + i) * heads + h] - mx);
  const float lse = mx + __logf(den);
  constexpr int V4 = DV / 128;  // float4 groups per lane
  float4 acc[V4];
#pragma unroll
  for (int v = 0; v < V4; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < num_splits; ++i) {
    const long long row = (static_cast<long long>(b) * num_splits + i) * heads + h;
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
  using L = MlaSmem<D, DV>;
  const AttnB200MlaShape& s = a->shape;
  CUtensorMap tmQ, tmQr, tmKV, tmKVr;
  const int esz = 2;
  // rope columns: a separate tensor, or columns [DV, D) of the fused rows
  const void* q_rope = a->q_rope != nullptr ? a->q_rope : static_cast<const uint8_t*>(a->q) + DV * esz;
  const void* kv_rope = a->kv_rope != nullptr ? a->kv_rope : static_cast<const uint8_t*>(a->kv) + DV * esz;
  const int64_t* qr_st = a->q_rope != nullptr ? a->q_rope_stride : a->q_stride;
  const int64_t* kr_st = a->kv_rope != nullptr ? a->kv_rope_stride : a->kv_stride;
  int rc = encode_3d(&tmQ, a->q, a->dtype, DV, s.heads_q, s.batch, a->q_stride[0], a->q_stride[1], kMlaHeads);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmQr, q_rope, a->dtype, D - DV, s.heads_q, s.batch, qr_st[0], qr_st[1], kMlaHeads);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmKV, a->kv, a->dtype, DV, s.seq_kv, s.batch, a->kv_stride[0], a->kv_stride[1], kMlaTileN);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_3d(&tmKVr, kv_rope, a->dtype, D - DV, s.seq_kv, s.batch, kr_st[0], kr_st[1], kMlaTileN);
  if (rc != ATTN_B200_OK) return rc;
  MlaParams p;
  std::memset(&p, 0, sizeof(p));
  const int total_tiles = (s.seq_kv + kMlaTileN - 1) / kMlaTileN;
  p.o = a->o;
  p.lse = a->lse;
  p.batch = s.batch;
  p.heads = s.heads_q;
  p.seq_kv = s.seq_kv;
  p.num_splits = a->num_splits;
  p.tiles_per_split = (total_tiles + a->num_splits - 1) / a->num_splits;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.status = status;
  if (a->num_splits > 1) {
    p.part_o = static_cast<float*>(a->workspace);
    p.part_lse = p.part_o + static_cast<long long>(s.batch) * a->num_splits * s.heads_q * DV;
  }
  auto kernel = mla_split_kernel<D, DV, kBf16>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  dim3 grid(2 * a->num_splits, (s.heads_q + kMlaHeads - 1) / kMlaHeads, s.batch);
  kernel<<<grid, kMlaThreads, L::kBytes, stream>>>(tmQ, tmQr, tmKV, tmKVr, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  if (a->num_splits > 1) {
    const long long warps = static_cast<long long>(s.batch) * s.heads_q;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    mla_combine_kernel<DV, kBf16><<<blocks, 256, 0, stream>>>(p.part_o, p.part_lse, a->o, a->lse, s.batch, s.heads_q, a->num_splits);
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
  // CTAs per split level: 2 (halves of dim_v) x head blocks x sequences, one CTA per SM at a time.
  // Pick the split count that fills whole waves best; every split must keep at least 8 KV tiles
  // (each CTA re-reads Q, and the combine pass costs one more sweep over the partial outputs).
  const long long base = 2LL * ((shape->heads_q + b200::kMlaHeads - 1) / b200::kMlaHeads) * shape->batch;
  const int total_tiles = (shape->seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  int best = 1;
  double best_score = -1.0;
  for (int s = 1; s <= 64; ++s) {
    const int tiles = (total_tiles + s - 1) / s;
    if (s > 1 && tiles < 8) break;
    if ((s - 1) * tiles >= total_tiles) continue;  // last split would be empty
    const long long ctas = base * s;
    const long long waves = (ctas + sm_count - 1) / sm_count;
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * sm_count);
    const double score = fill - 0.004 * (s - 1);
    if (score > best_score + 1e-9) {
      best_score = score;
      best = s;
    }
  }
  *num_splits_out = best;
  return ATTN_B200_OK;
}

int64_t attn_b200_mla_workspace_bytes(const AttnB200MlaShape* shape, int32_t num_splits) {
  if (b200::validate_mla_shape(shape) != ATTN_B200_OK || num_splits < 1) return -1;
  if (num_splits == 1) return 0;
  const int64_t rows = static_cast<int64_t>(shape->batch) * num_splits * shape->heads_q;
  return rows * shape->dim_v * 4 + rows * 4;
}

int attn_b200_mla_decode(const AttnB200MlaArgs* a, void* cuda_stream) {
  if (a == nullptr || a->q == nullptr || a->kv == nullptr || a->o == nullptr) return ATTN_B200_E_INVALID_ARG;
  int rc = b200::validate_mla_shape(&a->shape);
  if (rc != ATTN_B200_OK) return rc;
  if (a->dtype != ATTN_B200_DTYPE_FP16 && a->dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a->num_splits < 1 || a->num_splits > 32767) return ATTN_B200_E_INVALID_ARG;
  const int total_tiles = (a->shape.seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  if (a->num_splits > total_tiles) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  const int64_t need = attn_b200_mla_workspace_bytes(&a->shape, a->num_splits);
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
  if (a->num_splits < 1 || a->num_splits > 32767) return ATTN_B200_E_INVALID_ARG;
  const int total_tiles = (a->shape.seq_kv + b200::kMlaTileN - 1) / b200::kMlaTileN;
  if (a->num_splits > total_tiles) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0 || (reinterpret_cast<uintptr_t>(status_word) & 3) != 0)
    return ATTN_B200_E_UNSUPPORTED;
  const int64_t need = attn_b200_mla_workspace_bytes(&a->shape, a->num_splits);
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
