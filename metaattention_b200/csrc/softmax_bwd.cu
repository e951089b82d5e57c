// Backward of softmax attention for sm_100a (head dims 128 / 128 or 64 / 64, 16-bit inputs, fp32 accumulation).
//
//   P  = exp(scale * Q K^T - lse)            (recomputed from the forward's log-sum-exp, masked like the forward)
//   dV = P^T dO
//   dP = dO V^T,   delta_i = sum_d dO_id O_id,   dS = P o (dP - delta) * scale
//   dK = dS^T Q,   dQ = dS K
//
// the algorithm of the reference's generated backward (attention_engine/core/template/tl_template/attn/attn_tl.py:
// preprocess :212-244 = delta, main kernel :309-503 = dK/dV per KV tile with atomic adds into an fp32 dQ, postprocess
// :246-275 = dQ to 16 bits; autograd wrapper :669-694), for the built-in softmax.  Differences: three launches
// without atomics or an fp32 dQ buffer -- (1) delta and log2-domain lse into a padded scratch, (2) one CTA per KV tile
// accumulating dK and dV over the query tiles, (3) one CTA per query tile accumulating dQ over the KV tiles (S and dP
// are computed a second time there: 7 tile products instead of 5 for no read-modify-write traffic on dQ).
//
// Both main launches are one kernel template (attn_bwd.cuh, shared with the lowered functors).  A CTA keeps one 128-row tile pair resident (X: K_j, V_j or Q_i, dO_i)
// and streams the other (Y: Q_i, dO_i or K_j, V_j) through a two-stage TMA ring.  Per streamed tile:
//   S  = X1 Y1^T, dP = X2 Y2^T           tcgen05 SS, fp32 in tensor memory (columns [0,128) and [128,256))
//   row threads (thread = TMEM lane x column half): P and dS as 16-bit pairs written over S and dP
//   acc1 += P  Y2   (dV; KV role only)    tcgen05 TS, A from tensor memory, B = the streamed tile MN-major
//   acc2 += dS Y1   (dK or dQ)
// With the KV role the lanes are KV rows and the columns query rows (S^T, dP^T), so that P^T and dS^T are the A
// operands as they stand; the statistics (lse, delta) then belong to columns and come with the streamed tile.
#include "attn_bwd.cuh"

namespace b200 {

// The built-in softmax: P = exp2(s * scale * log2e - lse2), dS = P (dP - delta) * scale; the scale is left to the
// finished dK and dQ rows.
struct SoftmaxBwdFunctor {
  static constexpr bool kUsesStats = true;
  static constexpr bool kNegInfMask = true;
  struct Ctx {
    float c2, scale;
  };
  __device__ static Ctx make(const BwdParams& p) { return Ctx{p.scale * 1.4426950408889634f, p.scale}; }
  __device__ static void score(float s, float lse2, const Ctx& c, int, int, int, int, float& p_out, float& g_out) {
    p_out = g_out = fast_exp2(fmaf(s, c.c2, -lse2));
  }
  __device__ static float grad(float g, float dp, float delta, const Ctx&) { return g * (dp - delta); }
  __device__ static float out_scale(const Ctx& c) { return c.scale; }
};

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d] and lse2 = lse * log2(e), both padded to whole tiles (delta 0,
// lse2 +inf past the end).  One warp per (b, h, s); attn_tl.py:212-244 of the reference computes the same delta.
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd_prepare_kernel(const void* __restrict__ o, const void* __restrict__ d_o,
                                                        const float* __restrict__ lse, float* __restrict__ delta,
                                                        float* __restrict__ lse2, int batch, int heads, int seq_q,
                                                        int seq_q_pad, int dim_v, long long o_sb, long long o_ss,
                                                        long long o_sh, long long do_sb, long long do_ss, long long do_sh) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(batch) * heads * seq_q_pad) return;
  const int s = static_cast<int>(w % seq_q_pad);
  const int h = static_cast<int>((w / seq_q_pad) % heads);
  const int b = static_cast<int>(w / (static_cast<long long>(seq_q_pad) * heads));
  float acc = 0.0f;
  if (s < seq_q) {
    const uint32_t* po = reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(o) + b * o_sb + s * o_ss + h * o_sh);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(d_o) + b * do_sb + s * do_ss + h * do_sh);
    for (int i = lane; i < dim_v / 2; i += 32) {
      uint32_t a = po[i], c = pd[i];
      float a0, a1, c0, c1;
      if constexpr (kBf16) {
        const __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&a), y = *reinterpret_cast<__nv_bfloat162*>(&c);
        a0 = __bfloat162float(x.x); a1 = __bfloat162float(x.y); c0 = __bfloat162float(y.x); c1 = __bfloat162float(y.y);
      } else {
        const __half2 x = *reinterpret_cast<__half2*>(&a), y = *reinterpret_cast<__half2*>(&c);
        a0 = __half2float(x.x); a1 = __half2float(x.y); c0 = __half2float(y.x); c1 = __half2float(y.y);
      }
      acc = fmaf(a0, c0, fmaf(a1, c1, acc));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  }
  if (lane == 0) {
    const long long idx = (static_cast<long long>(b) * heads + h) * seq_q_pad + s;
    delta[idx] = acc;
    // rows past the end, and rows whose mask kept nothing (lse = -inf), get P = 0 everywhere
    const float l = s < seq_q ? lse[(static_cast<long long>(b) * heads + h) * seq_q + s] : INFINITY;
    lse2[idx] = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
  }
}

template <bool kBf16, int D>
int launch_softmax_bwd(const AttnB200SoftmaxBwdArgs* a, const BwdCall& call_in, cudaStream_t stream, int* status) {
  const int T = kBwdT;
  const int seq_q_pad = (a->seq_q + T - 1) / T * T;
  const long long rows = static_cast<long long>(a->batch) * a->heads * seq_q_pad;
  float* delta = static_cast<float*>(a->workspace);
  float* lse2 = delta + rows;
  {
    const long long threads = rows * 32;
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    bwd_prepare_kernel<kBf16><<<blocks, 256, 0, stream>>>(a->o, a->d_o, a->lse, delta, lse2, a->batch, a->heads, a->seq_q, seq_q_pad,
                                                         a->dim_v, a->o_stride[0], a->o_stride[1], a->o_stride[2], a->do_stride[0],
                                                         a->do_stride[1], a->do_stride[2]);
    if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  }
  BwdCall call = call_in;
  call.lse2 = lse2;
  call.delta = delta;
  return launch_attn_bwd<SoftmaxBwdFunctor, kBf16, D>(call, stream, status);
}

}  // namespace b200

extern "C" {

int64_t attn_b200_softmax_bwd_workspace_bytes(const AttnB200SoftmaxBwdArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->seq_q <= 0) return -1;
  const int64_t seq_q_pad = (static_cast<int64_t>(a->seq_q) + b200::kBwdT - 1) / b200::kBwdT * b200::kBwdT;
  return 2 * static_cast<int64_t>(a->batch) * a->heads * seq_q_pad * 4;
}

int attn_b200_softmax_bwd(const AttnB200SoftmaxBwdArgs* a, void* cuda_stream) {
  if (a == nullptr || a->o == nullptr || a->lse == nullptr) return ATTN_B200_E_INVALID_ARG;
  if (a->dim_qk != a->dim_v) return ATTN_B200_E_UNSUPPORTED;
  b200::BwdCall call{};
  if (!b200::bwd_mask_of(a->mask_kind, a->mask_left, a->mask_right, a->mask_bits_q, a->mask_bits_kv, a->mask_tiles_q, a->mask_tiles_kv, call)) return ATTN_B200_E_UNSUPPORTED;
  call.q = a->q; call.k = a->k; call.v = a->v; call.d_o = a->d_o;
  call.dq = a->dq; call.dk = a->dk; call.dv = a->dv;
  call.batch = a->batch; call.heads = a->heads; call.heads_kv = a->heads_kv > 0 ? a->heads_kv : a->heads;
  call.seq_q = a->seq_q; call.seq_kv = a->seq_kv; call.dim = a->dim_qk; call.dtype = a->dtype;
  call.scale = a->scale;
  call.q_stride = a->q_stride; call.k_stride = a->k_stride; call.v_stride = a->v_stride; call.do_stride = a->do_stride;
  call.dq_stride = a->dq_stride; call.dk_stride = a->dk_stride; call.dv_stride = a->dv_stride;
  const int rc = b200::validate_bwd_call(call);
  if (rc != ATTN_B200_OK) return rc;
  for (int d = 0; d < 3; ++d)
    if (a->o_stride[d] % 2 != 0 || a->do_stride[d] % 2 != 0) return ATTN_B200_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->o) & 3) != 0 || (reinterpret_cast<uintptr_t>(a->d_o) & 3) != 0) return ATTN_B200_E_UNSUPPORTED;
  const int64_t need = attn_b200_softmax_bwd_workspace_bytes(a);
  if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0)
    return ATTN_B200_E_WORKSPACE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ATTN_B200_E_LAUNCH;
  int* status = b200::device_status_word(dev);
  if (status == nullptr) return ATTN_B200_E_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const bool bf16 = a->dtype == ATTN_B200_DTYPE_BF16;
  if (a->dim_qk == 64)
    return bf16 ? b200::launch_softmax_bwd<true, 64>(a, call, stream, status) : b200::launch_softmax_bwd<false, 64>(a, call, stream, status);
  return bf16 ? b200::launch_softmax_bwd<true, 128>(a, call, stream, status) : b200::launch_softmax_bwd<false, 128>(a, call, stream, status);
}

}  // extern "C"
