// Row gathers around the linear-attention backward (sm_100a): the backward runs the forward kernel on time-reversed
// operands and on column ranges of dim_v, and adds up fp32 partial results.  torch does each of these as a pass of its
// own (flip, slice + contiguous, add, cast: ~0.2 ms apiece at the benchmark shape); here a reversed and / or
// column-sliced copy is one pass, and sum + cast + reversal of the partial results another.
//   rows_copy16:    dst[o][s'][0:width] = src[o][s][col0:col0+width],  s' = reverse ? seq-1-s : s   (16-bit elements)
//   rows_sum_cast:  dst16[o][s'][:]     = a[o][s][:] (+ b[o][s][:])                                 (fp32 -> fp16 / bf16)
// The reference needs neither: its backward kernels walk the sequence backwards themselves
// (core/template/tl_template/linear/linear_tl.py:461-975).
#include <cstdint>

#include "../../include/attn_b200.h"
#include "sm100.cuh"

namespace b200 {

__global__ void __launch_bounds__(256) rows_copy16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, long long rows,
                                                         int seq, int src_cols, int col0, int width, int reverse) {
  const int vpr = width / 8;   // 16-byte vectors per row
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int v = static_cast<int>(i - r * vpr);
    const long long o = r / seq;
    const int s = static_cast<int>(r - o * seq);
    const long long rd = o * seq + (reverse ? seq - 1 - s : s);
    const uint4 x = *reinterpret_cast<const uint4*>(src + r * src_cols + col0 + v * 8);
    *reinterpret_cast<uint4*>(dst + rd * width + v * 8) = x;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) rows_sum_cast_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                           uint16_t* __restrict__ dst, long long rows, int seq, int cols, int reverse) {
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int v = static_cast<int>(i - r * vpr);
    const long long o = r / seq;
    const int s = static_cast<int>(r - o * seq);
    const long long rd = o * seq + (reverse ? seq - 1 - s : s);
    const float4* pa = reinterpret_cast<const float4*>(a + r * cols + v * 8);
    float4 x0 = pa[0], x1 = pa[1];
    if (b != nullptr) {
      const float4* pb = reinterpret_cast<const float4*>(b + r * cols + v * 8);
      const float4 y0 = pb[0], y1 = pb[1];
      x0.x += y0.x; x0.y += y0.y; x0.z += y0.z; x0.w += y0.w;
      x1.x += y1.x; x1.y += y1.y; x1.z += y1.z; x1.w += y1.w;
    }
    uint4 pk;
    pk.x = pack2<kBf16>(x0.x, x0.y);
    pk.y = pack2<kBf16>(x0.z, x0.w);
    pk.z = pack2<kBf16>(x1.x, x1.y);
    pk.w = pack2<kBf16>(x1.z, x1.w);
    *reinterpret_cast<uint4*>(dst + rd * cols + v * 8) = pk;
  }
}

inline unsigned row_ops_grid(long long total_vectors) {
  const long long blocks = (total_vectors + 255) / 256;
  const long long cap = 148LL * 16;   // a multiple of the SM count; the loops stride over the rest
  return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace b200

extern "C" {

int attn_b200_rows_copy16(const void* src, void* dst, int64_t outer, int32_t seq, int32_t src_cols, int32_t col0, int32_t width,
                          int32_t reverse, void* cuda_stream) {
  if (src == nullptr || dst == nullptr || outer <= 0 || seq <= 0 || width <= 0) return ATTN_B200_E_INVALID_ARG;
  if (col0 < 0 || col0 + width > src_cols) return ATTN_B200_E_INVALID_ARG;
  if (width % 8 != 0 || col0 % 8 != 0 || src_cols % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  const long long rows = static_cast<long long>(outer) * seq;
  b200::rows_copy16_kernel<<<b200::row_ops_grid(rows * (width / 8)), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), rows, seq, src_cols, col0, width, reverse);
  return cudaGetLastError() == cudaSuccess ? ATTN_B200_OK : ATTN_B200_E_LAUNCH;
}

int attn_b200_rows_sum_cast(const float* a, const float* b, void* dst, int32_t dtype, int64_t outer, int32_t seq, int32_t cols,
                            int32_t reverse, void* cuda_stream) {
  if (a == nullptr || dst == nullptr || outer <= 0 || seq <= 0 || cols <= 0) return ATTN_B200_E_INVALID_ARG;
  if (dtype != ATTN_B200_DTYPE_FP16 && dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (cols % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(dst)) & 15) != 0)
    return ATTN_B200_E_UNSUPPORTED;
  const long long rows = static_cast<long long>(outer) * seq;
  const unsigned grid = b200::row_ops_grid(rows * (cols / 8));
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (dtype == ATTN_B200_DTYPE_BF16)
    b200::rows_sum_cast_kernel<true><<<grid, 256, 0, stream>>>(a, b, static_cast<uint16_t*>(dst), rows, seq, cols, reverse);
  else
    b200::rows_sum_cast_kernel<false><<<grid, 256, 0, stream>>>(a, b, static_cast<uint16_t*>(dst), rows, seq, cols, reverse);
  return cudaGetLastError() == cudaSuccess ? ATTN_B200_OK : ATTN_B200_E_LAUNCH;
}

}  // extern "C"
