// Host side of kernel family (1): argument validation, tensor-map encoding
// and launch.  Header-only so that functor libraries compiled at run time
// instantiate the same launcher as the built-in functors.
#pragma once

#include <algorithm>
#include <cstring>

#include "../../include/attn_b200.h"
#include "parallel_fwd.cuh"

namespace b200 {

typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);

inline TensorMapEncodeTiledFn tensor_map_encoder() {
  static TensorMapEncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<TensorMapEncodeTiledFn>(p);
  }();
  // The encoder is a driver entry point and wants a current context on the calling thread.  The runtime binds the
  // current device's primary context to a thread only at its first call that needs one, so a thread that has made
  // none yet (an autograd worker running a backward pass, with every per-device object of this library already
  // cached) would get CUDA_ERROR_INVALID_CONTEXT: setting the device it already has binds the context.
  thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) bound = true;
  }
  return fn;
}

// Tensor map over a 16-bit tensor addressed as [batch][seq][head][dim] through
// element strides (dim contiguous).  Dimension 0 of the map is `dim`; the
// other three are ordered by increasing stride, and `order` tells the kernel
// where each coordinate goes.  Box: 64 elements (128 bytes, the swizzle span)
// of one head and one batch entry by `box_rows` sequence positions.
inline int encode_rows_map(CUtensorMap* tm, CoordOrder* order, const void* base, int dtype, int dim, int batch,
                           int seq, int heads, const int64_t stride_bsh[3], int box_rows) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return ATTN_B200_E_LAUNCH;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  struct Dim { int which; uint64_t size; int64_t stride; };  // which: 0 batch, 1 seq, 2 head
  Dim dims[3] = {{0, (uint64_t)batch, stride_bsh[0]}, {1, (uint64_t)seq, stride_bsh[1]}, {2, (uint64_t)heads, stride_bsh[2]}};
  for (auto& d : dims) {
    if (d.size > 1 && (d.stride <= 0 || (d.stride % 8) != 0)) return ATTN_B200_E_UNSUPPORTED;
  }
  // extent-1 dimensions carry no addressing information: move them last
  std::stable_sort(dims, dims + 3, [](const Dim& a, const Dim& b) {
    const bool a1 = a.size <= 1, b1 = b.size <= 1;
    if (a1 != b1) return b1;
    if (a1 && b1) return false;
    return a.stride < b.stride;
  });
  int64_t next = dim;
  for (auto& d : dims) {
    if (d.size <= 1) d.stride = next;
    next = std::max<int64_t>(next, d.stride * (int64_t)d.size);
  }
  cuuint64_t gdim[4] = {(cuuint64_t)dim, dims[0].size, dims[1].size, dims[2].size};
  cuuint64_t gstride[3] = {(cuuint64_t)dims[0].stride * 2, (cuuint64_t)dims[1].stride * 2, (cuuint64_t)dims[2].stride * 2};
  cuuint32_t box[4] = {64, 1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  int pos[3] = {0, 0, 0};
  for (int i = 0; i < 3; ++i) {
    pos[dims[i].which] = i + 1;
    if (dims[i].which == 1) box[i + 1] = (cuuint32_t)box_rows;
  }
  order->pos_b = pos[0];
  order->pos_s = pos[1];
  order->pos_h = pos[2];
  const CUtensorMapDataType dt = dtype == ATTN_B200_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(tm, dt, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ATTN_B200_OK : ATTN_B200_E_UNSUPPORTED;
}

inline int validate_parallel_args(const AttnB200ParallelArgs* a) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr) return ATTN_B200_E_INVALID_ARG;
  if (a->batch <= 0 || a->heads <= 0 || a->seq_q <= 0 || a->seq_kv <= 0) return ATTN_B200_E_INVALID_ARG;
  if (a->dtype != ATTN_B200_DTYPE_FP16 && a->dtype != ATTN_B200_DTYPE_BF16) return ATTN_B200_E_INVALID_ARG;
  if (a->mask_kind != ATTN_B200_MASK_NONE && a->mask_kind != ATTN_B200_MASK_CAUSAL && a->mask_kind != ATTN_B200_MASK_BAND)
    return ATTN_B200_E_INVALID_ARG;
  if (a->mask_kind == ATTN_B200_MASK_BAND && (a->mask_left < 0 || a->mask_right < 0)) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  for (int i = 0; i < 3; ++i)
    if (a->o_stride[i] % 8 != 0) return ATTN_B200_E_UNSUPPORTED;
  if (a->heads > 65535 || a->batch > 65535) return ATTN_B200_E_UNSUPPORTED;
  if (a->heads_kv < 0 || (a->heads_kv > 0 && a->heads % a->heads_kv != 0)) return ATTN_B200_E_INVALID_ARG;
  if (a->tile_keep != nullptr) {
    // block sparsity: the bitmaps replace the mask kinds, and the walk is not combined with split-KV
    if (a->tile_partial == nullptr || a->mask_kind != ATTN_B200_MASK_NONE || a->num_splits > 1) return ATTN_B200_E_INVALID_ARG;
    if (a->sparse_batch != 1 && a->sparse_batch != a->batch) return ATTN_B200_E_INVALID_ARG;
    const int hkv = a->heads_kv > 0 ? a->heads_kv : a->heads;
    if (a->sparse_heads != 1 && a->sparse_heads != a->heads && a->sparse_heads != hkv) return ATTN_B200_E_INVALID_ARG;
    if (a->elem_mask_rows != 0 && a->elem_mask_rows != 128) return ATTN_B200_E_INVALID_ARG;
    if (a->elem_mask_rows == 128 && a->elem_mask != nullptr && a->tile_mask_base == nullptr) return ATTN_B200_E_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(a->elem_mask) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
    if ((a->seq_kv + 127) / 128 > 32 * kMaxTileWords) return ATTN_B200_E_UNSUPPORTED;
  }
  return ATTN_B200_OK;
}

// `dv0` selects a DV-column slice of v and o when dim_v is wider than the kernel's DV (see launch_parallel_sliced)
template <class F, int D, int DV, bool kBf16, int NT = 2, bool kSparse = false>
int launch_parallel(const AttnB200ParallelArgs* a, cudaStream_t stream, int* device_status, int dv0 = -1) {
  using L = ParallelSmem<D, DV, NT>;
  if ((a->tile_keep != nullptr) != kSparse) return ATTN_B200_E_UNSUPPORTED;   // this library was not built for that walk
  if (a->dim_qk != D || (dv0 < 0 ? a->dim_v != DV : (a->dim_v % DV != 0 || dv0 + DV > a->dim_v))) return ATTN_B200_E_UNSUPPORTED;
  const void* v_base = dv0 > 0 ? static_cast<const uint8_t*>(a->v) + 2 * dv0 : a->v;
  void* o_base = dv0 > 0 ? static_cast<uint8_t*>(a->o) + 2 * dv0 : a->o;
  if (device_status == nullptr) return ATTN_B200_E_INVALID_ARG;
  CUtensorMap tmQ, tmK, tmV;
  ParallelParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = encode_rows_map(&tmQ, &p.oq, a->q, a->dtype, D, a->batch, a->seq_q, a->heads, a->q_stride, L::kBM);
  if (rc != ATTN_B200_OK) return rc;
  const int heads_kv = a->heads_kv > 0 ? a->heads_kv : a->heads;
  rc = encode_rows_map(&tmK, &p.ok, a->k, a->dtype, D, a->batch, a->seq_kv, heads_kv, a->k_stride, L::kBN);
  if (rc != ATTN_B200_OK) return rc;
  rc = encode_rows_map(&tmV, &p.ov, v_base, a->dtype, DV, a->batch, a->seq_kv, heads_kv, a->v_stride, L::kBN);
  if (rc != ATTN_B200_OK) return rc;
  p.o = o_base;
  for (int i = 0; i < kMaxRowScales; ++i) p.final_out[i] = dv0 > 0 ? nullptr : a->final_rowscales[i];   // the first slice writes them
  p.batch = a->batch;
  p.heads = a->heads;
  p.kv_group = a->heads / heads_kv;
  p.seq_q = a->seq_q;
  p.seq_kv = a->seq_kv;
  p.o_sb = a->o_stride[0];
  p.o_ss = a->o_stride[1];
  p.o_sh = a->o_stride[2];
  p.mask_kind = a->mask_kind;
  p.win_left = a->mask_left > kNoBound ? kNoBound : a->mask_left;
  p.win_right = a->mask_right > kNoBound ? kNoBound : a->mask_right;
  p.status = device_status;
  for (int i = 0; i < 8; ++i) p.fa.f[i] = a->fparams[i];
  for (int i = 0; i < kMaxCustom; ++i) {
    p.fa.custom[i] = a->custom[i];
    for (int j = 0; j < 4; ++j) p.fa.cstride[i][j] = a->custom_stride[i][j];
  }
  const int splits = a->num_splits > 1 ? a->num_splits : 1;
  if (splits > 1) {
    const int n_kv_tiles = (a->seq_kv + L::kBN - 1) / L::kBN;
    if (splits > n_kv_tiles || static_cast<long long>(a->batch) * splits > 65535) return ATTN_B200_E_INVALID_ARG;
    const long long rows = static_cast<long long>(a->batch) * splits * a->heads * a->seq_q;
    const int n_final = F::kFinal > 0 ? F::kFinal : 1;
    const long long need = rows * (DV + n_final) * 4;
    if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0)
      return ATTN_B200_E_WORKSPACE;
    p.kv_splits = splits;
    p.tiles_per_split = (n_kv_tiles + splits - 1) / splits;
    // a functor other than the built-in softmax has no neutral value for a split without KV tiles: every split
    // must get some, which holds without a mask when the last split is not empty
    if (!F::kCombinedFinal && (a->mask_kind != ATTN_B200_MASK_NONE || (splits - 1) * p.tiles_per_split >= n_kv_tiles))
      return ATTN_B200_E_UNSUPPORTED;
    p.part_o = static_cast<float*>(a->workspace);
    p.part_final = p.part_o + rows * DV;
    p.part_final_stride = rows;
  }
  if constexpr (kSparse) {
    p.tile_keep = a->tile_keep;
    p.tile_partial = a->tile_partial;
    p.tile_mask_base = a->elem_mask_rows > 0 ? a->tile_mask_base : nullptr;
    p.elem_mask = a->elem_mask;
    p.sparse_batch = a->sparse_batch;
    p.sparse_heads = a->sparse_heads;
    p.elem_mask_rows = a->elem_mask_rows;
    p.tile_words = ((a->seq_kv + L::kBN - 1) / L::kBN + 31) / 32;
  }
  auto kernel = parallel_fwd_kernel<F, D, DV, kBf16, NT, kSparse>;
  constexpr int kSmem = kSparse ? L::kBytesSparse : L::kBytes;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  dim3 grid((a->seq_q + NT * L::kBM - 1) / (NT * L::kBM), a->heads, a->batch * splits);
  kernel<<<grid, (4 * NT + 2) * 32, kSmem, stream>>>(tmQ, tmK, tmV, p);
  if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  if (splits > 1) {
    const long long rows = static_cast<long long>(a->batch) * a->heads * a->seq_q;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    parallel_combine_kernel<F, DV, kBf16><<<blocks, 256, 0, stream>>>(p.part_o, p.part_final, p.part_final_stride, a->o,
                                                                     a->final_rowscales[0], a->batch, a->heads, a->seq_q, splits,
                                                                     p.o_sb, p.o_ss, p.o_sh);
    if (cudaGetLastError() != cudaSuccess) return ATTN_B200_E_LAUNCH;
  }
  return ATTN_B200_OK;
}

// dim_v wider than the 128 accumulator columns a query tile has beside its scores (the 256 / 512 of
// examples/retention_parallel.py, the 128 / 256 of the reference's functional suite, testing/test.py:55): one launch per
// 128-column slice of v and o, each recomputing the scores.  With dim_qk 256 a CTA holds one query tile (NT = 1).
template <class F, int D, bool kBf16, int NT, bool kSparse = false>
int launch_parallel_sliced(const AttnB200ParallelArgs* a, cudaStream_t stream, int* device_status) {
  if (a->num_splits > 1) return ATTN_B200_E_UNSUPPORTED;
  for (int dv0 = 0; dv0 < a->dim_v; dv0 += 128) {
    const int rc = launch_parallel<F, D, 128, kBf16, NT, kSparse>(a, stream, device_status, dv0);
    if (rc != ATTN_B200_OK) return rc;
  }
  return ATTN_B200_OK;
}

// The instantiation for one pair of head dims: 64/64 and 128/128 with two query tiles per CTA, 192/128 and 256/128 with
// one (their query and K tiles fill the shared memory), wider dim_v sliced.  A library built for one pair calls this.
template <class F, int D, int DV, bool kBf16, bool kSparse = false>
int launch_parallel_dims(const AttnB200ParallelArgs* a, cudaStream_t stream, int* device_status) {
  static_assert(D == 64 || D == 128 || D == 192 || D == 256, "dim_qk must be 64, 128, 192 or 256");
  constexpr int NT = D <= 128 ? 2 : 1;
  if constexpr (DV > 128) return launch_parallel_sliced<F, D, kBf16, NT, kSparse>(a, stream, device_status);
  else return launch_parallel<F, D, DV, kBf16, NT, kSparse>(a, stream, device_status);
}

// Dispatch over the head-dimension / dtype instantiations compiled for functor F.
template <class F, bool kSparse>
int dispatch_parallel_dims(const AttnB200ParallelArgs* a, cudaStream_t stream, int* device_status) {
  const bool bf16 = a->dtype == ATTN_B200_DTYPE_BF16;
#define ATTN_B200_DIMS(DQ, DVV)                                                                          \
  return bf16 ? launch_parallel_dims<F, DQ, DVV, true, kSparse>(a, stream, device_status)                \
              : launch_parallel_dims<F, DQ, DVV, false, kSparse>(a, stream, device_status)
  if (a->dim_qk == 128 && a->dim_v == 128) { ATTN_B200_DIMS(128, 128); }
  if (a->dim_qk == 64 && a->dim_v == 64) { ATTN_B200_DIMS(64, 64); }
  if (a->dim_qk == 192 && a->dim_v == 128) { ATTN_B200_DIMS(192, 128); }
  if (a->dim_qk == 128 && a->dim_v > 128 && a->dim_v % 128 == 0) { ATTN_B200_DIMS(128, 256); }   // any multiple: sliced
  if (a->dim_qk == 256 && a->dim_v % 128 == 0) { ATTN_B200_DIMS(256, 256); }
#undef ATTN_B200_DIMS
  return ATTN_B200_E_UNSUPPORTED;
}

template <class F>
int dispatch_parallel(const AttnB200ParallelArgs* a, cudaStream_t stream, int* device_status) {
  const int rc = validate_parallel_args(a);
  if (rc != ATTN_B200_OK) return rc;
  return a->tile_keep != nullptr ? dispatch_parallel_dims<F, true>(a, stream, device_status)
                                 : dispatch_parallel_dims<F, false>(a, stream, device_status);
}

}  // namespace b200
