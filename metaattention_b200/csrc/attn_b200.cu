// C ABI of libattn_b200.so: status/version entry points and the parallel-pattern forward with
// the built-in functors.  The MLA decode and linear-attention entry points live in their own
// translation units of the same library.
#include <mutex>

#include "../../include/attn_b200.h"
#include "common_host.cuh"
#include "functors.cuh"
#include "parallel_launch.cuh"

namespace b200 {

int* device_status_word(int device) {
  constexpr int kMaxDevices = 64;
  static int* words[kMaxDevices] = {};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (words[device] == nullptr) {
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return nullptr;
    int* w = nullptr;
    bool ok = cudaSetDevice(device) == cudaSuccess && cudaMalloc(&w, sizeof(int)) == cudaSuccess &&
              cudaMemset(w, 0, sizeof(int)) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    cudaSetDevice(prev);
    if (!ok) {
      cudaGetLastError();
      return nullptr;
    }
    words[device] = w;
  }
  return words[device];
}

// Tile bitmaps and column masks of a block-sparse, variable-length decode: one CTA per (sequence, KV head).
// A KV position takes part when its block is flagged and it lies inside the sequence's cache length.
__global__ void __launch_bounds__(128) decode_tiles_kernel(const uint8_t* __restrict__ block_mask, const int32_t* __restrict__ seq_lens,
                                                         int heads_kv, int n_blocks, int block_size, int seq_kv, int words,
                                                         uint32_t* __restrict__ keep, uint32_t* __restrict__ partial,
                                                         uint32_t* __restrict__ col_mask) {
  const int bh = blockIdx.x;
  const int b = bh / heads_kv;
  const int n_tiles = (seq_kv + 127) / 128;
  const int len = seq_lens != nullptr ? min(max(seq_lens[b], 0), seq_kv) : seq_kv;
  const uint8_t* bm = block_mask != nullptr ? block_mask + static_cast<long long>(bh) * n_blocks : nullptr;
  for (int w = threadIdx.x; w < words; w += blockDim.x) keep[static_cast<long long>(bh) * words + w] = partial[static_cast<long long>(bh) * words + w] = 0u;
  __syncthreads();
  for (int j = threadIdx.x; j < n_tiles; j += blockDim.x) {
    uint32_t word[4];
    bool any = false, all = true;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t bits = 0;
      for (int c = 0; c < 32; ++c) {
        const int pos = j * 128 + w * 32 + c;
        const int blk = pos / block_size;
        const bool k = pos < len && (bm == nullptr || (blk < n_blocks && bm[blk] != 0));
        bits |= static_cast<uint32_t>(k) << c;
      }
      word[w] = bits;
      any |= bits != 0u;
      all &= bits == 0xffffffffu;
    }
    uint4* dst = reinterpret_cast<uint4*>(col_mask + (static_cast<long long>(bh) * n_tiles + j) * 4);
    *dst = make_uint4(word[0], word[1], word[2], word[3]);
    if (any) atomicOr(&keep[static_cast<long long>(bh) * words + (j >> 5)], 1u << (j & 31));
    if (any && !all) atomicOr(&partial[static_cast<long long>(bh) * words + (j >> 5)], 1u << (j & 31));
  }
}

}  // namespace b200

extern "C" {

int attn_b200_version(void) { return 200; }

int64_t attn_b200_decode_tiles_bytes(int32_t batch, int32_t heads_kv, int32_t seq_kv) {
  if (batch <= 0 || heads_kv <= 0 || seq_kv <= 0) return -1;
  const int64_t tiles = (seq_kv + 127) / 128, words = (tiles + 31) / 32;
  return static_cast<int64_t>(batch) * heads_kv * (tiles * 16 + 2 * words * 4);
}

int attn_b200_decode_tiles(const uint8_t* block_mask, const int32_t* cache_seqlens, int32_t batch, int32_t heads_kv,
                           int32_t n_blocks, int32_t block_size, int32_t seq_kv, void* out, int64_t out_bytes,
                           void* cuda_stream) {
  if (out == nullptr || batch <= 0 || heads_kv <= 0 || seq_kv <= 0) return ATTN_B200_E_INVALID_ARG;
  if (block_mask != nullptr && (n_blocks <= 0 || block_size <= 0)) return ATTN_B200_E_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0) return ATTN_B200_E_UNSUPPORTED;
  if (static_cast<int64_t>(batch) * heads_kv > 0x7fffffff) return ATTN_B200_E_UNSUPPORTED;
  if (out_bytes < attn_b200_decode_tiles_bytes(batch, heads_kv, seq_kv)) return ATTN_B200_E_WORKSPACE;
  const int64_t tiles = (seq_kv + 127) / 128, words = (tiles + 31) / 32, bh = static_cast<int64_t>(batch) * heads_kv;
  uint32_t* col_mask = static_cast<uint32_t*>(out);
  uint32_t* keep = col_mask + bh * tiles * 4;
  uint32_t* partial = keep + bh * words;
  b200::decode_tiles_kernel<<<static_cast<unsigned>(bh), 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      block_mask, cache_seqlens, heads_kv, block_mask != nullptr ? n_blocks : 1, block_mask != nullptr ? block_size : seq_kv, seq_kv,
      static_cast<int>(words), keep, partial, col_mask);
  return cudaGetLastError() == cudaSuccess ? ATTN_B200_OK : ATTN_B200_E_LAUNCH;
}

int attn_b200_device_status_word(int32_t device, int32_t** word_out) {
  if (word_out == nullptr) return ATTN_B200_E_INVALID_ARG;
  int* w = b200::device_status_word(device);
  if (w == nullptr) return ATTN_B200_E_LAUNCH;
  *word_out = w;
  return ATTN_B200_OK;
}

int attn_b200_last_device_status(int32_t device, int32_t* status_out) {
  if (status_out == nullptr) return ATTN_B200_E_INVALID_ARG;
  int* w = b200::device_status_word(device);
  if (w == nullptr) return ATTN_B200_E_LAUNCH;
  int prev = -1;
  cudaGetDevice(&prev);
  int v = 0;
  bool ok = cudaSetDevice(device) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess &&
            cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess;
  if (ok && v != 0) ok = cudaMemset(w, 0, sizeof(int)) == cudaSuccess;
  cudaSetDevice(prev);
  if (!ok) {
    cudaGetLastError();
    return ATTN_B200_E_LAUNCH;
  }
  *status_out = v;
  return ATTN_B200_OK;
}

int64_t attn_b200_parallel_workspace_bytes(const AttnB200ParallelArgs* args) {
  if (args == nullptr || args->batch <= 0 || args->heads <= 0 || args->seq_q <= 0 || args->dim_v <= 0) return -1;
  if (args->num_splits <= 1) return 0;
  // fp32 partial rows plus the final row scales of every row and split
  return static_cast<int64_t>(args->batch) * args->num_splits * args->heads * args->seq_q * (args->dim_v + ATTN_B200_MAX_ROWSCALES) * 4;
}

int attn_b200_parallel_fwd(const AttnB200ParallelArgs* args, void* cuda_stream) {
  if (args == nullptr) return ATTN_B200_E_INVALID_ARG;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ATTN_B200_E_LAUNCH;
  int* status = b200::device_status_word(dev);
  if (status == nullptr) return ATTN_B200_E_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  switch (args->functor) {
    case ATTN_B200_FUNCTOR_SOFTMAX:
      return b200::dispatch_parallel<b200::SoftmaxFunctor>(args, stream, status);
    default:
      return ATTN_B200_E_INVALID_ARG;
  }
}

}  // extern "C"
