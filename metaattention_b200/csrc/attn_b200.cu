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

}  // namespace b200

extern "C" {

int attn_b200_version(void) { return 100; }

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
  // fp32 partial rows plus one log-sum-exp per row and split
  return static_cast<int64_t>(args->batch) * args->num_splits * args->heads * args->seq_q * (args->dim_v + 1) * 4;
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
