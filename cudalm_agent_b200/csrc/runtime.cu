// Process-wide state of the library: status strings, the device status word,
// launch counter, kernel introspection.
#include <cstring>

#include "common.cuh"

namespace cb200 {

thread_local int g_last_cuda_error = 0;
std::atomic<long long> g_launch_count{0};

// One status word per device, in the library's own device image.
__device__ int g_status_word = 0;

int* device_status_word() {
  // one lookup per device; the address never changes afterwards
  static std::atomic<int*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0) {
    int* hit = cached[dev].load(std::memory_order_acquire);
    if (hit) return hit;
  }
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_status_word);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return nullptr;
  }
  if (dev >= 0) cached[dev].store(static_cast<int*>(p), std::memory_order_release);
  return static_cast<int*>(p);
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace cb200

extern "C" {

const char* cudalm_b200_status_string(int status) {
  switch (status) {
    case CUDALM_B200_OK: return "ok";
    case CUDALM_B200_ERR_BAD_SHAPE: return "bad shape (need N >= 1, K > 0, K % 128 == 0, M >= 1)";
    case CUDALM_B200_ERR_NULL: return "null pointer";
    case CUDALM_B200_ERR_MISALIGNED: return "pointer misses a required alignment";
    case CUDALM_B200_ERR_CUDA: return "CUDA runtime error (see cudalm_b200_last_cuda_error)";
    case CUDALM_B200_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case CUDALM_B200_ERR_UNSUPPORTED: return "unsupported configuration";
    case CUDALM_B200_ERR_TOO_LARGE: return "size exceeds a fixed capacity";
    case CUDALM_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case CUDALM_B200_ERR_FILE: return "weight file missing or malformed";
    default: return "unknown status";
  }
}

int cudalm_b200_last_cuda_error(void) { return cb200::g_last_cuda_error; }

const char* cudalm_b200_build_info(void) { return "sm_100a;cudalm_b200 " __DATE__; }

int cudalm_b200_device_status(int* status_out) {
  if (!status_out) return CUDALM_B200_ERR_NULL;
  int* word = cb200::device_status_word();
  if (!word) return CUDALM_B200_ERR_CUDA;
  int v = 0;
  CB200_CUDA_TRY(cudaDeviceSynchronize());
  CB200_CUDA_TRY(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    const int zero = 0;
    CB200_CUDA_TRY(cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  *status_out = v;
  return CUDALM_B200_OK;
}

int64_t cudalm_b200_launch_count(void) {
  return cb200::g_launch_count.load(std::memory_order_relaxed);
}

}  // extern "C"
