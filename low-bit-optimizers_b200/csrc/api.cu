// Host-side plumbing of the C ABI: status texts, per-thread CUDA error text, device queries.
#include <string>

#include "common.cuh"

namespace lpmm_b200 {

static thread_local std::string g_last_cuda_error;

int set_cuda_error(cudaError_t e) {
  g_last_cuda_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e);
  return LPMM_B200_ERR_CUDA;
}

int num_sms() {
  static int cached[64];  // zero-initialised; 0 = not queried yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace lpmm_b200

extern "C" const char* lpmm_b200_strerror(int status) {
  switch (status) {
    case LPMM_B200_OK: return "ok";
    case LPMM_B200_ERR_NULL_POINTER: return "a required pointer is NULL";
    case LPMM_B200_ERR_BAD_SIZE: return "negative or inconsistent size / range";
    case LPMM_B200_ERR_BAD_KIND: return "unknown kind or option value";
    case LPMM_B200_ERR_CUDA: return "CUDA runtime error (see lpmm_b200_last_cuda_error)";
    case LPMM_B200_ERR_UNSUPPORTED: return "not supported by this build";
    case LPMM_B200_ERR_TOO_LARGE: return "size exceeds a documented static limit";
    default: return "unknown status";
  }
}

extern "C" const char* lpmm_b200_last_cuda_error(void) { return lpmm_b200::g_last_cuda_error.c_str(); }

extern "C" int lpmm_b200_abi_version(void) { return 3; }
