// fp32 -> bf16 / fp16 copy of a parameter range (round to nearest even): the 16-bit replicas of fp32 master
// parameters in the sharded step (every rank keeps fp32 parameters only for its own range and publishes them to the
// other ranks at half the bytes).  HBM-bound: 4 bytes read and 2 written per element, 8 elements per thread.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace lpmm_b200 {

template <typename T>
__device__ __forceinline__ uint32_t narrow2(float a, float b);
template <>
__device__ __forceinline__ uint32_t narrow2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);  // .x = a (low half), .y = b
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t narrow2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// `head` elements before the first 32-byte boundary of src and the tail after the last full lane are converted one
// by one; vector lanes need dst 16-byte aligned at that point as well (host-checked, else everything goes one by one).
template <typename T>
__global__ void __launch_bounds__(256) narrow_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n,
                                                     long long head, long long lanes) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < lanes; i += nthreads) {
    const long long e = head + i * 8;
    const float4 a = *reinterpret_cast<const float4*>(src + e);
    const float4 b = *reinterpret_cast<const float4*>(src + e + 4);
    uint4 o;
    o.x = narrow2<T>(a.x, a.y);
    o.y = narrow2<T>(a.z, a.w);
    o.z = narrow2<T>(b.x, b.y);
    o.w = narrow2<T>(b.z, b.w);
    *reinterpret_cast<uint4*>(dst + e) = o;
  }
  const long long done = head + lanes * 8;
  for (long long e = tid; e < head; e += nthreads) dst[e] = T(src[e]);
  for (long long e = done + tid; e < n; e += nthreads) dst[e] = T(src[e]);
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

extern "C" int lpmm_b200_narrow_fp32(const float* src, void* dst, int64_t numel, int dtype, void* stream) {
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (dtype != LPMM_B200_DTYPE_BF16 && dtype != LPMM_B200_DTYPE_FP16) return LPMM_B200_ERR_BAD_KIND;
  if (numel == 0) return LPMM_B200_OK;
  if (!src || !dst) return LPMM_B200_ERR_NULL_POINTER;
  if (((uintptr_t)src & 3) || ((uintptr_t)dst & 1)) return LPMM_B200_ERR_BAD_SIZE;
  // elements up to the first 32-byte boundary of src; the vector path needs dst on a 16-byte boundary there
  long long head = (long long)(((32 - ((uintptr_t)src & 31)) & 31) / 4);
  if (head > numel) head = numel;
  long long lanes = (numel - head) / 8;
  if (((uintptr_t)dst + 2 * (uintptr_t)head) & 15) {
    head = numel;
    lanes = 0;
  }
  const long long work = lanes > 0 ? lanes : numel;
  long long grid = (work + 255) / 256;
  const long long cap = (long long)num_sms() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  if (dtype == LPMM_B200_DTYPE_BF16)
    narrow_kernel<__nv_bfloat16><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
        src, reinterpret_cast<__nv_bfloat16*>(dst), numel, head, lanes);
  else
    narrow_kernel<__half><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(src, reinterpret_cast<__half*>(dst), numel,
                                                                             head, lanes);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
