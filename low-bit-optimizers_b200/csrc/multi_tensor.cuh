// Descriptor table of the one-launch multi-tensor steps (AdamW and SGD): the whole parameter list
// travels in the kernel parameters, and every half-warp walks the global sequence of 128-element
// groups through it.
#pragma once
#include "common.cuh"

namespace lpmm_b200 {

constexpr int MAX_TENSORS = 400;  // descriptors per launch (28.9 KB of the 32 KB parameter space)
// One 1024-thread CTA per SM: measured faster than 2 x 512 or 3 x 256 (6.2 vs 5.9 vs 5.3 TB/s in a burst).
constexpr unsigned PF_DIST = 1;  // the L2 prefetch runs this many of a half-warp's iterations ahead (2: same, 3: slower)
constexpr int CTA_THREADS = 1024;
constexpr int CTAS_PER_SM = 1;
constexpr int HW_PER_CTA = CTA_THREADS / 16;

struct TDesc {
  float* p;
  const float* g;
  void* m;
  void* v;
  float* sm;
  float* sv;
  long long numel;
  long long gstart;  // first global group index of this tensor
  int kind;          // LPMM_B200_KIND_*
  int aligned;       // all pointers satisfy the vector-access alignment
};

struct Table {
  int n;
  int pad;
  long long gtotal;  // groups in this table
  TDesc t[MAX_TENSORS];
};


__device__ __forceinline__ float hw_max(float x, unsigned mask) {
#pragma unroll
  for (int o = 8; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(mask, x, o, 16));
  return x;
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

static inline int64_t groups_of(int64_t numel) { return (numel + 127) / 128; }

}  // namespace lpmm_b200
