// Shared device helpers of the sm_100a 4-bit optimizer-step kernels: 256-bit global accesses,
// the nearest-code lookup table, exact division by a group-uniform divisor, host error plumbing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "lpmm_b200.h"

namespace lpmm_b200 {

// ---------------------------------------------------------------------------------------------
// host side: status codes and the per-thread CUDA error text
// ---------------------------------------------------------------------------------------------
int set_cuda_error(cudaError_t e);   // records the text, returns LPMM_B200_ERR_CUDA
int num_sms();                       // SM count of the current device (cached per device)

#define LPMM_CUDA_TRY(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::lpmm_b200::set_cuda_error(_e); \
  } while (0)

// ---------------------------------------------------------------------------------------------
// 256-bit global memory accesses (sm_100 ld/st .v8.f32); addresses must be 32-byte aligned
// ---------------------------------------------------------------------------------------------
struct f8 {
  float x[8];
};

__device__ __forceinline__ f8 ldg_f8(const float* ptr) {
  f8 r;
  asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.x[0]), "=f"(r.x[1]), "=f"(r.x[2]), "=f"(r.x[3]), "=f"(r.x[4]), "=f"(r.x[5]),
                 "=f"(r.x[6]), "=f"(r.x[7])
               : "l"(ptr));
  return r;
}

__device__ __forceinline__ void stg_f8(float* ptr, const f8& r) {
  asm volatile("st.global.v8.f32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"f"(r.x[0]), "f"(r.x[1]), "f"(r.x[2]),
               "f"(r.x[3]), "f"(r.x[4]), "f"(r.x[5]), "f"(r.x[6]), "f"(r.x[7]), "l"(ptr)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Nearest-code lookup table.
//
// The reference's rule (fused_adamw_kernel.cu:27-49, quantization_kernel.cu:397-427) is
//   code(x) = #{ i in 0..14 : mid_i < x },  mid_i = (q[i] + q[i+1]) * 0.5f,  NaN -> 15.
// A binary search costs four dependent shared-memory reads per element.  Instead the float's own
// exponent and top three mantissa bits pick a bucket; if no bucket holds more than one midpoint
// (true for both 4-bit maps of the optimizer) one table read and one compare give the code:
//   code = base[bucket] + (thr[bucket] < x).
// Buckets: index 0 covers |x| < 2^-16, then 8 per octave up to [1, 1.125), and a last one for
// everything larger including NaN (whose compare is false, so its base is 15).  Negative x uses
// a second bank of the same shape.  The table is built per CTA from the caller's qmap; a map that
// does not fit (two midpoints in a bucket, or a midpoint outside (-1.125, 1.125)) clears `valid`
// and the kernels fall back to the binary search.
// ---------------------------------------------------------------------------------------------
constexpr int LUT_LO = (127 - 16) << 3;  // bucket key of 2^-16: (biased exponent << 3) | mantissa[22:20]
constexpr int LUT_NB = 131;              // buckets per sign bank

struct __align__(8) LutEnt {
  float thr;
  int base;
};

struct QuantLut {
  float qmap[16];
  float mids[16];
  LutEnt ent[2 * LUT_NB];
  int valid;
};

// Must be called by every thread of the CTA (contains __syncthreads).
__device__ __forceinline__ void lut_build(QuantLut& L, const float* __restrict__ qmap_g) {
  const int tid = threadIdx.x;
  if (tid < 16) L.qmap[tid] = qmap_g[tid];
  if (tid == 0) L.valid = 1;
  __syncthreads();
  if (tid < 15) {
    const float m = __fmul_rn(__fadd_rn(L.qmap[tid], L.qmap[tid + 1]), 0.5f);
    L.mids[tid] = m;
    if (!(fabsf(m) < 1.125f) || !(L.qmap[tid] < L.qmap[tid + 1])) L.valid = 0;
  }
  __syncthreads();
  const float inf = __int_as_float(0x7f800000);
  for (int e = tid; e < 2 * LUT_NB; e += blockDim.x) {
    const int neg = e >= LUT_NB;
    const int t = e - neg * LUT_NB;
    float lo, hi;  // magnitudes: the bucket holds lo <= |x| < hi
    if (t == 0) {
      lo = 0.0f;
      hi = __int_as_float(LUT_LO << 20);
    } else if (t == LUT_NB - 1) {
      lo = __int_as_float((LUT_LO + t - 1) << 20);
      hi = inf;
    } else {
      lo = __int_as_float((LUT_LO + t - 1) << 20);
      hi = __int_as_float((LUT_LO + t) << 20);
    }
    int base = 0, cnt = 0;
    float thr = inf;
    for (int i = 0; i < 15; ++i) {
      const float m = L.mids[i];
      if (!neg) {
        if (m < lo) ++base;
        else if (m < hi) { ++cnt; thr = m; }
      } else {
        if (m <= -hi) ++base;
        else if (m <= -lo) { ++cnt; thr = m; }
      }
    }
    if (t == LUT_NB - 1) { base = 15; thr = inf; }  // NaN (either sign) -> 15
    if (cnt > 1) L.valid = 0;
    LutEnt en;
    en.thr = thr;
    en.base = base;
    L.ent[e] = en;
  }
  __syncthreads();
}

// code(x) through the table; requires L.valid.  x beyond +-1.125 maps to 15 (callers that can
// see such values clamp first).
__device__ __forceinline__ int lut_code(const LutEnt* __restrict__ ent, float x) {
  const uint32_t b = __float_as_uint(x);
  const int k = (int)((b & 0x7fffffffu) >> 20);
  int t = max(k, LUT_LO - 1);
  t = min(t, LUT_LO + LUT_NB - 2) - (LUT_LO - 1);
  const int idx = t + ((int)(b >> 31)) * LUT_NB;
  const LutEnt e = ent[idx];
  return e.base + (e.thr < x ? 1 : 0);
}

// The reference's search, verbatim in behaviour, for maps the table cannot hold.
__device__ __forceinline__ int bsearch_code(const float* __restrict__ q, float x) {
  if (x <= q[0]) return 0;
  if (q[15] <= x) return 15;
  if (x != x) return 15;
  int lo = 0, hi = 16;
  while (lo < hi) {
    const int mi = (lo + hi) >> 1;
    if (q[mi] <= x) lo = mi + 1;
    else hi = mi;
  }
  const float mid = __fmul_rn(__fadd_rn(q[lo - 1], q[lo]), 0.5f);
  return (mid < x) ? lo : lo - 1;
}

// ---------------------------------------------------------------------------------------------
// Correctly rounded x / d for a divisor shared by many elements.
// With r = RN(1/d), q = RN(x*r), e = x - q*d (exact in an FMA), RN(q + e*r) equals RN(x/d)
// whenever nothing under- or overflows.  Outside a conservative range of d the IEEE division is
// used instead.  Results below 2^-18 in magnitude may differ in the last bit when e underflows;
// every quantization threshold is far above that.
// ---------------------------------------------------------------------------------------------
struct UDiv {
  float d, r;
  bool fast;
};

__device__ __forceinline__ UDiv udiv_make(float d) {
  UDiv u;
  u.d = d;
  u.fast = (d >= 0x1p-60f) && (d <= 0x1p60f);
  u.r = __frcp_rn(d);
  return u;
}

__device__ __forceinline__ float udiv(float x, const UDiv& u) {
  if (u.fast) {
    const float q = __fmul_rn(x, u.r);
    const float e = __fmaf_rn(-q, u.d, x);
    return __fmaf_rn(e, u.r, q);
  }
  return __fdiv_rn(x, u.d);
}

}  // namespace lpmm_b200
