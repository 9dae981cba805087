// Shared device helpers of the sm_100a 4-bit optimizer-step kernels: 256-bit global accesses,
// the nearest-code lookup table, exact division by a group-uniform divisor, short correctly
// rounded sqrt / division sequences, host error plumbing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "lpmm_b200.h"

// Functions shared between the library's translation units but not part of its C ABI: C linkage, not exported.
#define LPMM_INTERNAL extern "C" __attribute__((visibility("hidden")))

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
               "f"(r.x[3]), "f"(r.x[4]), "f"(r.x[5]), "f"(r.x[6]), "f"(r.x[7]), "l"(ptr));
}

// ---------------------------------------------------------------------------------------------
// Nearest-code lookup table.
//
// The reference's rule (fused_adamw_kernel.cu:27-49, quantization_kernel.cu:397-427) is
//   code(x) = #{ i in 0..14 : mid_i < x },  mid_i = (q[i] + q[i+1]) * 0.5f,  NaN -> 15.
// A binary search costs four dependent shared-memory reads per element.  Instead the top 12 bits
// of the float (sign, exponent, three mantissa bits) index a 4096-entry table in shared memory;
// provided no bucket holds more than one midpoint (true for both 4-bit maps of the optimizer),
//   code = base[bucket] + (thr[bucket] < x)
// is exact for every bit pattern: buckets without a midpoint carry thr = +inf, the NaN buckets
// carry base 15 (a NaN compares false).  The one deviation: -inf shares its bucket with negative
// NaNs and therefore maps to 15 instead of 0; callers that may see -inf clamp first.  A map that
// does not fit (two midpoints in one bucket) clears `valid` and the kernels fall back to the
// binary search.  The table is built per CTA from the caller's qmap.
// ---------------------------------------------------------------------------------------------
constexpr int LUT_ENTRIES = 4096;

struct __align__(8) LutEnt {
  float thr;
  int base;
};

struct QMapSmem {   // small static part, one per map
  float qmap[16];
  float mids[16];
  int valid;        // table usable
  int linear16;     // qmap[i] == (i+1)/16 exactly: closed-form code available
};

// Must be called by every thread of the CTA (contains __syncthreads).  `ent` may be nullptr when
// the caller will not use the table (only qmap/mids/linear16 are filled then).
__device__ __forceinline__ void lut_build(QMapSmem& S, LutEnt* __restrict__ ent, const float* __restrict__ qmap_g) {
  const int tid = threadIdx.x;
  if (tid < 16) S.qmap[tid] = qmap_g[tid];
  if (tid == 0) {
    S.valid = 1;
    S.linear16 = 1;
  }
  __syncthreads();
  if (tid < 15) {
    S.mids[tid] = __fmul_rn(__fadd_rn(S.qmap[tid], S.qmap[tid + 1]), 0.5f);
    if (!(S.qmap[tid] < S.qmap[tid + 1])) S.valid = 0;
  }
  if (tid < 16 && S.qmap[tid] != (float)(tid + 1) * 0.0625f) S.linear16 = 0;
  __syncthreads();
  if (ent == nullptr) return;
  const float inf = __int_as_float(0x7f800000);
  for (int e = tid; e < LUT_ENTRIES; e += blockDim.x) {
    const int neg = e >> 11;
    const int key = e & 0x7ff;
    int base = 0, cnt = 0;
    float thr = inf;
    if (key >= 0x7f8) {  // inf and NaN
      base = 15;
    } else {
      const float lo = __int_as_float(key << 20);        // bucket holds lo <= |x| < hi
      const float hi = __int_as_float((key + 1) << 20);  // key 0x7f7 -> hi = +inf
      for (int i = 0; i < 15; ++i) {
        const float m = S.mids[i];
        if (!neg) {
          if (m < lo) ++base;
          else if (m < hi) { ++cnt; thr = m; }
        } else {
          if (m <= -hi) ++base;
          else if (m <= -lo) { ++cnt; thr = m; }
        }
      }
    }
    if (cnt > 1) S.valid = 0;
    LutEnt en;
    en.thr = thr;
    en.base = base;
    ent[e] = en;
  }
  __syncthreads();
}

__device__ __forceinline__ int lut_code(const LutEnt* __restrict__ ent, float x) {
  const LutEnt e = ent[__float_as_uint(x) >> 20];
  return e.base + (e.thr < x ? 1 : 0);
}

// Closed form of the rule for the map q[i] = (i+1)/16 (midpoints (2k+1)/32, k = 1..15):
// code = clamp(ceil(16x - 1.5), 0, 15).  16x - 1.5 is exact whenever it is positive, and the
// float->unsigned conversion with round-up saturates negatives to 0.  Valid for x <= 1 (always
// true of a value divided by its group maximum); NaN gives 0 here, so the caller handles the only
// NaN source, an all-zero group, itself.  Checked against the rule for every bit pattern in
// [-1e30, 1].
__device__ __forceinline__ uint32_t linear16_code(float x) {
  return __float2uint_ru(__fmaf_rn(x, 16.0f, -1.5f));
}

// Nearest-code rule of a 16-entry map as a branch-free four-step search over its 15 sorted midpoints
// (padded with +inf): code = #{midpoints < x}; a NaN gives 15 like the reference's search.
__device__ __forceinline__ int code16(const float* __restrict__ mids, float x) {
  int c = (mids[7] < x) ? 8 : 0;
  c += (mids[c + 3] < x) ? 4 : 0;
  c += (mids[c + 1] < x) ? 2 : 0;
  c += (mids[c] < x) ? 1 : 0;
  return (x != x) ? 15 : c;
}

// Monotone max of a non-negative float through an integer atomic; a stale read can only be too
// small, so skipping the atomic when the value is not larger is always safe.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float val) {
  if (val > *reinterpret_cast<volatile float*>(addr)) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(val));
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
// Correctly rounded x / d for a divisor shared by many elements (Markstein's correction):
// with r = RN(1/d), q = RN(x*r), e = x - q*d (exact in an FMA), RN(q + e*r) equals RN(x/d)
// whenever nothing under- or overflows.  Checked against IEEE division on 2.4e10 random and
// adversarial pairs.  d == 0 gives r = +inf and 0*inf = NaN, the same NaN 0/0 gives.
// Quotients below 2^-18 in magnitude may differ in the last bit when e underflows; every
// quantization threshold is far above that.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool udiv_ok(float d) { return (d <= 0x1p60f) && (d >= 0x1p-60f || d == 0.0f); }

__device__ __forceinline__ float udiv(float x, float d, float r) {
  const float q = __fmul_rn(x, r);
  const float e = __fmaf_rn(-q, d, x);
  return __fmaf_rn(e, r, q);
}

// ---------------------------------------------------------------------------------------------
// Short sequences for sqrt and division, each equal to the IEEE result on its stated domain.
// sqrt_rn_fast: every v >= 2^-102 and v == 0 (exhaustively checked against sqrt.rn.f32); in [2^-126, 2^-102)
//   the residual underflows and the last bit may differ; a denormal v gives v * 2^63 (at most 2^-63, like the
//   true root).  The hosts select it only when both cases vanish against eps or change it by a last bit.
// div_rn_fast: 2^-60 <= d <= 2^60, 2^-60 <= |m| <= 2^30 or m == 0 (2.4e10 random and adversarial
//   pairs against div.rn.f32); a denormal quotient may differ in the last bit.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float mufu_rsq(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float mufu_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Approximate square root (within 2^-23 relative; 0 and denormals give 0): tolerance-mode parameter update only.
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// MUFU reciprocal refined once; the reciprocal both fma-corrected divisions below are built on.
__device__ __forceinline__ float rcp_nr(float d) {
  const float r = mufu_rcp(d);
  return __fmaf_rn(r, __fmaf_rn(-d, r, 1.0f), r);
}

__device__ __forceinline__ float sqrt_rn_fast(float v) {
  const float y = mufu_rsq(fmaxf(v, 1.17549435e-38f));
  const float s = __fmul_rn(v, y);
  const float h = __fmul_rn(0.5f, y);
  const float e = __fmaf_rn(-s, s, v);
  return __fmaf_rn(e, h, s);
}

__device__ __forceinline__ float div_rn_fast(float m, float d) {
  const float r = rcp_nr(d);
  const float q = __fmul_rn(m, r);
  const float rem = __fmaf_rn(-d, q, m);
  return __fmaf_rn(rem, r, q);
}


// ---------------------------------------------------------------------------------------------
// Packed fp32x2 arithmetic (sm_100 add/mul/fma .f32x2): one instruction, two IEEE round-to-nearest
// results, each bit-identical to the scalar instruction on its half.  Values live in 64-bit
// registers (low half = element 2j, high half = element 2j+1).
// ---------------------------------------------------------------------------------------------
typedef unsigned long long f2;

__device__ __forceinline__ f2 f2_pack(float lo, float hi) {
  f2 r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f2 f2_splat(float x) { return f2_pack(x, x); }
__device__ __forceinline__ void f2_unpack(f2 v, float& lo, float& hi) {
  asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 f2_mul(f2 a, f2 b) {
  f2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f2 f2_add(f2 a, f2 b) {
  f2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f2 f2_fma(f2 a, f2 b, f2 c) {
  f2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// RN(RN(a * b) + c) per half, two roundings.  Done with scalar instructions: a packed mul.rn
// whose only use is a packed add.rn was observed (random inputs, against the scalar pair) to come
// out as one fused multiply-add, and so was an fma with a -0.0 addend followed by the add.
__device__ __forceinline__ f2 f2_mul_then_add(f2 a, f2 b, f2 c) {
  float a0, a1, b0, b1, c0, c1;
  f2_unpack(a, a0, a1);
  f2_unpack(b, b0, b1);
  f2_unpack(c, c0, c1);
  return f2_pack(__fadd_rn(__fmul_rn(a0, b0), c0), __fadd_rn(__fmul_rn(a1, b1), c1));
}

struct f2x4 {
  f2 v[4];
};
__device__ __forceinline__ f2x4 ldg_f2x4(const float* ptr) {
  f2x4 r;
    asm volatile("ld.global.L1::no_allocate.v4.b64 {%0,%1,%2,%3}, [%4];"
               : "=l"(r.v[0]), "=l"(r.v[1]), "=l"(r.v[2]), "=l"(r.v[3])
               : "l"(ptr));
  return r;
}
__device__ __forceinline__ void stg_f2x4(float* ptr, const f2x4& r) {
#ifdef LPMM_ST_CS  // streaming (evict-first) store hint (experiment)
    asm volatile("st.global.cs.v4.b64 [%4], {%0,%1,%2,%3};" ::"l"(r.v[0]), "l"(r.v[1]), "l"(r.v[2]), "l"(r.v[3]), "l"(ptr));
#else
    asm volatile("st.global.v4.b64 [%4], {%0,%1,%2,%3};" ::"l"(r.v[0]), "l"(r.v[1]), "l"(r.v[2]), "l"(r.v[3]), "l"(ptr));
#endif
}

}  // namespace lpmm_b200
