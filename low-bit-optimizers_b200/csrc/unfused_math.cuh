// Arithmetic of the reference's non-fused AdamW step (lpmm/optim/adamw.py:369, 412-422), i.e. of the
// torch CUDA kernels it runs, operation by operation:
//   p1 = p * float(1 - lr*wd)
//   m  = fma(w, g - m0, m0),  w = float(1 - beta1)                  torch lerp, weight < 0.5
//   v  = fma(float(1 - beta2), g*g, v0 * float(beta2))              mul_ then addcmul_
//   d  = sqrt(v) * float(1.0 / sqrt(1 - beta2^step)) + float(eps)    division by a host scalar
//   p  = fma(float(-lr / (1 - beta1^step)), m / d, p1)              addcdiv_
// with the scalar constants computed in double on the host exactly as Python computes them.
//
// The scalar functions also come in a second flavour (template argument A = true): the arithmetic of
// the reference's fused kernel (lpmm/cpp_extension/fused_adamw_kernel.cu:103-128), all in float,
//   m = fma(b1, m0, (1-b1)*g) ; v = fma(b2, v0, ((1-b2)*g)*g)
//   d = (sqrt(v)/sqrt(1-b2^t) + eps) * (1-b1^t) ; p = fma(-lr, fma(wd, p, m/d), p)
// with the bias corrections from the device's powf.  It lets the kernels built on this header run the
// fused step on the states the fused kernel cannot hold (rank-1 second-moment scales).
#pragma once
#include <math.h>

#include "common.cuh"

namespace lpmm_b200 {

struct UConsts {
  float wd_mul, lerp_w, lerp_omw, beta2, omb2, inv_bc2s, bc2s, eps, alpha;
  int lerp_small;
  int fast;  // eps keeps the denominator inside the domain of the short exact sqrt / division sequences
  // fused-kernel arithmetic (A = true): the hyper-parameters as floats; c1, c2s, rc2s are filled in on
  // the device by fused_consts()
  float f_beta1, f_omb1, f_beta2, f_omb2, f_lr, f_wd, f_eps, f_step, c1, c2s, rc2s;
  int f_fast;
};

// 1 - beta1^t, sqrt(1 - beta2^t) and the latter's reciprocal, as the fused kernel computes them.
__device__ __forceinline__ UConsts fused_consts(UConsts c) {
  c.c1 = __fsub_rn(1.0f, powf(c.f_beta1, c.f_step));
  c.c2s = __fsqrt_rn(__fsub_rn(1.0f, powf(c.f_beta2, c.f_step)));
  c.rc2s = __frcp_rn(c.c2s);
  return c;
}


template <bool A = false>
__device__ __forceinline__ float lerp_m(const UConsts& c, float m0, float g) {
  if (A) return __fmaf_rn(c.f_beta1, m0, __fmul_rn(c.f_omb1, g));
  const float diff = __fsub_rn(g, m0);
  return c.lerp_small ? __fmaf_rn(c.lerp_w, diff, m0) : __fmaf_rn(-diff, c.lerp_omw, g);
}
template <bool A = false>
__device__ __forceinline__ float upd_v2(const UConsts& c, float v0, float g) {
  if (A) return __fmaf_rn(c.f_beta2, v0, __fmul_rn(__fmul_rn(c.f_omb2, g), g));
  return __fmaf_rn(c.omb2, __fmul_rn(g, g), __fmul_rn(v0, c.beta2));
}
template <bool A = false>
__device__ __forceinline__ float upd_param(const UConsts& c, float p, float m, float v) {
  if (A) {
    float d = c.f_fast ? udiv(sqrt_rn_fast(v), c.c2s, c.rc2s) : __fdiv_rn(__fsqrt_rn(v), c.c2s);
    d = __fmul_rn(__fadd_rn(d, c.f_eps), c.c1);
    const float q = c.f_fast ? div_rn_fast(m, d) : __fdiv_rn(m, d);
    return __fmaf_rn(-c.f_lr, __fmaf_rn(c.f_wd, p, q), p);
  }
  const float p1 = __fmul_rn(p, c.wd_mul);
  if (c.fast) {
    const float d = __fadd_rn(__fmul_rn(sqrt_rn_fast(v), c.inv_bc2s), c.eps);
    return __fmaf_rn(c.alpha, div_rn_fast(m, d), p1);
  }
  const float d = __fadd_rn(__fmul_rn(__fsqrt_rn(v), c.inv_bc2s), c.eps);
  return __fmaf_rn(c.alpha, __fdiv_rn(m, d), p1);
}

// The same update for two elements per instruction (sm_100 packed fp32: each half is the IEEE
// result of the scalar instruction), for lanes whose 8 elements all exist and hyper-parameters in
// the domain of the short sqrt / division sequences.
struct UConsts2 {
  f2 wd_mul, lerp_a, beta2, omb2, inv_bc2s, eps, alpha, mone, half, one;
  int lerp_small;
};
__device__ __forceinline__ UConsts2 make_consts2(const UConsts& c) {
  UConsts2 k;
  k.wd_mul = f2_splat(c.wd_mul);
  k.lerp_a = f2_splat(c.lerp_small ? c.lerp_w : -c.lerp_omw);  // fma(-d, w', g) == fma(d, -w', g)
  k.beta2 = f2_splat(c.beta2);
  k.omb2 = f2_splat(c.omb2);
  k.inv_bc2s = f2_splat(c.inv_bc2s);
  k.eps = f2_splat(c.eps);
  k.alpha = f2_splat(c.alpha);
  k.mone = f2_splat(-1.0f);
  k.half = f2_splat(0.5f);
  k.one = f2_splat(1.0f);
  k.lerp_small = c.lerp_small;
  return k;
}
// p updated from the new moments m, v (pairs): sqrt and division as in sqrt_rn_fast / div_rn_fast.
__device__ __forceinline__ void param_pair(const UConsts2& k, f2& p, f2 m, f2 v) {
  float va, vb;
  f2_unpack(v, va, vb);
  const f2 y = f2_pack(mufu_rsq(fmaxf(va, 1.17549435e-38f)), mufu_rsq(fmaxf(vb, 1.17549435e-38f)));
  f2 sq = f2_mul(v, y);
  const f2 e = f2_fma(sq, f2_mul(sq, k.mone), v);
  sq = f2_fma(e, f2_mul(k.half, y), sq);
  // d = sqrt(v) * (1 / bc2s) + eps; m / d on the negated denominator
  const f2 d = f2_mul_then_add(sq, k.inv_bc2s, k.eps);  // two roundings, like the torch ops
  const f2 nd = f2_mul(d, k.mone);
  float da, db;
  f2_unpack(d, da, db);
  const f2 r0 = f2_pack(mufu_rcp(da), mufu_rcp(db));
  const f2 r = f2_fma(r0, f2_fma(nd, r0, k.one), r0);
  const f2 q = f2_mul(m, r);
  const f2 quo = f2_fma(f2_fma(nd, q, m), r, q);
  p = f2_fma(k.alpha, quo, f2_mul(p, k.wd_mul));               // addcdiv_ on the decayed parameter
}
// Tolerance mode of the same update (the parameter may differ from the exact path's in its last bits; the moments,
// and with them every code and scale, do not depend on it): approximate square root and reciprocal (2^-23 relative
// each), d = fma(sqrt(v), 1/bc2s, eps), p = fma(alpha * m, 1/d, p * wd_mul).  Needs d > 0, i.e. the eps of `fast`.
__device__ __forceinline__ void param_pair_apx(const UConsts2& k, f2& p, f2 m, f2 v) {
  float va, vb;
  f2_unpack(v, va, vb);
  const f2 sq = f2_pack(sqrt_approx(va), sqrt_approx(vb));
  float da, db;
  f2_unpack(f2_fma(sq, k.inv_bc2s, k.eps), da, db);
  const f2 r = f2_pack(mufu_rcp(da), mufu_rcp(db));
  p = f2_fma(f2_mul(k.alpha, m), r, f2_mul(p, k.wd_mul));
}
// First moment of a pair: lerp_(g, 1 - beta1); am collects max |m|.
__device__ __forceinline__ f2 lerp_pair(const UConsts2& k, f2 g, f2 m0, float& am) {
  const f2 diff = f2_fma(m0, k.mone, g);                       // g - m0
  const f2 m = f2_fma(k.lerp_a, diff, k.lerp_small ? m0 : g);
  float ma, mb;
  f2_unpack(m, ma, mb);
  am = fmaxf(am, fmaxf(fabsf(ma), fabsf(mb)));
  return m;
}
// In: g, p, the old moments m0, v0 (pairs).  Out: m, v, p updated; maxima via am / av.  APX: the tolerance mode
// of the parameter update.
template <bool APX = false>
__device__ __forceinline__ void update_pair(const UConsts2& k, f2 g, f2& p, f2 m0, f2 v0, f2& m, f2& v, float& am,
                                            float& av) {
  m = lerp_pair(k, g, m0, am);
  v = f2_fma(k.omb2, f2_mul(g, g), f2_mul(v0, k.beta2));       // mul_ then addcmul_
  float va, vb;
  f2_unpack(v, va, vb);
  av = fmaxf(av, fmaxf(va, vb));
  if (APX) param_pair_apx(k, p, m, v);
  else param_pair(k, p, m, v);
}

// Host side: the constants of one step.
static inline UConsts make_consts(double beta1, double beta2, double lr, double wd, double eps, double step) {
  UConsts c;
  const double bc1 = 1.0 - pow(beta1, step);
  const double bc2 = 1.0 - pow(beta2, step);
  const double step_size = lr / bc1;
  c.wd_mul = (float)(1.0 - lr * wd);
  c.lerp_w = (float)(1.0 - beta1);
  c.lerp_omw = 1.0f - c.lerp_w;
  c.lerp_small = fabsf(c.lerp_w) < 0.5f;
  c.beta2 = (float)beta2;
  c.omb2 = (float)(1.0 - beta2);
  c.bc2s = (float)sqrt(bc2);
  c.inv_bc2s = (float)(1.0 / sqrt(bc2));  // torch divides by a host scalar as x * float(1.0 / s)
  c.eps = (float)eps;
  c.alpha = (float)(-step_size);
  // eps * sqrt(bc2) >= 2^-37: the square root of a denormal second moment (below 2^-63, where the short sequence is
  // far off) times 1 / sqrt(bc2) stays under half a unit in the last place of eps: the denominator is eps either way
  c.fast = (eps >= 0x1p-40 && eps <= 0x1p30 && bc2 >= 0x1p-40 && eps * sqrt(bc2) >= 0x1p-37);
  // fused-kernel flavour: everything a float, as the reference's binding passes it
  c.f_beta1 = (float)beta1;
  c.f_beta2 = (float)beta2;
  c.f_omb1 = 1.0f - c.f_beta1;
  c.f_omb2 = 1.0f - c.f_beta2;
  c.f_lr = (float)lr;
  c.f_wd = (float)wd;
  c.f_eps = (float)eps;
  c.f_step = (float)step;
  c.c1 = c.c2s = c.rc2s = 0.0f;
  // the short sequences need the denominator, at least eps * (1 - beta1), inside [2^-60, 2^60]
  c.f_fast = (c.f_beta1 >= 0.0f && c.f_beta1 < 1.0f && c.f_beta2 >= 0.0f && c.f_beta2 < 1.0f && c.f_step >= 1.0f &&
              (double)c.f_eps * (1.0 - (double)c.f_beta1) >= 0x1p-50 && c.f_eps <= 0x1p30f &&
              sqrt(1.0 - (double)c.f_beta2) >= 0x1p-20 &&
              (double)c.f_eps * sqrt(1.0 - (double)c.f_beta2) >= 0x1p-37);
  return c;
}

}  // namespace lpmm_b200
