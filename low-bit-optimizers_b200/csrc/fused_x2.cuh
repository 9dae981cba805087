// The fused kernel's arithmetic (lpmm/cpp_extension/fused_adamw_kernel.cu:103-128) for two elements per
// instruction (sm_100 packed fp32: each half is the IEEE result of the scalar instruction), shared by the
// fp32 and the 16-bit multi-tensor kernels.  Uses the short exact sqrt / division sequences of common.cuh,
// so callers select it only where the hyper-parameters keep the denominator inside their domain.
#pragma once
#include "common.cuh"

namespace lpmm_b200 {

struct Consts2 {
  f2 beta1, beta2, omb1, omb2, wd, nlr, eps, nc1, nc2s, rc2s, half, mone, one, k16, km15;
  // tolerance-mode parameter update (fused_pair_x2<true>): -lr / d = 1 / (sqrt(v) * apx_a + apx_b),
  // apx_a = c1 / (c2s * -lr), apx_b = eps * c1 / -lr;  p' = p + fma(apx_w, p, m * (-lr / d)), apx_w = -lr * wd
  f2 apx_a, apx_b, apx_w;
};

// beta1, beta2, omb1 = 1 - beta1, omb2 = 1 - beta2 (float subtraction), lr, wd, eps, c1 = 1 - beta1^t,
// c2s = sqrt(1 - beta2^t), rc2s = RN(1 / c2s).
__device__ __forceinline__ Consts2 make_consts_x2(float beta1, float beta2, float omb1, float omb2, float lr, float wd,
                                                  float eps, float c1, float c2s, float rc2s) {
  Consts2 k;
  k.beta1 = f2_splat(beta1);
  k.beta2 = f2_splat(beta2);
  k.omb1 = f2_splat(omb1);
  k.omb2 = f2_splat(omb2);
  k.wd = f2_splat(wd);
  k.nlr = f2_splat(-lr);
  k.eps = f2_splat(eps);
  k.nc1 = f2_splat(-c1);
  k.nc2s = f2_splat(-c2s);
  k.rc2s = f2_splat(rc2s);
  k.half = f2_splat(0.5f);
  k.mone = f2_splat(-1.0f);
  k.one = f2_splat(1.0f);
  k.k16 = f2_splat(16.0f);
  k.km15 = f2_splat(-1.5f);
  k.apx_a = f2_splat(__fdiv_rn(c1, __fmul_rn(c2s, -lr)));
  k.apx_b = f2_splat(__fdiv_rn(__fmul_rn(eps, c1), -lr));
  k.apx_w = f2_splat(__fmul_rn(-lr, wd));
  return k;
}

// One pair: new moments from the old ones and the gradient (their maxima folded into am / av), new parameter
// returned.  m = fma(b1, m0, (1-b1) g); v = fma(b2, v0, ((1-b2) g) g); d = (sqrt(v)/c2s + eps) c1;
// p' = fma(-lr, fma(wd, p, m/d), p).
// APX (the tolerance mode of the parameter update): the moments -- and with them every code and scale --
// are computed exactly as above, but the new parameter comes from the hardware's approximate square root
// and reciprocal (each within 2^-23 relative) with the constant factors folded on the host side of the
// loop: p' = p + ((-lr*wd) p + m / ((sqrt(v)/c2s + eps) c1 / -lr)), the parameter itself rounded once as in
// the exact update.  The step lr*(m/d) is then within ~4e-7 of its own size of the exact one, i.e. off by at
// most a few 1e-10 for a step of size 1e-3: the new parameter equals the exact one or its fp32 neighbour.
// Needs lr >= 2^-60 (the folded constants stay finite); callers check.
template <bool APX = false>
__device__ __forceinline__ f2 fused_pair_x2(const Consts2& c, f2 gj, f2 pj, f2 m0, f2 v0, f2& m, f2& v, float& am,
                                            float& av) {
  m = f2_fma(c.beta1, m0, f2_mul(c.omb1, gj));
  v = f2_fma(c.beta2, v0, f2_mul(f2_mul(c.omb2, gj), gj));
  float ma, mb, va, vb;
  f2_unpack(m, ma, mb);
  f2_unpack(v, va, vb);
  am = fmaxf(am, fmaxf(fabsf(ma), fabsf(mb)));
  av = fmaxf(av, fmaxf(va, vb));
  if (APX) {
    const f2 s = f2_pack(sqrt_approx(va), sqrt_approx(vb));
    float da, db;
    f2_unpack(f2_fma(s, c.apx_a, c.apx_b), da, db);
    const f2 r = f2_pack(mufu_rcp(da), mufu_rcp(db));
    // one rounding of the parameter itself, like the exact update: p + (-lr*wd*p - lr*m/d)
    return f2_add(pj, f2_fma(c.apx_w, pj, f2_mul(m, r)));
  }
  // sqrt(v): y = rsqrt(max(v, FLT_MIN)); s = v*y; s += (v - s*s) * (y/2)
  const f2 y = f2_pack(mufu_rsq(fmaxf(va, 1.17549435e-38f)), mufu_rsq(fmaxf(vb, 1.17549435e-38f)));
  f2 s = f2_mul(v, y);
  const f2 e = f2_fma(s, f2_mul(s, c.mone), v);
  s = f2_fma(e, f2_mul(c.half, y), s);
  // nd = -(s / c2s + eps) * c1  (the negated denominator: what the division's residuals need)
  f2 q = f2_mul(s, c.rc2s);
  q = f2_fma(f2_fma(q, c.nc2s, s), c.rc2s, q);
  const f2 nd = f2_mul(f2_add(q, c.eps), c.nc1);
  // m / d: r = rcp(d) refined once, quotient corrected by its exact residual
  float nda, ndb;
  f2_unpack(nd, nda, ndb);
  const f2 r0 = f2_pack(mufu_rcp(fabsf(nda)), mufu_rcp(fabsf(ndb)));
  const f2 r = f2_fma(r0, f2_fma(nd, r0, c.one), r0);
  const f2 qq = f2_mul(m, r);
  const f2 quo = f2_fma(f2_fma(nd, qq, m), r, qq);
  // p -= lr * (quo + wd * p)
  return f2_fma(c.nlr, f2_fma(c.wd, pj, quo), pj);
}

// Codes of a lane's 8 elements (4 pairs) for group maxima am, av inside the shared-reciprocal domain
// (udiv_ok): x / max by Markstein's correction, first-moment codes from the table, second-moment codes
// from the closed form of the linear map (VLIN) or its table.
template <bool VLIN>
__device__ __forceinline__ void requant_x2(const Consts2& c, const f2* m, const f2* v, float am, float av,
                                           const LutEnt* __restrict__ lut_m, const LutEnt* __restrict__ lut_v,
                                           uint32_t& mo, uint32_t& vo) {
  const float rm = rcp_nr(am), rv = rcp_nr(av);
  const f2 rm2 = f2_splat(rm), rv2 = f2_splat(rv), nam2 = f2_splat(-am), nav2 = f2_splat(-av);
  mo = 0;
  vo = 0;
#pragma unroll
  for (int j = 3; j >= 0; --j) {
    f2 xm = f2_mul(m[j], rm2);
    xm = f2_fma(f2_fma(xm, nam2, m[j]), rm2, xm);
    f2 xv = f2_mul(v[j], rv2);
    xv = f2_fma(f2_fma(xv, nav2, v[j]), rv2, xv);
    float xa, xb;
    f2_unpack(xm, xa, xb);
    mo = (mo << 4) + (uint32_t)lut_code(lut_m, xb);
    mo = (mo << 4) + (uint32_t)lut_code(lut_m, xa);
    if (VLIN) {
      float ta, tb;
      f2_unpack(f2_fma(xv, c.k16, c.km15), ta, tb);
      vo = vo * 16u + __float2uint_ru(tb);
      vo = vo * 16u + __float2uint_ru(ta);
    } else {
      f2_unpack(xv, xa, xb);
      vo = (vo << 4) + (uint32_t)lut_code(lut_v, xb);
      vo = (vo << 4) + (uint32_t)lut_code(lut_v, xa);
    }
  }
  if (am == 0.0f) mo = 0xFFFFFFFFu;  // 0/0 = NaN -> code 15 for the whole group
  if (av == 0.0f) vo = 0xFFFFFFFFu;
}

}  // namespace lpmm_b200
