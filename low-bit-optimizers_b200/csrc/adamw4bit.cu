// Fused 4-bit AdamW step for sm_100a: one pass over p, g, packed m/v codes and group scales.
//
// Arithmetic follows the reference kernels (lpmm/cpp_extension/fused_adamw_kernel.cu:81-174 for
// 4-bit states, :52-78 for fp32 states) operation by operation, with every rounding spelled out
// as an intrinsic so the compiler cannot re-associate or re-contract it:
//   m  = fma(beta1, qmap_m[code]*scale_m, (1-beta1)*g)
//   v  = fma(beta2, qmap_v[code]*scale_v, ((1-beta2)*g)*g)
//   d  = (sqrt(v)/c2s + eps) * c1 ;  p = fma(-lr, fma(wd, p, m/d), p)
//   new scale = group max of |m| (resp. v); new code = nearest-code rule on m/scale.
// These are the contractions nvcc's default -fmad=true makes of the reference's expressions;
// the choice was settled against the outputs of the reference binary itself.
//
// Work decomposition is new.  A 128-element group is owned by a half-warp (16 lanes x 8
// elements).  Each lane moves its 8 p and g values with one 256-bit access and its 8 codes per
// moment with one 32-bit access.  Dequantization is a shuffle: lane i of the half-warp holds
// qmap[i]*scale, and element k reads it from lane `code`.  Group maxima are four-step shuffle
// reductions.  Normalisation by the group maximum is a correctly rounded division done with a
// shared reciprocal and an FMA residual.  Requantization is one shared-memory table read and one
// compare per element (first moment) or a closed form (second moment, linear map).  One launch
// walks the whole parameter list (or a ZeRO-1 shard of it) through a descriptor table carried
// in the kernel parameters.
#include <math.h>

#include "common.cuh"
#include "fused_x2.cuh"
#include "multi_tensor.cuh"

namespace lpmm_b200 {

constexpr size_t DYN_SMEM = 2 * LUT_ENTRIES * sizeof(LutEnt);  // one table per moment

struct Consts {
  float beta1, beta2, omb1, omb2, lr, wd, eps, c1;
  float c2s, rc2s;  // sqrt(1 - beta2^step) and its correctly rounded reciprocal
};

// Peers of a ZeRO-1 step: byte offsets from an address in this GPU's flat parameter buffer to the
// same element in each peer's buffer (peer-mapped memory).  Every updated parameter is stored
// locally and at each of these offsets, so the all-gather happens inside the update kernel,
// group by group, over NVLink.
struct PeerInfo {
  int n;
  long long off[7];
  // Gradient reduction inside the same kernel: when gn > 0 the gradient of an element is the sum, in
  // rank order, of the values at the gn byte offsets goff[] from its address in this GPU's gradient
  // buffer (offset 0 = this GPU's own copy), times gscale.  Each rank reads the gradients of its own
  // group range from every peer over NVLink: the reduce-scatter of ZeRO-1 happens in the update kernel.
  int gn;
  float gscale;
  long long goff[8];
};
// PEERS false (single-GPU instantiations): plain loads, no trace of the above in the code.
template <bool PEERS>
__device__ __forceinline__ float load_g1(const float* a, const PeerInfo& pi) {
  if (!PEERS || pi.gn == 0) return *a;
  float s = *reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[0]);
  for (int i = 1; i < pi.gn; ++i)
    s = __fadd_rn(s, *reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[i]));
  return __fmul_rn(s, pi.gscale);
}
template <bool PEERS>
__device__ __forceinline__ f8 load_g8(const float* a, const PeerInfo& pi) {
  if (!PEERS || pi.gn == 0) return ldg_f8(a);
  f8 s = ldg_f8(reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[0]));
  for (int i = 1; i < pi.gn; ++i) {
    const f8 x = ldg_f8(reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[i]));
#pragma unroll
    for (int k = 0; k < 8; ++k) s.x[k] = __fadd_rn(s.x[k], x.x[k]);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) s.x[k] = __fmul_rn(s.x[k], pi.gscale);
  return s;
}
__device__ __forceinline__ f2x4 load_g2x4(const float* a, const PeerInfo& pi) {
  f2x4 s = ldg_f2x4(reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[0]));
  for (int i = 1; i < pi.gn; ++i) {
    const f2x4 x = ldg_f2x4(reinterpret_cast<const float*>(reinterpret_cast<const char*>(a) + pi.goff[i]));
#pragma unroll
    for (int j = 0; j < 4; ++j) s.v[j] = f2_add(s.v[j], x.v[j]);
  }
  const f2 sc = f2_splat(pi.gscale);
#pragma unroll
  for (int j = 0; j < 4; ++j) s.v[j] = f2_mul(s.v[j], sc);
  return s;
}
__device__ __forceinline__ void peer_store1(float* addr, float val, const PeerInfo& pi) {
  for (int i = 0; i < pi.n; ++i) *reinterpret_cast<float*>(reinterpret_cast<char*>(addr) + pi.off[i]) = val;
}

__device__ __forceinline__ float upd_m(const Consts& c, float m0, float g) {
  return __fmaf_rn(c.beta1, m0, __fmul_rn(c.omb1, g));
}
__device__ __forceinline__ float upd_v(const Consts& c, float v0, float g) {
  return __fmaf_rn(c.beta2, v0, __fmul_rn(__fmul_rn(c.omb2, g), g));
}
// FAST: the short sqrt/division sequences of common.cuh; the host selects it only when eps and
// beta1 keep the denominator inside their checked domain.
template <bool FAST>
__device__ __forceinline__ float upd_p(const Consts& c, float p, float m, float v) {
  float d;
  if (FAST) d = udiv(sqrt_rn_fast(v), c.c2s, c.rc2s);
  else d = __fdiv_rn(__fsqrt_rn(v), c.c2s);
  d = __fmul_rn(__fadd_rn(d, c.eps), c.c1);
  const float q = FAST ? div_rn_fast(m, d) : __fdiv_rn(m, d);
  const float u = __fmaf_rn(c.wd, p, q);
  return __fmaf_rn(-c.lr, u, p);
}

// Any 4-bit group, any alignment, any map: scalar accesses predicated on numel
// (fused_adamw_kernel.cu:114,130-143,160-165), IEEE sqrt and division, the reference's search.
// The fast path falls back to this before it has stored anything.
template <bool PEERS>
__device__ __noinline__ void group_q4_generic(const TDesc& t, long long gl, int l16, unsigned hmask,
                                              const Consts& c, const QMapSmem& Sm, const QMapSmem& Sv,
                                              const PeerInfo& pi) {
  const long long e0 = gl * 128 + l16 * 8;
  const long long n = t.numel;
  uint8_t* mb = reinterpret_cast<uint8_t*>(t.m) + (e0 >> 1);
  uint8_t* vb = reinterpret_cast<uint8_t*>(t.v) + (e0 >> 1);
  const float sm = t.sm[gl];
  const float sv = t.sv[gl];
  float m[8], v[8];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    m[k] = 0.0f;
    v[k] = 0.0f;
    if (e0 + k < n) {
      const uint8_t mbyte = mb[k >> 1], vbyte = vb[k >> 1];
      const float g = load_g1<PEERS>(t.g + e0 + k, pi);
      const float m0 = __fmul_rn(Sm.qmap[(mbyte >> (4 * (k & 1))) & 15u], sm);
      const float v0 = __fmul_rn(Sv.qmap[(vbyte >> (4 * (k & 1))) & 15u], sv);
      m[k] = upd_m(c, m0, g);
      v[k] = upd_v(c, v0, g);
      const float pn = upd_p<false>(c, t.p[e0 + k], m[k], v[k]);
      t.p[e0 + k] = pn;
      peer_store1(t.p + e0 + k, pn, pi);
      am = fmaxf(am, fabsf(m[k]));
      av = fmaxf(av, v[k]);
    }
  }
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (e0 + 2 * j < n) {
      uint32_t mo = bsearch_code(Sm.qmap, __fdiv_rn(m[2 * j], am)) & 15;
      uint32_t vo = bsearch_code(Sv.qmap, __fdiv_rn(v[2 * j], av)) & 15;
      if (e0 + 2 * j + 1 < n) {
        mo |= (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(m[2 * j + 1], am)) & 15) << 4;
        vo |= (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(v[2 * j + 1], av)) & 15) << 4;
      }
      mb[j] = (uint8_t)mo;
      vb[j] = (uint8_t)vo;
    }
  }
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

// Codes of one lane's 8 elements with IEEE division and the reference's search; used when a
// group's scale lies outside the domain of the shared-reciprocal division.
__device__ __noinline__ uint2 quant8_exact(const QMapSmem& Sm, const QMapSmem& Sv, float am, float av, float m0,
                                           float m1, float m2, float m3, float m4, float m5, float m6, float m7,
                                           float v0, float v1, float v2, float v3, float v4, float v5, float v6,
                                           float v7) {
  const float m[8] = {m0, m1, m2, m3, m4, m5, m6, m7};
  const float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  uint2 o = make_uint2(0u, 0u);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    o.x |= (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(m[k], am)) & 15) << (4 * k);
    o.y |= (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(v[k], av)) & 15) << (4 * k);
  }
  return o;
}

// Pointers of one 4-bit tensor, already offset to this lane's first element of group 0.
struct LanePtrs {
  float* p;
  const float* g;
  uint32_t* mc;
  uint32_t* vc;
  float* sm;
  float* sv;
};

// One full, aligned 4-bit group: lane owns elements [8*l16, 8*l16+8) of group gl.
// qm_l / qv_l: this lane's entry of the two maps (qmap[l16]).  pf: how many groups ahead this
// half-warp's next group lies (0 = none); its lines are requested into L2 now.
template <bool FAST, bool VLIN, bool PEERS>
__device__ __forceinline__ void group_q4_fast(const LanePtrs& t, unsigned gl, int l16, unsigned hmask,
                                              const Consts& c, const QMapSmem& Sm, const QMapSmem& Sv,
                                              const LutEnt* __restrict__ lut_m, const LutEnt* __restrict__ lut_v,
                                              float qm_l, float qv_l, unsigned pf, const PeerInfo& pi) {
  float* pp = t.p + (size_t)gl * 128;
  const float* gp = t.g + (size_t)gl * 128;
  uint32_t* mcp = t.mc + (size_t)gl * 16;
  uint32_t* vcp = t.vc + (size_t)gl * 16;
  f8 p = ldg_f8(pp);
  const f8 g = load_g8<PEERS>(gp, pi);
  const uint32_t mc = *mcp;
  const uint32_t vc = *vcp;
  const float pm = __fmul_rn(qm_l, t.sm[gl]);  // lane i: qmap_m[i] * scale
  const float pv = __fmul_rn(qv_l, t.sv[gl]);
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 128);
    prefetch_l2(gp + (size_t)pf * 128);
    prefetch_l2(mcp + (size_t)pf * 16);
    prefetch_l2(vcp + (size_t)pf * 16);
  }

  float m[8], v[8];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float m0 = __shfl_sync(hmask, pm, (int)(mc >> (4 * k)), 16);  // source lane = code (mod 16)
    const float v0 = __shfl_sync(hmask, pv, (int)(vc >> (4 * k)), 16);
    m[k] = upd_m(c, m0, g.x[k]);
    v[k] = upd_v(c, v0, g.x[k]);
    p.x[k] = upd_p<FAST>(c, p.x[k], m[k], v[k]);
    am = fmaxf(am, fabsf(m[k]));
    av = fmaxf(av, v[k]);
  }
  stg_f8(pp, p);
  for (int i = 0; i < pi.n; ++i) stg_f8(reinterpret_cast<float*>(reinterpret_cast<char*>(pp) + pi.off[i]), p);
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
  uint32_t mo = 0, vo = 0;
  if (udiv_ok(am) && udiv_ok(av)) {
    const float rm = rcp_nr(am), rv = rcp_nr(av);
#pragma unroll
    for (int k = 7; k >= 0; --k) {
      const float xm = udiv(m[k], am, rm);
      const float xv = udiv(v[k], av, rv);
      mo = (mo << 4) + (uint32_t)lut_code(lut_m, xm);
      if (VLIN) vo = vo * 16u + linear16_code(xv);
      else vo = (vo << 4) + (uint32_t)lut_code(lut_v, xv);
    }
    if (am == 0.0f) mo = 0xFFFFFFFFu;          // 0/0 = NaN -> code 15 for the whole group
    if (av == 0.0f) vo = 0xFFFFFFFFu;
  } else {  // scales outside the shared-reciprocal domain
    const uint2 o = quant8_exact(Sm, Sv, am, av, m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], v[0], v[1], v[2],
                                 v[3], v[4], v[5], v[6], v[7]);
    mo = o.x;
    vo = o.y;
  }
  *mcp = mo;
  *vcp = vo;
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

// The same group update written with packed fp32x2 instructions: elements (2j, 2j+1) of a lane share
// every multiply / add / fma, each half rounding exactly like the scalar instruction, so results
// are bit-identical to group_q4_fast<true, VLIN>.  Uses the short sqrt/division sequences, so it is
// selected only where those are (FAST).
// APX: the tolerance mode of the parameter update (fused_x2.cuh); moments, maxima and codes unchanged.
template <bool VLIN, bool PEERS, bool APX>
__device__ __forceinline__ void group_q4_x2(const LanePtrs& t, unsigned gl, int l16, unsigned hmask,
                                            const Consts2& c, const QMapSmem& Sm, const QMapSmem& Sv,
                                            const LutEnt* __restrict__ lut_m, const LutEnt* __restrict__ lut_v,
                                            float qm_l, float qv_l, unsigned pf, const PeerInfo& pi) {
  float* pp = t.p + (size_t)gl * 128;
  const float* gp = t.g + (size_t)gl * 128;
  uint32_t* mcp = t.mc + (size_t)gl * 16;
  uint32_t* vcp = t.vc + (size_t)gl * 16;
  f2x4 p = ldg_f2x4(pp);
  const f2x4 g = (PEERS && pi.gn > 0) ? load_g2x4(gp, pi) : ldg_f2x4(gp);
  const uint32_t mc = *mcp;
  const uint32_t vc = *vcp;
  const float pm = __fmul_rn(qm_l, t.sm[gl]);  // lane i: qmap_m[i] * scale
  const float pv = __fmul_rn(qv_l, t.sv[gl]);
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 128);
    prefetch_l2(gp + (size_t)pf * 128);
    prefetch_l2(mcp + (size_t)pf * 16);
    prefetch_l2(vcp + (size_t)pf * 16);
  }
  f2 m[4], v[4];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float m0a = __shfl_sync(hmask, pm, (int)(mc >> (8 * j)), 16);  // source lane = code (mod 16)
    const float m0b = __shfl_sync(hmask, pm, (int)(mc >> (8 * j + 4)), 16);
    const float v0a = __shfl_sync(hmask, pv, (int)(vc >> (8 * j)), 16);
    const float v0b = __shfl_sync(hmask, pv, (int)(vc >> (8 * j + 4)), 16);
    p.v[j] = fused_pair_x2<APX>(c, g.v[j], p.v[j], f2_pack(m0a, m0b), f2_pack(v0a, v0b), m[j], v[j], am, av);
  }
  stg_f2x4(pp, p);
  if (PEERS) {
    for (int i = 0; i < pi.n; ++i) stg_f2x4(reinterpret_cast<float*>(reinterpret_cast<char*>(pp) + pi.off[i]), p);
  }
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
  uint32_t mo = 0, vo = 0;
  if (udiv_ok(am) && udiv_ok(av)) {
    requant_x2<VLIN>(c, m, v, am, av, lut_m, lut_v, mo, vo);
  } else {  // scales outside the shared-reciprocal domain
    float mm[8], vv[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f2_unpack(m[j], mm[2 * j], mm[2 * j + 1]);
      f2_unpack(v[j], vv[2 * j], vv[2 * j + 1]);
    }
    const uint2 o = quant8_exact(Sm, Sv, am, av, mm[0], mm[1], mm[2], mm[3], mm[4], mm[5], mm[6], mm[7], vv[0],
                                 vv[1], vv[2], vv[3], vv[4], vv[5], vv[6], vv[7]);
    mo = o.x;
    vo = o.y;
  }
  *mcp = mo;
  *vcp = vo;
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

// fp32-state tensors (the numel <= threshold fallback), 128 elements per half-warp step.
template <bool FAST, bool PEERS>
__device__ __forceinline__ void group_fp32(const TDesc& t, long long gl, int l16, const Consts& c, const PeerInfo& pi) {
  const long long e0 = gl * 128 + l16 * 8;
  float* mp = reinterpret_cast<float*>(t.m);
  float* vp = reinterpret_cast<float*>(t.v);
  if (t.aligned && (gl + 1) * 128 <= t.numel) {
    f8 p = ldg_f8(t.p + e0);
    const f8 g = load_g8<PEERS>(t.g + e0, pi);
    f8 m = ldg_f8(mp + e0);
    f8 v = ldg_f8(vp + e0);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      m.x[k] = upd_m(c, m.x[k], g.x[k]);
      v.x[k] = upd_v(c, v.x[k], g.x[k]);
      p.x[k] = upd_p<FAST>(c, p.x[k], m.x[k], v.x[k]);
    }
    stg_f8(mp + e0, m);
    stg_f8(vp + e0, v);
    stg_f8(t.p + e0, p);
    for (int i = 0; i < pi.n; ++i) stg_f8(reinterpret_cast<float*>(reinterpret_cast<char*>(t.p + e0) + pi.off[i]), p);
  } else {
    for (int k = 0; k < 8; ++k) {
      const long long e = e0 + k;
      if (e < t.numel) {
        const float g = load_g1<PEERS>(t.g + e, pi);
        const float m = upd_m(c, mp[e], g);
        const float v = upd_v(c, vp[e], g);
        mp[e] = m;
        vp[e] = v;
        const float pn = upd_p<false>(c, t.p[e], m, v);
        t.p[e] = pn;
        peer_store1(t.p + e, pn, pi);
      }
    }
  }
}

// The tensor loop is uniform across the CTA (descriptor fields come from the launch parameters
// through uniform loads); each half-warp walks its own arithmetic progression of global group
// indices gi = gbeg + id, gbeg + id + stride, ... through the tensors in order.
// MATH: 0 = IEEE sqrt / division, 1 = the short exact sequences (same results), 2 = as 1 with the tolerance-mode
// parameter update on full aligned 4-bit groups.
template <int MATH, bool VLIN, bool PEERS>
__device__ __forceinline__ void run_groups(const Table& tab, const Consts& c, const QMapSmem& Sm,
                                           const QMapSmem& Sv, const LutEnt* lut_m, const LutEnt* lut_v,
                                           bool tables_ok, long long gbeg, long long gend, const PeerInfo& pi) {
  constexpr bool FAST = MATH >= 1;
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = gbeg + (long long)blockIdx.x * HW_PER_CTA + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * HW_PER_CTA;
  const float qm_l = Sm.qmap[l16], qv_l = Sv.qmap[l16];
  int ti = 0;
  while (ti + 1 < tab.n && tab.t[ti + 1].gstart <= gbeg) ++ti;
  for (; ti < tab.n; ++ti) {
    const TDesc& t = tab.t[ti];
    const long long tstart = t.gstart;
    if (tstart >= gend) break;
    long long tend = (ti + 1 < tab.n) ? tab.t[ti + 1].gstart : tab.gtotal;
    if (tend > gend) tend = gend;
    if (t.kind == LPMM_B200_KIND_Q4) {
      if (tables_ok && t.aligned) {
        long long fend = tstart + t.numel / 128;  // end of the full groups
        if (fend > tend) fend = tend;
        if (gi < fend) {
          LanePtrs lp;
          lp.p = t.p + l16 * 8;
          lp.g = t.g + l16 * 8;
          lp.mc = reinterpret_cast<uint32_t*>(t.m) + l16;
          lp.vc = reinterpret_cast<uint32_t*>(t.v) + l16;
          lp.sm = t.sm;
          lp.sv = t.sv;
          unsigned gl = (unsigned)(gi - tstart);           // groups per tensor fit 32 bits (host-checked)
          const unsigned lim = (unsigned)(fend - tstart);
          const unsigned st = (unsigned)stride;
          if (FAST) {
            const Consts2 c2 = make_consts_x2(c.beta1, c.beta2, c.omb1, c.omb2, c.lr, c.wd, c.eps, c.c1, c.c2s, c.rc2s);
            for (; gl < lim; gl += st)
              group_q4_x2<VLIN, PEERS, MATH == 2>(lp, gl, l16, hmask, c2, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                       (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u, pi);
          } else {
            for (; gl < lim; gl += st)
              group_q4_fast<FAST, VLIN, PEERS>(lp, gl, l16, hmask, c, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                        (gl + st < lim) ? st : 0u, pi);
          }
          gi = tstart + gl;
        }
      }
      for (; gi < tend; gi += stride) group_q4_generic<PEERS>(t, gi - tstart, l16, hmask, c, Sm, Sv, pi);
    } else {
      for (; gi < tend; gi += stride) group_fp32<FAST, PEERS>(t, gi - tstart, l16, c, pi);
    }
  }
}

template <bool HAS_Q4, int MATH, bool PEERS>
__global__ void __launch_bounds__(CTA_THREADS, CTAS_PER_SM)
adamw4bit_multi_kernel(const __grid_constant__ Table tab, const float* __restrict__ qmap_m,
                       const float* __restrict__ qmap_v, const lpmm_b200_hyper h, long long gbeg, long long gend,
                       const PeerInfo pi) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm, Sv;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  LutEnt* lut_v = lut_m + LUT_ENTRIES;
  bool vlin = true, tables_ok = true;
  if (HAS_Q4) {
    lut_build(Sv, nullptr, qmap_v);  // learn whether the second-moment map is the linear one
    vlin = Sv.linear16 != 0;
    if (!vlin) lut_build(Sv, lut_v, qmap_v);
    lut_build(Sm, lut_m, qmap_m);
    tables_ok = Sm.valid && Sv.valid;
  }
  Consts c;
  c.beta1 = h.beta1;
  c.beta2 = h.beta2;
  c.omb1 = __fsub_rn(1.0f, h.beta1);
  c.omb2 = __fsub_rn(1.0f, h.beta2);
  c.lr = h.lr;
  c.wd = h.weight_decay;
  c.eps = h.eps;
  c.c1 = __fsub_rn(1.0f, powf(h.beta1, h.step));
  c.c2s = __fsqrt_rn(__fsub_rn(1.0f, powf(h.beta2, h.step)));
  c.rc2s = __frcp_rn(c.c2s);
  if (vlin) run_groups<MATH, true, PEERS>(tab, c, Sm, Sv, lut_m, lut_v, tables_ok, gbeg, gend, pi);
  else run_groups<MATH, false, PEERS>(tab, c, Sm, Sv, lut_m, lut_v, tables_ok, gbeg, gend, pi);
}

__global__ void bias_corrections_kernel(float beta1, float beta2, float step, float* out) {
  out[0] = __fsub_rn(1.0f, powf(beta1, step));
  out[1] = __fsqrt_rn(__fsub_rn(1.0f, powf(beta2, step)));
}

// The short sqrt/division sequences are exact for denominators in [2^-60, 2^60]; the denominator
// is at least eps * (1 - beta1^step) >= eps * (1 - beta1).
static bool fast_math_ok(const lpmm_b200_hyper& h) {
  if (!(h.beta1 >= 0.0f && h.beta1 < 1.0f && h.beta2 >= 0.0f && h.beta2 < 1.0f && h.step >= 1.0f)) return false;
  const double dmin = (double)h.eps * (1.0 - (double)h.beta1);
  const double c2s_min = sqrt(1.0 - (double)h.beta2);
  // eps * c2s >= 2^-37: the square root of a denormal second moment (below 2^-63, where the short sequence is far
  // off) divided by c2s stays under half a unit in the last place of eps, so the denominator is eps either way
  return dmin >= 0x1p-50 && h.eps <= 0x1p30f && c2s_min >= 0x1p-20 && (double)h.eps * c2s_min >= 0x1p-37;
}
// The tolerance-mode parameter update folds 1 / -lr into its constants.
static bool approx_math_ok(const lpmm_b200_hyper& h) {
  return fast_math_ok(h) && h.lr >= 0x1p-60f && h.lr <= 0x1p30f && h.weight_decay <= 0x1p30f;
}

template <bool HAS_Q4, int MATH, bool PEERS>
static cudaError_t launch_one(const Table& tab, unsigned grid, const float* qm, const float* qv,
                              const lpmm_b200_hyper& h, long long lo, long long hi, cudaStream_t st,
                              const PeerInfo& pi) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = HAS_Q4 ? DYN_SMEM : 0;
  if (HAS_Q4 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(adamw4bit_multi_kernel<HAS_Q4, MATH, PEERS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DYN_SMEM);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  adamw4bit_multi_kernel<HAS_Q4, MATH, PEERS><<<grid, CTA_THREADS, smem, st>>>(tab, qm, qv, h, lo, hi, pi);
  return cudaGetLastError();
}

template <bool HAS_Q4, bool PEERS>
static cudaError_t launch_fast_or_exact(int math, const Table& tab, unsigned grid, const float* qm, const float* qv,
                                        const lpmm_b200_hyper& h, long long lo, long long hi, cudaStream_t st,
                                        const PeerInfo& pi) {
  if (math == 2 && HAS_Q4) return launch_one<HAS_Q4, HAS_Q4 ? 2 : 1, PEERS>(tab, grid, qm, qv, h, lo, hi, st, pi);
  return math ? launch_one<HAS_Q4, 1, PEERS>(tab, grid, qm, qv, h, lo, hi, st, pi)
              : launch_one<HAS_Q4, 0, PEERS>(tab, grid, qm, qv, h, lo, hi, st, pi);
}

static int launch_multi(const lpmm_b200_tensor* ts, int n, const float* qm, const float* qv,
                        const lpmm_b200_hyper& h, int64_t gbeg, int64_t gend, cudaStream_t st,
                        const PeerInfo& pi = PeerInfo{}, uint32_t flags = 0) {
  // `ts` may hold more than MAX_TENSORS entries: walk it in windows, each window one launch over
  // the part of [gbeg, gend) that falls inside it.
  static thread_local Table tab;  // 28.9 KB; copied into the launch parameters by the runtime
  const int fast = ((flags & LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) && approx_math_ok(h)) ? 2 : (fast_math_ok(h) ? 1 : 0);
  int64_t gcursor = 0;
  int i = 0;
  while (i < n) {
    const Window w = next_window(ts, n, i, gcursor, gbeg, gend, true, tab);
    if (!w.work) continue;
    const unsigned grid = multi_grid(w);
    cudaError_t e;
    if (pi.n > 0 || pi.gn > 0)
      e = w.any_q4 ? launch_fast_or_exact<true, true>(fast, tab, grid, qm, qv, h, w.lo, w.hi, st, pi)
                   : launch_fast_or_exact<false, true>(fast, tab, grid, qm, qv, h, w.lo, w.hi, st, pi);
    else
      e = w.any_q4 ? launch_fast_or_exact<true, false>(fast, tab, grid, qm, qv, h, w.lo, w.hi, st, pi)
                   : launch_fast_or_exact<false, false>(fast, tab, grid, qm, qv, h, w.lo, w.hi, st, pi);
    LPMM_CUDA_TRY(e);
  }
  return LPMM_B200_OK;
}

static int check_list(const lpmm_b200_tensor* ts, int n, bool need_qmaps, const float* qm, const float* qv) {
  bool any_q4 = false;
  int64_t total = 0;
  const int rc = check_tensor_list(ts, n, true, &any_q4, &total);
  if (rc != LPMM_B200_OK) return rc;
  if ((any_q4 || need_qmaps) && (!qm || !qv)) return LPMM_B200_ERR_NULL_POINTER;
  return LPMM_B200_OK;
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

extern "C" int64_t lpmm_b200_count_groups(const lpmm_b200_tensor* tensors, int n_tensors) {
  if (n_tensors < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (n_tensors > 0 && !tensors) return LPMM_B200_ERR_NULL_POINTER;
  int64_t g = 0;
  for (int i = 0; i < n_tensors; ++i) {
    if (tensors[i].numel < 0) return LPMM_B200_ERR_BAD_SIZE;
    g += groups_of(tensors[i].numel);
  }
  return g;
}

// Range checks shared by the list entry points; on success *run tells whether anything is to be launched.
static int check_range(const lpmm_b200_tensor* tensors, int n_tensors, const float* qm, const float* qv,
                       int64_t group_begin, int64_t* group_end, uint32_t flags, bool* run) {
  *run = false;
  if (flags & ~(uint32_t)LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) return LPMM_B200_ERR_BAD_KIND;
  int rc = check_list(tensors, n_tensors, false, qm, qv);
  if (rc != LPMM_B200_OK) return rc;
  const int64_t total = lpmm_b200_count_groups(tensors, n_tensors);
  if (*group_end < 0) *group_end = total;
  if (group_begin < 0 || group_begin > *group_end || *group_end > total) return LPMM_B200_ERR_BAD_SIZE;
  *run = group_begin != *group_end;
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_flags(const lpmm_b200_tensor* tensors, int n_tensors,
                                                      const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                      lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                      uint32_t flags, void* stream) {
  bool run;
  const int rc = check_range(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, group_begin, &group_end, flags, &run);
  if (rc != LPMM_B200_OK || !run) return rc;
  return launch_multi(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, hyper, group_begin, group_end,
                      (cudaStream_t)stream, PeerInfo{}, flags);
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor(const lpmm_b200_tensor* tensors, int n_tensors,
                                                const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                void* stream) {
  return lpmm_b200_adamw4bit_multi_tensor_flags(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, hyper, group_begin,
                                                group_end, 0u, stream);
}

extern "C" int lpmm_b200_adamw4bit_single_tensor(float* p, const float* g, int8_t* exp_avg, int8_t* exp_avg_sq,
                                                 float* exp_avg_scale, float* exp_avg_sq_scale,
                                                 const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                 float beta1, float beta2, float lr, float weight_decay, float eps,
                                                 float step, int64_t numel, void* stream) {
  lpmm_b200_tensor t;
  t.p = p;
  t.g = g;
  t.m = exp_avg;
  t.v = exp_avg_sq;
  t.m_scale = exp_avg_scale;
  t.v_scale = exp_avg_sq_scale;
  t.numel = numel;
  t.kind = LPMM_B200_KIND_Q4;
  t.reserved = 0;
  const lpmm_b200_hyper h = {beta1, beta2, lr, weight_decay, eps, step};
  int rc = check_list(&t, 1, true, exp_avg_qmap, exp_avg_sq_qmap);
  if (rc != LPMM_B200_OK) return rc;
  if (numel == 0) return LPMM_B200_OK;
  return launch_multi(&t, 1, exp_avg_qmap, exp_avg_sq_qmap, h, 0, groups_of(numel), (cudaStream_t)stream);
}

extern "C" int lpmm_b200_adamw_single_tensor(float* p, const float* g, float* exp_avg, float* exp_avg_sq,
                                             float beta1, float beta2, float lr, float weight_decay, float eps,
                                             float step, int64_t numel, void* stream) {
  lpmm_b200_tensor t;
  t.p = p;
  t.g = g;
  t.m = exp_avg;
  t.v = exp_avg_sq;
  t.m_scale = nullptr;
  t.v_scale = nullptr;
  t.numel = numel;
  t.kind = LPMM_B200_KIND_FP32;
  t.reserved = 0;
  const lpmm_b200_hyper h = {beta1, beta2, lr, weight_decay, eps, step};
  int rc = check_list(&t, 1, false, nullptr, nullptr);
  if (rc != LPMM_B200_OK) return rc;
  if (numel == 0) return LPMM_B200_OK;
  return launch_multi(&t, 1, nullptr, nullptr, h, 0, groups_of(numel), (cudaStream_t)stream);
}

extern "C" int lpmm_b200_bias_corrections(float beta1, float beta2, float step, float* out, void* stream) {
  if (!out) return LPMM_B200_ERR_NULL_POINTER;
  bias_corrections_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(beta1, beta2, step, out);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_peers_flags(const lpmm_b200_tensor* tensors, int n_tensors,
                                                            const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                            lpmm_b200_hyper hyper, int64_t group_begin,
                                                            int64_t group_end, const int64_t* peer_byte_offsets,
                                                            int n_peers, uint32_t flags, void* stream) {
  if (n_peers < 0 || n_peers > 7) return LPMM_B200_ERR_BAD_SIZE;
  if (n_peers > 0 && !peer_byte_offsets) return LPMM_B200_ERR_NULL_POINTER;
  bool run;
  const int rc = check_range(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, group_begin, &group_end, flags, &run);
  if (rc != LPMM_B200_OK || !run) return rc;
  PeerInfo pi = {};
  pi.n = n_peers;
  for (int i = 0; i < n_peers; ++i) {
    if (peer_byte_offsets[i] % 32 != 0) return LPMM_B200_ERR_BAD_SIZE;  // keeps the 256-bit stores aligned
    pi.off[i] = peer_byte_offsets[i];
  }
  return launch_multi(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, hyper, group_begin, group_end,
                      (cudaStream_t)stream, pi, flags);
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_peers(const lpmm_b200_tensor* tensors, int n_tensors,
                                                      const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                      lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                      const int64_t* peer_byte_offsets, int n_peers, void* stream) {
  return lpmm_b200_adamw4bit_multi_tensor_peers_flags(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, hyper,
                                                      group_begin, group_end, peer_byte_offsets, n_peers, 0u, stream);
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_zero1(const lpmm_b200_tensor* tensors, int n_tensors,
                                                      const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                      lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                      const int64_t* peer_byte_offsets, int n_peers,
                                                      const int64_t* grad_byte_offsets, int n_grads, float grad_scale,
                                                      void* stream) {
  if (n_peers < 0 || n_peers > 7 || n_grads < 0 || n_grads > 8) return LPMM_B200_ERR_BAD_SIZE;
  if ((n_peers > 0 && !peer_byte_offsets) || (n_grads > 0 && !grad_byte_offsets)) return LPMM_B200_ERR_NULL_POINTER;
  int rc = check_list(tensors, n_tensors, false, exp_avg_qmap, exp_avg_sq_qmap);
  if (rc != LPMM_B200_OK) return rc;
  const int64_t total = lpmm_b200_count_groups(tensors, n_tensors);
  if (group_end < 0) group_end = total;
  if (group_begin < 0 || group_begin > group_end || group_end > total) return LPMM_B200_ERR_BAD_SIZE;
  if (group_begin == group_end) return LPMM_B200_OK;
  PeerInfo pi = {};
  pi.n = n_peers;
  for (int i = 0; i < n_peers; ++i) {
    if (peer_byte_offsets[i] % 32 != 0) return LPMM_B200_ERR_BAD_SIZE;  // keeps the 256-bit stores aligned
    pi.off[i] = peer_byte_offsets[i];
  }
  pi.gn = n_grads;
  pi.gscale = grad_scale;
  for (int i = 0; i < n_grads; ++i) {
    if (grad_byte_offsets[i] % 32 != 0) return LPMM_B200_ERR_BAD_SIZE;  // keeps the 256-bit loads aligned
    pi.goff[i] = grad_byte_offsets[i];
  }
  return launch_multi(tensors, n_tensors, exp_avg_qmap, exp_avg_sq_qmap, hyper, group_begin, group_end,
                      (cudaStream_t)stream, pi);
}
