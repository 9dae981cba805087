// Fused 4-bit AdamW for 16-bit parameters and gradients (bf16 or fp16), one launch for a whole list.
//
// The reference's fused kernel is instantiated for half (AT_DISPATCH_FLOATING_TYPES_AND_HALF,
// lpmm/cpp_extension/fused_adamw_kernel.cu:188,222) but cannot be reached with it: its launcher asks
// the fp32 scale tensors that lpmm/optim/adamw.py:515-521 allocates for data_ptr<Half>(), and bf16 is
// not dispatched at all.  This step defines what it would do in the obvious way: parameters and
// gradients are widened to fp32 on load (exact), the step is the fp32 fused step to the bit -- the
// arithmetic of fused_adamw_kernel.cu:103-128 with fp32 scales and codes as in adamw4bit.cu -- and the
// new parameter is rounded to nearest-even on store.  Moments, codes and scales are therefore those
// of the fp32 kernel run on the widened inputs; traffic falls from 14.06 to 8.06 bytes per parameter.
// Tensors of kind FP32 keep fp32 moments next to their 16-bit parameters.
//
// Same decomposition as adamw4bit.cu: a 128-element group is a half-warp, a lane owns 8 consecutive
// elements (one 128-bit access of parameters and of gradients, one 32-bit word of codes per moment),
// persistent 1024-thread CTAs stride over the global group sequence of the descriptor table.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"
#include "fused_x2.cuh"
#include "multi_tensor.cuh"
#include "unfused_math.cuh"

namespace lpmm_b200 {

constexpr size_t H_DYN_SMEM = 2 * LUT_ENTRIES * sizeof(LutEnt);

template <typename T>
struct Half16;
template <>
struct Half16<__nv_bfloat16> {
  static __device__ __forceinline__ float widen(unsigned short b) { return __uint_as_float((unsigned)b << 16); }
  static __device__ __forceinline__ unsigned short narrow(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
};
template <>
struct Half16<__half> {
  static __device__ __forceinline__ float widen(unsigned short b) { return __half2float(__ushort_as_half(b)); }
  static __device__ __forceinline__ unsigned short narrow(float x) { return __half_as_ushort(__float2half_rn(x)); }
};

template <typename T>
__device__ __forceinline__ void widen8(const uint4& r, float* x) {
  const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x[2 * j] = Half16<T>::widen((unsigned short)(w[j] & 0xFFFFu));
    x[2 * j + 1] = Half16<T>::widen((unsigned short)(w[j] >> 16));
  }
}
template <typename T>
__device__ __forceinline__ uint4 narrow8(const float* x) {
  unsigned w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    w[j] = (unsigned)Half16<T>::narrow(x[2 * j]) | ((unsigned)Half16<T>::narrow(x[2 * j + 1]) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Pairs: one 32-bit word holds elements (2j, 2j+1); each half widens exactly and narrows to nearest-even.
template <typename T>
__device__ __forceinline__ f2 widen2(unsigned w);
template <>
__device__ __forceinline__ f2 widen2<__nv_bfloat16>(unsigned w) {
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ f2 widen2<__half>(unsigned w) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  return f2_pack(f.x, f.y);
}
template <typename T>
__device__ __forceinline__ unsigned narrow2(f2 x);
template <>
__device__ __forceinline__ unsigned narrow2<__nv_bfloat16>(f2 x) {
  float lo, hi;
  f2_unpack(x, lo, hi);
  const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&r);
}
template <>
__device__ __forceinline__ unsigned narrow2<__half>(f2 x) {
  float lo, hi;
  f2_unpack(x, lo, hi);
  const __half2 r = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&r);
}

// One full, aligned 4-bit group with packed fp32x2 instructions: elements (2j, 2j+1) share every
// multiply / add / fma, each half rounding like the scalar instruction, so the results are those of
// h_group_fast with the short sqrt / division sequences (selected only where those apply).
// APX: the tolerance mode of the parameter update (fused_x2.cuh); moments, maxima and codes unchanged.
template <typename T, bool VLIN, bool APX, bool PEERS>
__device__ __forceinline__ void h_group_x2(const TDesc& t, unsigned gl, int l16, unsigned hmask, const Consts2& c,
                                           const QMapSmem& Sm, const QMapSmem& Sv, const LutEnt* __restrict__ lut_m,
                                           const LutEnt* __restrict__ lut_v, float qm_l, float qv_l, unsigned pf,
                                           const PeerStores& ps) {
  const size_t e0 = (size_t)gl * 128 + (size_t)l16 * 8;
  uint4* pp = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(t.p) + e0);
  const uint4* gp = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(t.g) + e0);
  uint32_t* mcp = reinterpret_cast<uint32_t*>(t.m) + (size_t)gl * 16 + l16;
  uint32_t* vcp = reinterpret_cast<uint32_t*>(t.v) + (size_t)gl * 16 + l16;
  const uint4 praw = *pp;
  const uint4 graw = __ldg(gp);
  const uint32_t mc = *mcp;
  const uint32_t vc = *vcp;
  const float pm = __fmul_rn(qm_l, t.sm[gl]);
  const float pv = __fmul_rn(qv_l, t.sv[gl]);
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 16);
    prefetch_l2(gp + (size_t)pf * 16);
    prefetch_l2(mcp + (size_t)pf * 16);
    prefetch_l2(vcp + (size_t)pf * 16);
  }
  const unsigned pw[4] = {praw.x, praw.y, praw.z, praw.w}, gw[4] = {graw.x, graw.y, graw.z, graw.w};
  unsigned po[4];
  f2 m[4], v[4];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float m0a = __shfl_sync(hmask, pm, (int)(mc >> (8 * j)), 16);  // source lane = code (mod 16)
    const float m0b = __shfl_sync(hmask, pm, (int)(mc >> (8 * j + 4)), 16);
    const float v0a = __shfl_sync(hmask, pv, (int)(vc >> (8 * j)), 16);
    const float v0b = __shfl_sync(hmask, pv, (int)(vc >> (8 * j + 4)), 16);
    const f2 gj = widen2<T>(gw[j]);
    const f2 pj = widen2<T>(pw[j]);
    po[j] = narrow2<T>(fused_pair_x2<APX>(c, gj, pj, f2_pack(m0a, m0b), f2_pack(v0a, v0b), m[j], v[j], am, av));
  }
  const uint4 pnew = make_uint4(po[0], po[1], po[2], po[3]);
  *pp = pnew;
  if (PEERS) {
    for (int i = 0; i < ps.n; ++i) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(pp) + ps.off[i]) = pnew;
  }
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
  uint32_t mo = 0, vo = 0;
  if (udiv_ok(am) && udiv_ok(av)) {
    requant_x2<VLIN>(c, m, v, am, av, lut_m, lut_v, mo, vo);
  } else {  // scales outside the shared-reciprocal domain
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      float ma, mb, va, vb;
      f2_unpack(m[j], ma, mb);
      f2_unpack(v[j], va, vb);
      mo = (mo << 4) + (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(mb, am)) & 15);
      mo = (mo << 4) + (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(ma, am)) & 15);
      vo = (vo << 4) + (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(vb, av)) & 15);
      vo = (vo << 4) + (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(va, av)) & 15);
    }
  }
  *mcp = mo;
  *vcp = vo;
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

// Any 4-bit group, any alignment, any map: scalar accesses predicated on numel, IEEE sqrt and
// division, the reference's search (fused_adamw_kernel.cu:114,130-143,160-165).
template <typename T>
__device__ __noinline__ void h_group_generic(const TDesc& t, long long gl, int l16, unsigned hmask, const UConsts& c,
                                             const QMapSmem& Sm, const QMapSmem& Sv, const PeerStores& ps) {
  const long long e0 = gl * 128 + l16 * 8;
  const long long n = t.numel;
  unsigned short* p16 = reinterpret_cast<unsigned short*>(t.p);
  const unsigned short* g16 = reinterpret_cast<const unsigned short*>(t.g);
  uint8_t* mb = reinterpret_cast<uint8_t*>(t.m) + (e0 >> 1);
  uint8_t* vb = reinterpret_cast<uint8_t*>(t.v) + (e0 >> 1);
  const float sm = t.sm[gl];
  const float sv = t.sv[gl];
  UConsts ce = c;
  ce.f_fast = 0;
  float m[8], v[8];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    m[k] = 0.0f;
    v[k] = 0.0f;
    if (e0 + k < n) {
      const uint8_t mbyte = mb[k >> 1], vbyte = vb[k >> 1];
      const float g = Half16<T>::widen(g16[e0 + k]);
      const float m0 = __fmul_rn(Sm.qmap[(mbyte >> (4 * (k & 1))) & 15u], sm);
      const float v0 = __fmul_rn(Sv.qmap[(vbyte >> (4 * (k & 1))) & 15u], sv);
      m[k] = lerp_m<true>(ce, m0, g);
      v[k] = upd_v2<true>(ce, v0, g);
      const unsigned short pn = Half16<T>::narrow(upd_param<true>(ce, Half16<T>::widen(p16[e0 + k]), m[k], v[k]));
      p16[e0 + k] = pn;
      for (int i = 0; i < ps.n; ++i) *reinterpret_cast<unsigned short*>(reinterpret_cast<char*>(p16 + e0 + k) + ps.off[i]) = pn;
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

// One full, aligned 4-bit group, element by element (IEEE sqrt / division when the hyper-parameters lie
// outside the short sequences' domain).  qm_l / qv_l: this lane's entry of the two maps; the
// dequantised values come from a shuffle whose source lane is the code.
template <typename T, bool VLIN>
__device__ __forceinline__ void h_group_fast(const TDesc& t, unsigned gl, int l16, unsigned hmask, const UConsts& c,
                                             const QMapSmem& Sm, const QMapSmem& Sv, const LutEnt* __restrict__ lut_m,
                                             const LutEnt* __restrict__ lut_v, float qm_l, float qv_l, unsigned pf,
                                             const PeerStores& ps) {
  const size_t e0 = (size_t)gl * 128 + (size_t)l16 * 8;
  uint4* pp = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(t.p) + e0);
  const uint4* gp = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(t.g) + e0);
  uint32_t* mcp = reinterpret_cast<uint32_t*>(t.m) + (size_t)gl * 16 + l16;
  uint32_t* vcp = reinterpret_cast<uint32_t*>(t.v) + (size_t)gl * 16 + l16;
  const uint4 praw = *pp;
  const uint4 graw = __ldg(gp);
  const uint32_t mc = *mcp;
  const uint32_t vc = *vcp;
  const float pm = __fmul_rn(qm_l, t.sm[gl]);
  const float pv = __fmul_rn(qv_l, t.sv[gl]);
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 16);
    prefetch_l2(gp + (size_t)pf * 16);
    prefetch_l2(mcp + (size_t)pf * 16);
    prefetch_l2(vcp + (size_t)pf * 16);
  }
  float p[8], g[8], m[8], v[8];
  widen8<T>(praw, p);
  widen8<T>(graw, g);
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float m0 = __shfl_sync(hmask, pm, (int)(mc >> (4 * k)), 16);
    const float v0 = __shfl_sync(hmask, pv, (int)(vc >> (4 * k)), 16);
    m[k] = lerp_m<true>(c, m0, g[k]);
    v[k] = upd_v2<true>(c, v0, g[k]);
    p[k] = upd_param<true>(c, p[k], m[k], v[k]);
    am = fmaxf(am, fabsf(m[k]));
    av = fmaxf(av, v[k]);
  }
  const uint4 pnew = narrow8<T>(p);
  *pp = pnew;
  for (int i = 0; i < ps.n; ++i) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(pp) + ps.off[i]) = pnew;
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
    if (am == 0.0f) mo = 0xFFFFFFFFu;  // 0/0 = NaN -> code 15 for the whole group
    if (av == 0.0f) vo = 0xFFFFFFFFu;
  } else {
#pragma unroll
    for (int k = 7; k >= 0; --k) {
      mo = (mo << 4) + (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(m[k], am)) & 15);
      vo = (vo << 4) + (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(v[k], av)) & 15);
    }
  }
  *mcp = mo;
  *vcp = vo;
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

// fp32 moments (the numel <= threshold fallback) next to 16-bit parameters.
template <typename T>
__device__ __forceinline__ void h_group_fp32(const TDesc& t, long long gl, int l16, const UConsts& c, const PeerStores& ps) {
  const long long e0 = gl * 128 + l16 * 8;
  unsigned short* p16 = reinterpret_cast<unsigned short*>(t.p);
  const unsigned short* g16 = reinterpret_cast<const unsigned short*>(t.g);
  float* mp = reinterpret_cast<float*>(t.m);
  float* vp = reinterpret_cast<float*>(t.v);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const long long e = e0 + k;
    if (e < t.numel) {
      const float g = Half16<T>::widen(g16[e]);
      const float m = lerp_m<true>(c, mp[e], g);
      const float v = upd_v2<true>(c, vp[e], g);
      mp[e] = m;
      vp[e] = v;
      const unsigned short pn = Half16<T>::narrow(upd_param<true>(c, Half16<T>::widen(p16[e]), m, v));
      p16[e] = pn;
      for (int i = 0; i < ps.n; ++i) *reinterpret_cast<unsigned short*>(reinterpret_cast<char*>(p16 + e) + ps.off[i]) = pn;
    }
  }
}

// MATH: 0 = IEEE sqrt / division (hyper-parameters outside the short sequences' domain), 1 = the short exact
// sequences with packed arithmetic, 2 = as 1 with the tolerance-mode parameter update.  PEERS: every updated
// parameter also goes to the ZeRO-1 peers (ps); without it ps.n is 0 and the stores vanish from the packed path.
template <typename T, bool HAS_Q4, int MATH, bool PEERS>
__global__ void __launch_bounds__(CTA_THREADS, CTAS_PER_SM)
adamw4bit_half_kernel(const __grid_constant__ Table tab, const float* __restrict__ qmap_m,
                      const float* __restrict__ qmap_v, const UConsts cin, long long gbeg, long long gend,
                      const PeerStores ps) {
  const UConsts c = fused_consts(cin);
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm, Sv;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  LutEnt* lut_v = lut_m + LUT_ENTRIES;
  bool vlin = true, tables_ok = true;
  if (HAS_Q4) {
    lut_build(Sv, nullptr, qmap_v);
    vlin = Sv.linear16 != 0;
    if (!vlin) lut_build(Sv, lut_v, qmap_v);
    lut_build(Sm, lut_m, qmap_m);
    tables_ok = Sm.valid && Sv.valid;
  }
  const Consts2 k2 = make_consts_x2(c.f_beta1, c.f_beta2, c.f_omb1, c.f_omb2, c.f_lr, c.f_wd, c.f_eps, c.c1, c.c2s, c.rc2s);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = gbeg + (long long)blockIdx.x * HW_PER_CTA + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * HW_PER_CTA;
  const float qm_l = HAS_Q4 ? Sm.qmap[l16] : 0.0f, qv_l = HAS_Q4 ? Sv.qmap[l16] : 0.0f;
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
          unsigned gl = (unsigned)(gi - tstart);
          const unsigned lim = (unsigned)(fend - tstart);
          const unsigned st = (unsigned)stride;
          if (MATH >= 1 && vlin) {
            for (; gl < lim; gl += st)
              h_group_x2<T, true, MATH == 2, PEERS>(t, gl, l16, hmask, k2, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                                    (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u, ps);
          } else if (MATH >= 1) {
            for (; gl < lim; gl += st)
              h_group_x2<T, false, MATH == 2, PEERS>(t, gl, l16, hmask, k2, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                                     (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u, ps);
          } else if (vlin) {  // hyper-parameters outside the short sequences' domain: IEEE sqrt and division
            for (; gl < lim; gl += st)
              h_group_fast<T, true>(t, gl, l16, hmask, c, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                    (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u, ps);
          } else {
            for (; gl < lim; gl += st)
              h_group_fast<T, false>(t, gl, l16, hmask, c, Sm, Sv, lut_m, lut_v, qm_l, qv_l,
                                     (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u, ps);
          }
          gi = tstart + gl;
        }
      }
      for (; gi < tend; gi += stride) h_group_generic<T>(t, gi - tstart, l16, hmask, c, Sm, Sv, ps);
    } else {
      for (; gi < tend; gi += stride) h_group_fp32<T>(t, gi - tstart, l16, c, ps);
    }
  }
}

template <typename T, bool HAS_Q4, int MATH, bool PEERS>
static cudaError_t launch_half(const Table& tab, unsigned grid, const float* qm, const float* qv, const UConsts& c,
                               long long lo, long long hi, cudaStream_t st, const PeerStores& ps) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = HAS_Q4 ? H_DYN_SMEM : 0;
  if (HAS_Q4 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(adamw4bit_half_kernel<T, HAS_Q4, MATH, PEERS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)H_DYN_SMEM);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  adamw4bit_half_kernel<T, HAS_Q4, MATH, PEERS><<<grid, CTA_THREADS, smem, st>>>(tab, qm, qv, c, lo, hi, ps);
  return cudaGetLastError();
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

template <typename T, bool HAS_Q4, bool PEERS>
static cudaError_t launch_half_math(int math, const Table& tab, unsigned grid, const float* qm, const float* qv,
                                    const UConsts& c, long long lo, long long hi, cudaStream_t st, const PeerStores& ps) {
  if (math == 2 && HAS_Q4) return launch_half<T, HAS_Q4, HAS_Q4 ? 2 : 1, PEERS>(tab, grid, qm, qv, c, lo, hi, st, ps);
  return math ? launch_half<T, HAS_Q4, 1, PEERS>(tab, grid, qm, qv, c, lo, hi, st, ps)
              : launch_half<T, HAS_Q4, 0, PEERS>(tab, grid, qm, qv, c, lo, hi, st, ps);
}

// math: 0 IEEE, 1 short exact sequences, 2 tolerance-mode parameter update
template <typename T>
static cudaError_t launch_half_any(bool any_q4, int math, const Table& tab, unsigned grid, const float* qm, const float* qv,
                                   const UConsts& c, long long lo, long long hi, cudaStream_t st, const PeerStores& ps) {
  if (ps.n > 0)  // with peers always the 4-bit instantiation (it also steps fp32-state tensors); the maps are required
    return launch_half_math<T, true, true>(math, tab, grid, qm, qv, c, lo, hi, st, ps);
  if (!any_q4) return launch_half_math<T, false, false>(math, tab, grid, qm, qv, c, lo, hi, st, ps);
  return launch_half_math<T, true, false>(math, tab, grid, qm, qv, c, lo, hi, st, ps);
}

static int half_entry(const lpmm_b200_tensor* ts, int n, int dtype, const float* qmap_m, const float* qmap_v,
                      lpmm_b200_hyper h, int64_t group_begin, int64_t group_end, uint32_t flags, void* stream,
                      const PeerStores& ps) {
  if (dtype != LPMM_B200_DTYPE_BF16 && dtype != LPMM_B200_DTYPE_FP16) return LPMM_B200_ERR_BAD_KIND;
  if (flags & ~(uint32_t)LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) return LPMM_B200_ERR_BAD_KIND;
  bool any_q4 = false;
  int64_t total = 0;
  const int rc = check_tensor_list(ts, n, true, &any_q4, &total);
  if (rc != LPMM_B200_OK) return rc;
  if ((any_q4 || ps.n > 0) && (!qmap_m || !qmap_v)) return LPMM_B200_ERR_NULL_POINTER;
  if (group_end < 0) group_end = total;
  if (group_begin < 0 || group_begin > group_end || group_end > total) return LPMM_B200_ERR_BAD_SIZE;
  if (group_begin == group_end) return LPMM_B200_OK;
  const UConsts c = make_consts(h.beta1, h.beta2, h.lr, h.weight_decay, h.eps, h.step);
  // the folded constants of the tolerance mode need a finite 1 / lr
  const bool apx = (flags & LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) && c.f_fast && h.lr >= 0x1p-60f && h.lr <= 0x1p30f &&
                   h.weight_decay <= 0x1p30f;
  const int math = apx ? 2 : (c.f_fast ? 1 : 0);
  static thread_local Table tab;
  int64_t gcursor = 0;
  int i = 0;
  cudaStream_t st = (cudaStream_t)stream;
  while (i < n) {
    const Window w = next_window(ts, n, i, gcursor, group_begin, group_end, true, tab);
    if (!w.work) continue;
    const unsigned grid = multi_grid(w);
    const cudaError_t e = dtype == LPMM_B200_DTYPE_BF16
                              ? launch_half_any<__nv_bfloat16>(w.any_q4, math, tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st, ps)
                              : launch_half_any<__half>(w.any_q4, math, tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st, ps);
    LPMM_CUDA_TRY(e);
  }
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_16bit_flags(const lpmm_b200_tensor* ts, int n, int dtype,
                                                            const float* qmap_m, const float* qmap_v, lpmm_b200_hyper h,
                                                            int64_t group_begin, int64_t group_end, uint32_t flags,
                                                            void* stream) {
  return half_entry(ts, n, dtype, qmap_m, qmap_v, h, group_begin, group_end, flags, stream, PeerStores{});
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_16bit_peers(const lpmm_b200_tensor* ts, int n, int dtype,
                                                            const float* qmap_m, const float* qmap_v, lpmm_b200_hyper h,
                                                            int64_t group_begin, int64_t group_end,
                                                            const int64_t* peer_byte_offsets, int n_peers, uint32_t flags,
                                                            void* stream) {
  if (n_peers < 0 || n_peers > 7) return LPMM_B200_ERR_BAD_SIZE;
  if (n_peers > 0 && !peer_byte_offsets) return LPMM_B200_ERR_NULL_POINTER;
  PeerStores ps = {};
  ps.n = n_peers;
  for (int i = 0; i < n_peers; ++i) {
    if (peer_byte_offsets[i] % 16 != 0) return LPMM_B200_ERR_BAD_SIZE;  // keeps the 128-bit stores aligned
    ps.off[i] = peer_byte_offsets[i];
  }
  return half_entry(ts, n, dtype, qmap_m, qmap_v, h, group_begin, group_end, flags, stream, ps);
}

extern "C" int lpmm_b200_adamw4bit_multi_tensor_16bit(const lpmm_b200_tensor* ts, int n, int dtype, const float* qmap_m,
                                                      const float* qmap_v, lpmm_b200_hyper h, int64_t group_begin,
                                                      int64_t group_end, void* stream) {
  return lpmm_b200_adamw4bit_multi_tensor_16bit_flags(ts, n, dtype, qmap_m, qmap_v, h, group_begin, group_end, 0u, stream);
}
