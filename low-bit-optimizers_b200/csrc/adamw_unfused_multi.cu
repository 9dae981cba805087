// One launch for every tensor of a list whose two moments are 4-bit with group-128 scales (the
// reference's configuration when no qconfig is given) or both fp32, with the arithmetic and the state
// layout of the reference's NON-fused step (lpmm/optim/adamw.py:332-436 around vectorwise_quant /
// vectorwise_dequant).  The reference runs that path as a Python loop over parameters, a dozen torch
// kernels and two extension calls each; results here are those of the per-tensor launch of
// unfused.cu, bit for bit, with the work decomposition of the fused step (adamw4bit.cu): half-warp
// per 128-element group, 256-bit accesses, shuffle dequantisation, table / closed-form requantisation,
// packed fp32x2 arithmetic, L2 prefetch, descriptor table in the launch parameters.
//
// Differences from the fused step, all of them the reference's own: the order and contraction of
// the floating-point operations (unfused_math.cuh), bias corrections computed on the host in double,
// and the packed-code layout of vectorwise_quant, in which the zero padding of a tensor's last group
// is quantised together with the group.  The padding after the last group and the trailing byte are
// written once by the per-tensor launch that creates the states and never change.
#include <math.h>

#include "common.cuh"
#include "multi_tensor.cuh"
#include "unfused_math.cuh"

namespace lpmm_b200 {

constexpr size_t UM_DYN_SMEM = 2 * LUT_ENTRIES * sizeof(LutEnt);  // one table per moment

// Any 4-bit group, any alignment, any map: scalar accesses predicated on numel, IEEE division, the
// reference's search.  The whole group is requantised (its padding is 0 / max).
template <bool A>
__device__ __noinline__ void um_group_generic(const TDesc& t, long long gl, int l16, unsigned hmask, const UConsts& c,
                                              const QMapSmem& Sm, const QMapSmem& Sv) {
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
      const float g = t.g[e0 + k];
      const float m0 = __fmul_rn(Sm.qmap[(mbyte >> (4 * (k & 1))) & 15u], sm);
      const float v0 = __fmul_rn(Sv.qmap[(vbyte >> (4 * (k & 1))) & 15u], sv);
      m[k] = lerp_m<A>(c, m0, g);
      v[k] = upd_v2<A>(c, v0, g);
      t.p[e0 + k] = upd_param<A>(c, t.p[e0 + k], m[k], v[k]);
      am = fmaxf(am, fabsf(m[k]));
      av = fmaxf(av, v[k]);
    }
  }
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t mo = (uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(m[2 * j], am)) & 15) |
                        ((uint32_t)(bsearch_code(Sm.qmap, __fdiv_rn(m[2 * j + 1], am)) & 15) << 4);
    const uint32_t vo = (uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(v[2 * j], av)) & 15) |
                        ((uint32_t)(bsearch_code(Sv.qmap, __fdiv_rn(v[2 * j + 1], av)) & 15) << 4);
    mb[j] = (uint8_t)mo;
    vb[j] = (uint8_t)vo;
  }
  if (l16 == 0) {
    t.sm[gl] = am;
    t.sv[gl] = av;
  }
}

struct UmLane {
  float* p;
  const float* g;
  uint32_t* mc;
  uint32_t* vc;
  float* sm;
  float* sv;
};

// One full, aligned group with packed arithmetic (update_pair) and the short exact division for the
// normalisation; selected only when the hyper-parameters are in the domain of the short sequences.
// APX: the tolerance mode of the parameter update (unfused_math.cuh); moments, maxima and codes unchanged.
template <bool APX>
__device__ __forceinline__ void um_group_x2(const UmLane& t, unsigned gl, int l16, unsigned hmask, const UConsts2& k,
                                            const QMapSmem& Sm, const QMapSmem& Sv, const LutEnt* __restrict__ lut_m,
                                            const LutEnt* __restrict__ lut_v, bool vlin, float qm_l, float qv_l,
                                            unsigned pf) {
  float* pp = t.p + (size_t)gl * 128;
  const float* gp = t.g + (size_t)gl * 128;
  uint32_t* mcp = t.mc + (size_t)gl * 16;
  uint32_t* vcp = t.vc + (size_t)gl * 16;
  f2x4 p = ldg_f2x4(pp);
  const f2x4 g = ldg_f2x4(gp);
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
    update_pair<APX>(k, g.v[j], p.v[j], f2_pack(m0a, m0b), f2_pack(v0a, v0b), m[j], v[j], am, av);
  }
  stg_f2x4(pp, p);
  am = hw_max(am, hmask);
  av = hw_max(av, hmask);
  uint32_t mo = 0, vo = 0;
  if (udiv_ok(am) && udiv_ok(av)) {
    const f2 rm2 = f2_splat(rcp_nr(am)), rv2 = f2_splat(rcp_nr(av)), nam2 = f2_splat(-am), nav2 = f2_splat(-av);
    const f2 k16 = f2_splat(16.0f), km15 = f2_splat(-1.5f);
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
      if (vlin) {
        float ta, tb;
        f2_unpack(f2_fma(xv, k16, km15), ta, tb);
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
  } else {  // scales outside the shared-reciprocal domain: IEEE division and the search
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

// fp32 moments (the numel <= threshold fallback), 128 elements per half-warp step.
template <bool A>
__device__ __forceinline__ void um_group_fp32(const TDesc& t, long long gl, int l16, const UConsts& c) {
  const long long e0 = gl * 128 + l16 * 8;
  float* mp = reinterpret_cast<float*>(t.m);
  float* vp = reinterpret_cast<float*>(t.v);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const long long e = e0 + k;
    if (e < t.numel) {
      const float g = t.g[e];
      const float m = lerp_m<A>(c, mp[e], g);
      const float v = upd_v2<A>(c, vp[e], g);
      mp[e] = m;
      vp[e] = v;
      t.p[e] = upd_param<A>(c, t.p[e], m, v);
    }
  }
}

// A: the arithmetic of the reference's fused kernel (scalar paths only) instead of its torch operations.
// APX (with A false): the tolerance-mode parameter update on full aligned 4-bit groups.
template <bool HAS_Q4, bool A, bool APX>
__global__ void __launch_bounds__(CTA_THREADS, CTAS_PER_SM)
adamw_unfused_multi_kernel(const __grid_constant__ Table tab, const float* __restrict__ qmap_m,
                           const float* __restrict__ qmap_v, const UConsts cin, long long gbeg, long long gend) {
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
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
  const UConsts2 k2 = make_consts2(c);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = gbeg + (long long)blockIdx.x * HW_PER_CTA + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * HW_PER_CTA;
  const float qm_l = HAS_Q4 ? Sm.qmap[l16] : 0.0f, qv_l = HAS_Q4 ? Sv.qmap[l16] : 0.0f;
  // the tensor loop is uniform across the CTA; each half-warp walks gi, gi + stride, ... through it
  int ti = 0;
  while (ti + 1 < tab.n && tab.t[ti + 1].gstart <= gbeg) ++ti;
  for (; ti < tab.n; ++ti) {
    const TDesc& t = tab.t[ti];
    const long long tstart = t.gstart;
    if (tstart >= gend) break;
    long long tend = (ti + 1 < tab.n) ? tab.t[ti + 1].gstart : tab.gtotal;
    if (tend > gend) tend = gend;
    if (t.kind == LPMM_B200_KIND_Q4) {
      if (!A && tables_ok && t.aligned && c.fast) {
        long long fend = tstart + t.numel / 128;  // end of the full groups
        if (fend > tend) fend = tend;
        if (gi < fend) {
          UmLane lp;
          lp.p = t.p + l16 * 8;
          lp.g = t.g + l16 * 8;
          lp.mc = reinterpret_cast<uint32_t*>(t.m) + l16;
          lp.vc = reinterpret_cast<uint32_t*>(t.v) + l16;
          lp.sm = t.sm;
          lp.sv = t.sv;
          unsigned gl = (unsigned)(gi - tstart);  // groups per tensor fit 32 bits (host-checked)
          const unsigned lim = (unsigned)(fend - tstart);
          const unsigned st = (unsigned)stride;
          for (; gl < lim; gl += st)
            um_group_x2<APX>(lp, gl, l16, hmask, k2, Sm, Sv, lut_m, lut_v, vlin, qm_l, qv_l,
                        (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u);
          gi = tstart + gl;
        }
      }
      for (; gi < tend; gi += stride) um_group_generic<A>(t, gi - tstart, l16, hmask, c, Sm, Sv);
    } else {
      for (; gi < tend; gi += stride) um_group_fp32<A>(t, gi - tstart, l16, c);
    }
  }
}

template <bool HAS_Q4, bool A, bool APX>
static cudaError_t launch_um(const Table& tab, unsigned grid, const float* qm, const float* qv, const UConsts& c,
                             long long lo, long long hi, cudaStream_t st) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = HAS_Q4 ? UM_DYN_SMEM : 0;
  if (HAS_Q4 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(adamw_unfused_multi_kernel<HAS_Q4, A, APX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)UM_DYN_SMEM);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  adamw_unfused_multi_kernel<HAS_Q4, A, APX><<<grid, CTA_THREADS, smem, st>>>(tab, qm, qv, c, lo, hi);
  return cudaGetLastError();
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

static int um_step(const lpmm_b200_tensor* ts, int n, const float* qmap_m, const float* qmap_v, double beta1, double beta2,
                   double lr, double weight_decay, double eps, double step, int64_t group_begin, int64_t group_end,
                   void* stream, int arith, int apx) {
  bool any_q4 = false;
  int64_t total = 0;
  const int rc = check_tensor_list(ts, n, true, &any_q4, &total);
  if (rc != LPMM_B200_OK) return rc;
  if (any_q4 && (!qmap_m || !qmap_v)) return LPMM_B200_ERR_NULL_POINTER;
  if (group_end < 0) group_end = total;
  if (group_begin < 0 || group_begin > group_end || group_end > total) return LPMM_B200_ERR_BAD_SIZE;
  if (group_begin == group_end) return LPMM_B200_OK;
  const UConsts c = make_consts(beta1, beta2, lr, weight_decay, eps, step);
  static thread_local Table tab;
  int64_t gcursor = 0;
  int i = 0;
  while (i < n) {
    const Window w = next_window(ts, n, i, gcursor, group_begin, group_end, true, tab);
    if (!w.work) continue;
    const unsigned grid = multi_grid(w);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (arith) e = w.any_q4 ? launch_um<true, true, false>(tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st)
                            : launch_um<false, true, false>(tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st);
    else if (apx && w.any_q4) e = launch_um<true, false, true>(tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st);
    else e = w.any_q4 ? launch_um<true, false, false>(tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st)
                      : launch_um<false, false, false>(tab, grid, qmap_m, qmap_v, c, w.lo, w.hi, st);
    LPMM_CUDA_TRY(e);
  }
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_adamw4bit_unfused_multi_tensor(const lpmm_b200_tensor* ts, int n, const float* qmap_m,
                                                        const float* qmap_v, double beta1, double beta2, double lr,
                                                        double weight_decay, double eps, double step,
                                                        int64_t group_begin, int64_t group_end, void* stream) {
  return um_step(ts, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, group_begin, group_end, stream, 0, 0);
}

// The same launch with the tolerance-mode parameter update (flags & LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE); internal
// to the library, reached through lpmm_b200_adamw4bit_unfused_step_many_flags.
LPMM_INTERNAL int lpmm_b200_unfused_multi_tensor_apx(const lpmm_b200_tensor* ts, int n, const float* qmap_m,
                                                  const float* qmap_v, double beta1, double beta2, double lr,
                                                  double weight_decay, double eps, double step, void* stream) {
  return um_step(ts, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, 0, -1, stream, 0, 1);
}

// The same launch with the fused kernel's arithmetic on these (padded) states; internal to the library,
// reached through lpmm_b200_adamw4bit_fused_arith_step_many.
LPMM_INTERNAL int lpmm_b200_fused_arith_multi_tensor(const lpmm_b200_tensor* ts, int n, const float* qmap_m,
                                                  const float* qmap_v, double beta1, double beta2, double lr,
                                                  double weight_decay, double eps, double step, void* stream) {
  return um_step(ts, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, 0, -1, stream, 1, 0);
}
