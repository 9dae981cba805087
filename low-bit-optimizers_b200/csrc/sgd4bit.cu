// One-launch momentum SGD over a whole parameter list with 4-bit group-128 momentum buffers.
//
// The reference refuses fused=True for SGD (lpmm/optim/sgd.py:31-32) and steps one tensor at a
// time through torch ops and its quantize / dequantize calls (sgd.py:133-187).  This kernel does
// the arithmetic of that per-tensor path, operation by operation,
//   d = maximize ? -g : g;  d = fma(wd, p, d)                      d_p.add(param, alpha=wd)
//   b = fma(1 - dampening, d, b0 * momentum)                       buf.mul_(momentum).add_(d_p, alpha=1-dampening)
//   d = nesterov ? fma(momentum, b, d) : b                         d_p.add(buf, alpha=momentum)
//   p = fma(-lr, d, p)                                             param.add_(d_p, alpha=-lr)
//   new scale = group max |b|, new code = nearest-code rule on b / scale
// for every tensor of the list in one launch, with the work decomposition of the fused AdamW step:
// a half-warp owns a 128-element group, one 256-bit access per lane for p and g, one 32-bit access
// for the 8 codes, dequantization by shuffle, table-driven requantization.  Buffers use the
// non-fused layout (codes at byte e/2 of the padded tensor, one scale per group), so a state written
// by the per-tensor path continues here and vice versa; the zero padding after the last group and
// the trailing byte are not touched (the per-tensor step that creates the buffer writes them).
// The first step of a tensor (buffer = clone of d_p) belongs to the per-tensor entry point.
#include <math.h>

#include "common.cuh"
#include "multi_tensor.cuh"

namespace lpmm_b200 {

constexpr size_t SGD_DYN_SMEM = LUT_ENTRIES * sizeof(LutEnt);

struct SgdK {
  float wd, momentum, omd, neg_lr;
  int has_wd, nesterov, maximize;
};

__device__ __forceinline__ float sgd_elem(const SgdK& c, float& p, float g, float b0) {
  float d = c.maximize ? -g : g;
  if (c.has_wd) d = __fmaf_rn(c.wd, p, d);
  const float b = __fmaf_rn(c.omd, d, __fmul_rn(b0, c.momentum));
  d = c.nesterov ? __fmaf_rn(c.momentum, b, d) : b;
  p = __fmaf_rn(c.neg_lr, d, p);
  return b;
}

// Any group, any alignment, any map: scalar accesses predicated on numel, IEEE division, the
// reference's search (quantization_kernel.cu:397-427).
__device__ __noinline__ void sgd_group_generic(const TDesc& t, long long gl, int l16, unsigned hmask, const SgdK& c,
                                               const QMapSmem& S) {
  const long long e0 = gl * 128 + l16 * 8;
  const long long n = t.numel;
  uint8_t* bb = reinterpret_cast<uint8_t*>(t.m) + (e0 >> 1);
  const float sc = t.sm[gl];
  float b[8];
  float ab = 0.0f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    b[k] = 0.0f;
    if (e0 + k < n) {
      const uint8_t byte = bb[k >> 1];
      const int code = (k & 1) ? (byte >> 4) : (byte & 15);
      float p = t.p[e0 + k];
      b[k] = sgd_elem(c, p, t.g[e0 + k], __fmul_rn(S.qmap[code], sc));
      t.p[e0 + k] = p;
      ab = fmaxf(ab, fabsf(b[k]));
    }
  }
  ab = hw_max(ab, hmask);
  // the zero padding inside the last group is requantized with it (0 / max), as the per-tensor step
  // does; the packed tensor is padded to whole rows of 2048 codes, so the whole group is addressable
#pragma unroll
  for (int k = 0; k < 8; k += 2) {
    const int c0 = bsearch_code(S.qmap, __fdiv_rn(b[k], ab)) & 15;
    const int c1 = bsearch_code(S.qmap, __fdiv_rn(b[k + 1], ab)) & 15;
    bb[k >> 1] = (uint8_t)(c0 | (c1 << 4));
  }
  if (l16 == 0) t.sm[gl] = ab;
}

struct SgdK2 {
  f2 wd, momentum, omd, neg_lr, mone;
};

// One full, aligned group with packed fp32x2 arithmetic (each half rounds like the scalar instruction).
__device__ __forceinline__ void sgd_group_x2(float* __restrict__ pbase, const float* __restrict__ gbase,
                                             uint32_t* __restrict__ cbase, float* __restrict__ scales, unsigned gl,
                                             int l16, unsigned hmask, const SgdK& c, const SgdK2& k, const QMapSmem& S,
                                             const LutEnt* __restrict__ lut, float q_l, unsigned pf) {
  float* pp = pbase + (size_t)gl * 128;
  const float* gp = gbase + (size_t)gl * 128;
  uint32_t* cp = cbase + (size_t)gl * 16;
  f2x4 p = ldg_f2x4(pp);
  const f2x4 g = ldg_f2x4(gp);
  const uint32_t codes = *cp;
  const float pq = __fmul_rn(q_l, scales[gl]);  // lane i: qmap[i] * scale
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 128);
    prefetch_l2(gp + (size_t)pf * 128);
    prefetch_l2(cp + (size_t)pf * 16);
  }
  f2 b[4];
  float ab = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float b0a = __shfl_sync(hmask, pq, (int)(codes >> (8 * j)), 16);  // source lane = code (mod 16)
    const float b0b = __shfl_sync(hmask, pq, (int)(codes >> (8 * j + 4)), 16);
    f2 d = c.maximize ? f2_mul(g.v[j], k.mone) : g.v[j];
    if (c.has_wd) d = f2_fma(k.wd, p.v[j], d);
    b[j] = f2_fma(k.omd, d, f2_mul(f2_pack(b0a, b0b), k.momentum));
    d = c.nesterov ? f2_fma(k.momentum, b[j], d) : b[j];
    p.v[j] = f2_fma(k.neg_lr, d, p.v[j]);
    float ba, bb;
    f2_unpack(b[j], ba, bb);
    ab = fmaxf(ab, fmaxf(fabsf(ba), fabsf(bb)));
  }
  stg_f2x4(pp, p);
  ab = hw_max(ab, hmask);
  uint32_t out = 0;
  if (udiv_ok(ab)) {
    const f2 r2 = f2_splat(rcp_nr(ab)), nab2 = f2_splat(-ab);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      f2 x = f2_mul(b[j], r2);
      x = f2_fma(f2_fma(x, nab2, b[j]), r2, x);
      float xa, xb;
      f2_unpack(x, xa, xb);
      out = (out << 4) + (uint32_t)lut_code(lut, xb);
      out = (out << 4) + (uint32_t)lut_code(lut, xa);
    }
    if (ab == 0.0f) out = 0xFFFFFFFFu;  // 0/0 = NaN -> code 15 for the whole group
  } else {  // scale outside the shared-reciprocal domain
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      float ba, bb;
      f2_unpack(b[j], ba, bb);
      out = (out << 4) + (uint32_t)(bsearch_code(S.qmap, __fdiv_rn(bb, ab)) & 15);
      out = (out << 4) + (uint32_t)(bsearch_code(S.qmap, __fdiv_rn(ba, ab)) & 15);
    }
  }
  *cp = out;
  if (l16 == 0) scales[gl] = ab;
}

// fp32 buffers (the numel <= threshold fallback).
__device__ __forceinline__ void sgd_group_fp32(const TDesc& t, long long gl, int l16, const SgdK& c) {
  const long long e0 = gl * 128 + l16 * 8;
  float* bp = reinterpret_cast<float*>(t.m);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const long long e = e0 + k;
    if (e < t.numel) {
      float p = t.p[e];
      bp[e] = sgd_elem(c, p, t.g[e], bp[e]);
      t.p[e] = p;
    }
  }
}

template <bool HAS_Q4>
__global__ void __launch_bounds__(CTA_THREADS, CTAS_PER_SM)
sgd4bit_multi_kernel(const __grid_constant__ Table tab, const float* __restrict__ qmap, const SgdK c, long long gbeg,
                     long long gend) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem S;
  LutEnt* lut = reinterpret_cast<LutEnt*>(dyn_smem);
  bool table_ok = true;
  if (HAS_Q4) {
    lut_build(S, lut, qmap);
    table_ok = S.valid != 0;
  }
  SgdK2 k;
  k.wd = f2_splat(c.wd);
  k.momentum = f2_splat(c.momentum);
  k.omd = f2_splat(c.omd);
  k.neg_lr = f2_splat(c.neg_lr);
  k.mone = f2_splat(-1.0f);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = gbeg + (long long)blockIdx.x * HW_PER_CTA + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * HW_PER_CTA;
  const float q_l = HAS_Q4 ? S.qmap[l16] : 0.0f;
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
      if (table_ok && t.aligned) {
        long long fend = tstart + t.numel / 128;  // end of the full groups
        if (fend > tend) fend = tend;
        if (gi < fend) {
          float* pb = t.p + l16 * 8;
          const float* gb = t.g + l16 * 8;
          uint32_t* cb = reinterpret_cast<uint32_t*>(t.m) + l16;
          unsigned gl = (unsigned)(gi - tstart);  // groups per tensor fit 32 bits (host-checked)
          const unsigned lim = (unsigned)(fend - tstart);
          const unsigned st = (unsigned)stride;
          for (; gl < lim; gl += st)
            sgd_group_x2(pb, gb, cb, t.sm, gl, l16, hmask, c, k, S, lut, q_l, (gl + PF_DIST * st < lim) ? PF_DIST * st : 0u);
          gi = tstart + gl;
        }
      }
      for (; gi < tend; gi += stride) sgd_group_generic(t, gi - tstart, l16, hmask, c, S);
    } else {
      for (; gi < tend; gi += stride) sgd_group_fp32(t, gi - tstart, l16, c);
    }
  }
}

template <bool HAS_Q4>
static cudaError_t launch_sgd(const Table& tab, unsigned grid, const float* qmap, const SgdK& c, long long lo,
                              long long hi, cudaStream_t st) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = HAS_Q4 ? SGD_DYN_SMEM : 0;
  if (HAS_Q4 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(sgd4bit_multi_kernel<HAS_Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)SGD_DYN_SMEM);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  sgd4bit_multi_kernel<HAS_Q4><<<grid, CTA_THREADS, smem, st>>>(tab, qmap, c, lo, hi);
  return cudaGetLastError();
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

extern "C" int lpmm_b200_sgd4bit_multi_tensor(const lpmm_b200_tensor* ts, int n, const float* qmap,
                                              double weight_decay, double momentum, double lr, double dampening,
                                              int nesterov, int maximize, int64_t group_begin, int64_t group_end,
                                              void* stream) {
  if (momentum == 0.0 && n >= 0) return LPMM_B200_ERR_BAD_KIND;  // no buffer to step: use the per-tensor entry point
  bool any_q4 = false;
  int64_t total = 0;
  const int rc = check_tensor_list(ts, n, false, &any_q4, &total);
  if (rc != LPMM_B200_OK) return rc;
  if (any_q4 && !qmap) return LPMM_B200_ERR_NULL_POINTER;
  if (group_end < 0) group_end = total;
  if (group_begin < 0 || group_begin > group_end || group_end > total) return LPMM_B200_ERR_BAD_SIZE;
  if (group_begin == group_end) return LPMM_B200_OK;
  SgdK c;
  c.wd = (float)weight_decay;
  c.momentum = (float)momentum;
  c.omd = (float)(1.0 - dampening);
  c.neg_lr = (float)(-lr);
  c.has_wd = weight_decay != 0.0;
  c.nesterov = nesterov != 0;
  c.maximize = maximize != 0;
  static thread_local Table tab;
  int64_t gcursor = 0;
  int i = 0;
  while (i < n) {
    const Window w = next_window(ts, n, i, gcursor, group_begin, group_end, false, tab);
    if (!w.work) continue;
    const cudaError_t e = w.any_q4 ? launch_sgd<true>(tab, multi_grid(w), qmap, c, w.lo, w.hi, (cudaStream_t)stream)
                                   : launch_sgd<false>(tab, multi_grid(w), qmap, c, w.lo, w.hi, (cudaStream_t)stream);
    LPMM_CUDA_TRY(e);
  }
  return LPMM_B200_OK;
}
