// Per-tensor kernels with the arithmetic and state layout of the reference's non-fused Python
// path, and the standalone quantize / dequantize kernels behind lpmm.functional.
//
// The reference runs these steps as a chain of torch element-wise kernels around two extension
// calls (lpmm/optim/adamw.py:332-436, 579-627; lpmm/optim/sgd.py:133-187; lpmm/functional.py:26-151).
// Here each tensor is updated by one launch (plus a statistics pass where the normalisation
// needs tensor-wide maxima or sums) that performs the same fp32 operations in the same order:
//   p1 = p * float(1 - lr*wd)
//   m  = fma(w, g - m0, m0),  w = float(1 - beta1)                  torch lerp, weight < 0.5
//   v  = fma(float(1 - beta2), g*g, v0 * float(beta2))              mul_ then addcmul_
//   d  = sqrt(v) * float(1.0 / sqrt(1 - beta2^step)) + float(eps)    division by a host scalar
//   p  = fma(float(-lr / (1 - beta1^step)), m / d, p1)              addcdiv_
// with the scalar constants computed in double on the host exactly as Python computes them.
// The contraction choices were settled against torch's own CUDA kernels.
//
// Layout: a half-warp owns a unit of 128 consecutive elements (lane = 8 elements), as in the
// fused step.  Codes live in the reference's padded layout: ceil(n'/2048)*1024 bytes plus one
// trailing byte, n' = numel rounded up to 128 (group scales) or numel (rank-1 scales).
#include <math.h>

#include "common.cuh"

namespace lpmm_b200 {

constexpr int UT = 256;  // threads per CTA

struct Shape {
  int nd;
  long long dim[8];
};

struct UConsts {
  float wd_mul, lerp_w, lerp_omw, beta2, omb2, inv_bc2s, bc2s, eps, alpha;
  int lerp_small;
  int fast;  // eps keeps the denominator inside the domain of the short exact sqrt / division sequences
};

struct StepArgs {
  float* p;
  const float* g;
  long long n;
  long long units;  // padded length / 128
  int first;
  int vec_ok;  // p and g are 16-byte aligned: full lanes use 128-bit accesses
  void* m;
  float* m_max1;
  void* v;
  float* v_max1;
  const float* v_old[8];
  float* v_new[8];
  float* row;
  float* col;
  const float* row_mean;  // per batch (factored)
  Shape s;
};

struct Maps {
  float qm[16];
  float qv[16];
  float mm[16];  // midpoints of qm, padded with +inf
  float mv[16];
  int zero_m, zero_v;  // code of 0.0f in each map (what padding quantizes to)
};

// Nearest-code rule as a branch-free four-step search over the 15 sorted midpoints:
// code = #{midpoints < x}; a NaN gives 15 like the reference's search.
__device__ __forceinline__ int code16(const float* __restrict__ mids, float x) {
  int c = (mids[7] < x) ? 8 : 0;
  c += (mids[c + 3] < x) ? 4 : 0;
  c += (mids[c + 1] < x) ? 2 : 0;
  c += (mids[c] < x) ? 1 : 0;
  return (x != x) ? 15 : c;
}

// x / d for the 8 values of a lane with a divisor shared by the half-warp: the shared-reciprocal
// division (equal to IEEE division, see common.cuh) when d is in its domain, IEEE division otherwise.
__device__ __forceinline__ uint32_t codes_by_group_scale(const float* __restrict__ mids, const float* x, float d) {
  uint32_t out = 0;
  if (udiv_ok(d)) {
    const float r = rcp_nr(d);
#pragma unroll
    for (int k = 0; k < 8; ++k) out |= (uint32_t)code16(mids, udiv(x[k], d, r)) << (4 * k);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) out |= (uint32_t)code16(mids, __fdiv_rn(x[k], d)) << (4 * k);
  }
  return out;
}

__device__ __forceinline__ void load_maps(Maps& M, const float* __restrict__ qm, const float* __restrict__ qv) {
  const int tid = threadIdx.x;
  if (tid < 16) {
    M.qm[tid] = qm ? qm[tid] : 0.0f;
    M.qv[tid] = qv ? qv[tid] : 0.0f;
  }
  __syncthreads();
  if (tid < 16) {
    const float inf = __int_as_float(0x7f800000);
    M.mm[tid] = tid < 15 ? __fmul_rn(__fadd_rn(M.qm[tid], M.qm[tid + 1]), 0.5f) : inf;
    M.mv[tid] = tid < 15 ? __fmul_rn(__fadd_rn(M.qv[tid], M.qv[tid + 1]), 0.5f) : inf;
  }
  __syncthreads();
  if (tid == 0) {
    M.zero_m = code16(M.mm, 0.0f);
    M.zero_v = code16(M.mv, 0.0f);
  }
  __syncthreads();
}

__device__ __forceinline__ float hmax16(float x, unsigned mask) {
#pragma unroll
  for (int o = 8; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(mask, x, o, 16));
  return x;
}

// Row-major coordinates of a flat index, and the step to the next element.  ND is the exact
// number of axes for 2, 3 and 4 (loops fully unrolled, no guards) and 8 means "up to 8, see s.nd".
template <int ND>
__device__ __forceinline__ void decompose(long long e, const Shape& s, int* c) {
#pragma unroll
  for (int i = ND - 1; i >= 0; --i) {
    if (ND < 8 || i < s.nd) {
      const long long q = e / s.dim[i];
      c[i] = (int)(e - q * s.dim[i]);
      e = q;
    } else {
      c[i] = 0;
    }
  }
}
template <int ND>
__device__ __forceinline__ void advance(int* c, const Shape& s) {
#pragma unroll
  for (int i = ND - 1; i >= 0; --i) {
    if (ND < 8 || i < s.nd) {
      if (++c[i] < s.dim[i]) return;
      c[i] = 0;
    }
  }
}
template <int ND>
__device__ __forceinline__ float axis_min(const float* const* vecs, const int* c, int nd) {
  float st = __ldg(vecs[0] + c[0]);
#pragma unroll
  for (int i = 1; i < ND; ++i)
    if (ND < 8 || i < nd) st = fminf(st, __ldg(vecs[i] + c[i]));
  return st;
}

// min_i vecs[i][idx_i] for the 8 consecutive elements starting at flat index e0.  2-D tensors whose
// lane stays inside one row read the row value once and the 8 column values as two 128-bit loads.
template <int ND>
__device__ __forceinline__ void lane_scales(const float* const* vecs, long long e0, long long n, const Shape& s,
                                            float* out) {
  if (ND == 2) {
    const long long C = s.dim[1];
    const long long r = e0 / C;
    const long long col = e0 - r * C;
    if (col + 8 <= C && e0 + 8 <= n && ((reinterpret_cast<uintptr_t>(vecs[1] + col) & 15) == 0)) {
      const float rv = __ldg(vecs[0] + r);
      const float4 c0 = __ldg(reinterpret_cast<const float4*>(vecs[1] + col));
      const float4 c1 = __ldg(reinterpret_cast<const float4*>(vecs[1] + col + 4));
      out[0] = fminf(rv, c0.x); out[1] = fminf(rv, c0.y); out[2] = fminf(rv, c0.z); out[3] = fminf(rv, c0.w);
      out[4] = fminf(rv, c1.x); out[5] = fminf(rv, c1.y); out[6] = fminf(rv, c1.z); out[7] = fminf(rv, c1.w);
      return;
    }
  }
  int co[8];
  decompose<ND>(e0, s, co);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    out[k] = 1.0f;
    if (e0 + k < n) out[k] = axis_min<ND>(vecs, co, s.nd);
    advance<ND>(co, s);
  }
}

// Monotone max of a non-negative float through an integer atomic; a stale read can only be too
// small, so skipping the atomic when the value is not larger is always safe.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float val) {
  if (val > *reinterpret_cast<volatile float*>(addr)) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(val));
}

__device__ __forceinline__ float lerp_m(const UConsts& c, float m0, float g) {
  const float diff = __fsub_rn(g, m0);
  return c.lerp_small ? __fmaf_rn(c.lerp_w, diff, m0) : __fmaf_rn(-diff, c.lerp_omw, g);
}
__device__ __forceinline__ float upd_v2(const UConsts& c, float v0, float g) {
  return __fmaf_rn(c.omb2, __fmul_rn(g, g), __fmul_rn(v0, c.beta2));
}
__device__ __forceinline__ float upd_param(const UConsts& c, float p, float m, float v) {
  const float p1 = __fmul_rn(p, c.wd_mul);
  if (c.fast) {
    const float d = __fadd_rn(__fmul_rn(sqrt_rn_fast(v), c.inv_bc2s), c.eps);
    return __fmaf_rn(c.alpha, div_rn_fast(m, d), p1);
  }
  const float d = __fadd_rn(__fmul_rn(__fsqrt_rn(v), c.inv_bc2s), c.eps);
  return __fmaf_rn(c.alpha, __fdiv_rn(m, d), p1);
}

// ---------------------------------------------------------------------------------------------
// AdamW, non-fused semantics.  MM: first-moment storage, VM: second-moment storage / source.
// ---------------------------------------------------------------------------------------------
template <int MM, int VM, int ND>
__global__ void __launch_bounds__(UT) unfused_adamw_kernel(const StepArgs a, const UConsts c,
                                                            const float* __restrict__ qmap_m,
                                                            const float* __restrict__ qmap_v) {
  __shared__ Maps M;
  load_maps(M, qmap_m, qmap_v);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long n = a.n;
  const long long real_units = (n + 127) / 128;
  const long long C = (VM == LPMM_B200_STATE_FACTORED) ? a.s.dim[a.s.nd - 1] : 1;
  const long long RC = (VM == LPMM_B200_STATE_FACTORED) ? C * a.s.dim[a.s.nd - 2] : 1;
  for (long long u = (long long)blockIdx.x * (UT / 16) + (threadIdx.x >> 4); u < a.units;
       u += (long long)gridDim.x * (UT / 16)) {
    const long long e0 = u * 128 + l16 * 8;
    uint8_t* mb = (MM == LPMM_B200_STATE_GROUP4) ? reinterpret_cast<uint8_t*>(a.m) + (e0 >> 1) : nullptr;
    uint8_t* vb = (VM == LPMM_B200_STATE_GROUP4 || VM == LPMM_B200_STATE_RANK1_4)
                      ? reinterpret_cast<uint8_t*>(a.v) + (e0 >> 1) : nullptr;
    if (u >= real_units) {  // rows of 2048 are filled up with zeros after normalisation
      if (mb) *reinterpret_cast<uint32_t*>(mb) = 0x11111111u * (uint32_t)M.zero_m;
      if (vb) *reinterpret_cast<uint32_t*>(vb) = 0x11111111u * (uint32_t)M.zero_v;
      continue;
    }
    uint32_t mcodes = 0, vcodes = 0;
    float sm = 0.0f, sv = 0.0f;
    if (!a.first) {
      if (MM == LPMM_B200_STATE_GROUP4) {
        mcodes = *reinterpret_cast<const uint32_t*>(mb);
        sm = a.m_max1[u];
      }
      if (vb) vcodes = *reinterpret_cast<const uint32_t*>(vb);
      if (VM == LPMM_B200_STATE_GROUP4) sv = a.v_max1[u];
    }
    float st_old[8], st_new[8];
    if (VM == LPMM_B200_STATE_RANK1_4) {
      if (!a.first) lane_scales<ND>(a.v_old, e0, n, a.s, st_old);
      lane_scales<ND>(a.v_new, e0, n, a.s, st_new);
    }
    long long rowi = 0, cc = 0, bi = 0;  // factored: row index in the [B*R, C] view, column, batch entry
    if (VM == LPMM_B200_STATE_FACTORED) {
      rowi = e0 / C;
      cc = e0 - rowi * C;
      bi = e0 / RC;
    }
    float m[8], v[8], gx[8], px[8];
    float am = 0.0f, av = 0.0f;
    const bool full = a.vec_ok && (e0 + 8 <= n);
    if (full) {
      const float4 g0 = *reinterpret_cast<const float4*>(a.g + e0), g1 = *reinterpret_cast<const float4*>(a.g + e0 + 4);
      const float4 p0 = *reinterpret_cast<const float4*>(a.p + e0), p1 = *reinterpret_cast<const float4*>(a.p + e0 + 4);
      gx[0] = g0.x; gx[1] = g0.y; gx[2] = g0.z; gx[3] = g0.w; gx[4] = g1.x; gx[5] = g1.y; gx[6] = g1.z; gx[7] = g1.w;
      px[0] = p0.x; px[1] = p0.y; px[2] = p0.z; px[3] = p0.w; px[4] = p1.x; px[5] = p1.y; px[6] = p1.z; px[7] = p1.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        gx[k] = (e0 + k < n) ? a.g[e0 + k] : 0.0f;
        px[k] = (e0 + k < n) ? a.p[e0 + k] : 0.0f;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const long long e = e0 + k;
      m[k] = 0.0f;
      v[k] = 0.0f;
      if (e < n) {
        const float g = gx[k];
        float m0 = 0.0f, v0 = 0.0f;
        if (!a.first) {
          if (MM == LPMM_B200_STATE_GROUP4) m0 = __fmul_rn(M.qm[(mcodes >> (4 * k)) & 15u], sm);
          else m0 = reinterpret_cast<const float*>(a.m)[e];
          if (VM == LPMM_B200_STATE_GROUP4) v0 = __fmul_rn(M.qv[(vcodes >> (4 * k)) & 15u], sv);
          else if (VM == LPMM_B200_STATE_RANK1_4)
            v0 = __fmul_rn(M.qv[(vcodes >> (4 * k)) & 15u], st_old[k]);
          else if (VM == LPMM_B200_STATE_FP32) v0 = reinterpret_cast<const float*>(a.v)[e];
        }
        m[k] = lerp_m(c, m0, g);
        if (VM == LPMM_B200_STATE_FACTORED) {
          const float rf = __fdiv_rn(a.row[rowi], a.row_mean[bi]);
          v[k] = __fmul_rn(rf, a.col[bi * C + cc]);
        } else {
          v[k] = upd_v2(c, v0, g);
        }
        px[k] = upd_param(c, px[k], m[k], v[k]);
        am = fmaxf(am, fabsf(m[k]));
        av = fmaxf(av, v[k]);
        if (MM == LPMM_B200_STATE_FP32) reinterpret_cast<float*>(a.m)[e] = m[k];
        if (VM == LPMM_B200_STATE_FP32) reinterpret_cast<float*>(a.v)[e] = v[k];
      }
      if (VM == LPMM_B200_STATE_FACTORED && ++cc == C) {
        cc = 0;
        ++rowi;
        bi = rowi / a.s.dim[a.s.nd - 2];
      }
    }
    if (full) {
      *reinterpret_cast<float4*>(a.p + e0) = make_float4(px[0], px[1], px[2], px[3]);
      *reinterpret_cast<float4*>(a.p + e0 + 4) = make_float4(px[4], px[5], px[6], px[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (e0 + k < n) a.p[e0 + k] = px[k];
    }
    if (MM == LPMM_B200_STATE_GROUP4) {
      am = hmax16(am, hmask);
      // padding inside the last group is 0 / max
      *reinterpret_cast<uint32_t*>(mb) = codes_by_group_scale(M.mm, m, am);
      if (l16 == 0) a.m_max1[u] = am;
    }
    if (VM == LPMM_B200_STATE_GROUP4) {
      av = hmax16(av, hmask);
      *reinterpret_cast<uint32_t*>(vb) = codes_by_group_scale(M.mv, v, av);
      if (l16 == 0) a.v_max1[u] = av;
    }
    if (VM == LPMM_B200_STATE_RANK1_4) {
      uint32_t out = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int code = (e0 + k < n) ? code16(M.mv, __fdiv_rn(v[k], st_new[k])) : M.zero_v;
        out |= (uint32_t)(code & 15) << (4 * k);
      }
      *reinterpret_cast<uint32_t*>(vb) = out;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {  // the trailing byte of the packed layout
    if (MM == LPMM_B200_STATE_GROUP4) reinterpret_cast<uint8_t*>(a.m)[a.units * 64] = 0;
    if (VM == LPMM_B200_STATE_GROUP4 || VM == LPMM_B200_STATE_RANK1_4)
      reinterpret_cast<uint8_t*>(a.v)[a.units * 64] = 0;
  }
}

// Statistics pass of the rank-1 second moment: recompute v exactly as the update pass will and
// fold it into the (zeroed) per-axis maxima.  The innermost axis changes with every element, so
// its maxima are first combined in shared memory (when the axis has at most STAT_LAST entries) and
// flushed once per CTA; the outer axes change rarely along a lane's 8 consecutive elements, so a
// lane combines runs of equal coordinates in registers before touching global memory.
constexpr int STAT_LAST = 8192;
template <int ND>
__global__ void __launch_bounds__(UT) rank1_stats_kernel(const StepArgs a, const UConsts c,
                                                          const float* __restrict__ qmap_v) {
  __shared__ Maps M;
  __shared__ int lastmax[STAT_LAST];
  load_maps(M, nullptr, qmap_v);
  const int nd = a.s.nd;
  const int last = nd - 1;
  const bool use_smem = a.s.dim[last] <= STAT_LAST;
  if (use_smem) {
    for (int i = threadIdx.x; i < (int)a.s.dim[last]; i += UT) lastmax[i] = 0;
    __syncthreads();
  }
  const long long n = a.n;
  const long long nchunks = (n + 7) / 8;
  for (long long ch = (long long)blockIdx.x * UT + threadIdx.x; ch < nchunks; ch += (long long)gridDim.x * UT) {
    const long long e0 = ch * 8;
    uint32_t vcodes = 0;
    if (!a.first) vcodes = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.v) + (e0 >> 1));
    float gx[8];
    if (a.vec_ok && e0 + 8 <= n) {
      const float4 g0 = *reinterpret_cast<const float4*>(a.g + e0), g1 = *reinterpret_cast<const float4*>(a.g + e0 + 4);
      gx[0] = g0.x; gx[1] = g0.y; gx[2] = g0.z; gx[3] = g0.w; gx[4] = g1.x; gx[5] = g1.y; gx[6] = g1.z; gx[7] = g1.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) gx[k] = (e0 + k < n) ? a.g[e0 + k] : 0.0f;
    }
    int co[8], run_co[8];
    float run_max[8], st_old[8];
    if (!a.first) lane_scales<ND>(a.v_old, e0, n, a.s, st_old);
    decompose<ND>(e0, a.s, co);
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      run_co[i] = co[i];
      run_max[i] = 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (e0 + k < n) {
        float v0 = 0.0f;
        if (!a.first) v0 = __fmul_rn(M.qv[(vcodes >> (4 * k)) & 15u], st_old[k]);
        const float v = upd_v2(c, v0, gx[k]);
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          if (ND < 8 || i < nd) {
            if (i == last && use_smem) {
              if (__float_as_int(v) > lastmax[co[i]]) atomicMax(&lastmax[co[i]], __float_as_int(v));
            } else {
              if (co[i] != run_co[i]) {
                atomic_max_nonneg(a.v_new[i] + run_co[i], run_max[i]);
                run_co[i] = co[i];
                run_max[i] = 0.0f;
              }
              run_max[i] = fmaxf(run_max[i], v);
            }
          }
        }
        advance<ND>(co, a.s);
      }
    }
#pragma unroll
    for (int i = 0; i < ND; ++i)
      if ((ND < 8 || i < nd) && !(i == last && use_smem)) atomic_max_nonneg(a.v_new[i] + run_co[i], run_max[i]);
  }
  if (use_smem) {
    __syncthreads();
    for (int i = threadIdx.x; i < (int)a.s.dim[last]; i += UT)
      atomic_max_nonneg(a.v_new[last] + i, __int_as_float(lastmax[i]));
  }
}

// The same statistics pass for a matrix whose row length is a multiple of 8: a thread keeps its 8
// columns for all the rows of its CTA, so column maxima live in registers and reach global memory
// once per CTA; a row's maximum is reduced across the warp and costs one atomic per warp and row.
__global__ void __launch_bounds__(UT) rank1_stats2d_kernel(const StepArgs a, const UConsts c,
                                                            const float* __restrict__ qmap_v, int rows_per_cta) {
  __shared__ Maps M;
  load_maps(M, nullptr, qmap_v);
  const long long R = a.s.dim[0], C = a.s.dim[1];
  const long long c0 = ((long long)blockIdx.x * UT + threadIdx.x) * 8;
  const bool active = c0 < C;
  float col_old[8], col_max[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    col_old[k] = (active && !a.first) ? __ldg(a.v_old[1] + c0 + k) : 0.0f;
    col_max[k] = 0.0f;
  }
  const long long r_begin = (long long)blockIdx.y * rows_per_cta;
  const long long r_end = (r_begin + rows_per_cta < R) ? r_begin + rows_per_cta : R;
  for (long long r = r_begin; r < r_end; ++r) {
    float row_max = 0.0f;
    if (active) {
      const long long e0 = r * C + c0;
      const float4 g0 = *reinterpret_cast<const float4*>(a.g + e0), g1 = *reinterpret_cast<const float4*>(a.g + e0 + 4);
      const float gx[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      uint32_t vcodes = 0;
      float row_old = 0.0f;
      if (!a.first) {
        vcodes = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.v) + (e0 >> 1));
        row_old = __ldg(a.v_old[0] + r);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float v0 = a.first ? 0.0f : __fmul_rn(M.qv[(vcodes >> (4 * k)) & 15u], fminf(row_old, col_old[k]));
        const float v = upd_v2(c, v0, gx[k]);
        col_max[k] = fmaxf(col_max[k], v);
        row_max = fmaxf(row_max, v);
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    if ((threadIdx.x & 31) == 0) atomic_max_nonneg(a.v_new[0] + r, row_max);
  }
  if (active) {
#pragma unroll
    for (int k = 0; k < 8; ++k) atomic_max_nonneg(a.v_new[1] + c0 + k, col_max[k]);
  }
}

// ---------------------------------------------------------------------------------------------
// Factored second moment: row / column means of g^2, fixed summation order.
// ---------------------------------------------------------------------------------------------
// One warp per row of the [B*R, C] view: row = fma(1-beta2, mean_c(g^2), row*beta2).
__global__ void factored_rows_kernel(const float* __restrict__ g, float* __restrict__ row, long long rows,
                                     long long C, UConsts c) {
  const int lane = threadIdx.x & 31;
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows;
       r += (long long)gridDim.x * (blockDim.x >> 5)) {
    const float* gr = g + r * C;
    float acc = 0.0f;
    for (long long j = lane; j < C; j += 32) {
      const float x = gr[j];
      acc = __fadd_rn(acc, __fmul_rn(x, x));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (lane == 0) row[r] = __fmaf_rn(c.omb2, __fdiv_rn(acc, (float)C), __fmul_rn(row[r], c.beta2));
  }
}
// Column partial sums over tiles of TR rows: partial[(b*tiles + t)*C + col].
constexpr int TR = 64;
__global__ void factored_cols_partial_kernel(const float* __restrict__ g, float* __restrict__ partial, long long B,
                                             long long R, long long C) {
  const long long tiles = (R + TR - 1) / TR;
  const long long total = B * tiles * C;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long col = idx % C;
    const long long t = (idx / C) % tiles;
    const long long b = idx / (C * tiles);
    const long long r0 = t * TR, r1 = (r0 + TR < R) ? r0 + TR : R;
    const float* gp = g + (b * R) * C + col;
    float acc = 0.0f;
    for (long long r = r0; r < r1; ++r) {
      const float x = gp[r * C];
      acc = __fadd_rn(acc, __fmul_rn(x, x));
    }
    partial[idx] = acc;
  }
}
__global__ void factored_cols_final_kernel(const float* __restrict__ partial, float* __restrict__ col, long long B,
                                           long long R, long long C, UConsts c) {
  const long long tiles = (R + TR - 1) / TR;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < B * C;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / C, cc = idx % C;
    float acc = 0.0f;
    for (long long t = 0; t < tiles; ++t) acc = __fadd_rn(acc, partial[(b * tiles + t) * C + cc]);
    col[idx] = __fmaf_rn(c.omb2, __fdiv_rn(acc, (float)R), __fmul_rn(col[idx], c.beta2));
  }
}
// Mean over R of the updated row accumulator, one CTA per batch entry.
__global__ void factored_row_mean_kernel(const float* __restrict__ row, float* __restrict__ row_mean, long long R) {
  __shared__ float red[256];
  const float* rb = row + (long long)blockIdx.x * R;
  float acc = 0.0f;
  for (long long j = threadIdx.x; j < R; j += blockDim.x) acc = __fadd_rn(acc, rb[j]);
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) row_mean[blockIdx.x] = __fdiv_rn(red[0], (float)R);
}

// ---------------------------------------------------------------------------------------------
// Momentum SGD, non-fused semantics (sgd.py:152-187).
// ---------------------------------------------------------------------------------------------
struct SgdConsts {
  float wd, momentum, omd, neg_lr;
  int has_wd, has_momentum, nesterov, maximize;
};

template <int BM>
__global__ void __launch_bounds__(UT) sgd_kernel(float* __restrict__ p, const float* __restrict__ g, long long n,
                                                  long long units, void* buf, float* __restrict__ buf_max1,
                                                  int first, const float* __restrict__ qmap, const SgdConsts c) {
  __shared__ Maps M;
  load_maps(M, qmap, nullptr);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long real_units = (n + 127) / 128;
  for (long long u = (long long)blockIdx.x * (UT / 16) + (threadIdx.x >> 4); u < units;
       u += (long long)gridDim.x * (UT / 16)) {
    const long long e0 = u * 128 + l16 * 8;
    uint8_t* bb = (BM == LPMM_B200_STATE_GROUP4 && c.has_momentum) ? reinterpret_cast<uint8_t*>(buf) + (e0 >> 1)
                                                                    : nullptr;
    if (u >= real_units) {
      if (bb) *reinterpret_cast<uint32_t*>(bb) = 0x11111111u * (uint32_t)M.zero_m;
      continue;
    }
    uint32_t codes = 0;
    float sc = 0.0f;
    if (bb && !first) {
      codes = *reinterpret_cast<const uint32_t*>(bb);
      sc = buf_max1[u];
    }
    float b[8];
    float ab = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const long long e = e0 + k;
      b[k] = 0.0f;
      if (e < n) {
        float d = c.maximize ? -g[e] : g[e];
        const float pe = p[e];
        if (c.has_wd) d = __fmaf_rn(c.wd, pe, d);                      // d_p.add(param, alpha=wd)
        if (c.has_momentum) {
          float bv;
          if (first) {
            bv = d;                                                    // clone of d_p
          } else {
            const float b0 = (BM == LPMM_B200_STATE_GROUP4) ? __fmul_rn(M.qm[(codes >> (4 * k)) & 15u], sc)
                                                            : reinterpret_cast<const float*>(buf)[e];
            bv = __fmaf_rn(c.omd, d, __fmul_rn(b0, c.momentum));       // mul_(momentum).add_(d_p, alpha=1-dampening)
          }
          b[k] = bv;
          ab = fmaxf(ab, fabsf(bv));
          if (BM == LPMM_B200_STATE_FP32) reinterpret_cast<float*>(buf)[e] = bv;
          d = c.nesterov ? __fmaf_rn(c.momentum, bv, d) : bv;
        }
        p[e] = __fmaf_rn(c.neg_lr, d, pe);                             // param.add_(d_p, alpha=-lr)
      }
    }
    if (bb) {
      ab = hmax16(ab, hmask);
      *reinterpret_cast<uint32_t*>(bb) = codes_by_group_scale(M.mm, b, ab);
      if (l16 == 0) buf_max1[u] = ab;
    }
  }
  if (BM == LPMM_B200_STATE_GROUP4 && c.has_momentum && blockIdx.x == 0 && threadIdx.x == 0)
    reinterpret_cast<uint8_t*>(buf)[units * 64] = 0;
}

// ---------------------------------------------------------------------------------------------
// Standalone quantize / dequantize
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(UT) pack4_kernel(const float* __restrict__ x, long long n,
                                                    const float* __restrict__ qmap, uint8_t* __restrict__ out) {
  __shared__ Maps M;
  load_maps(M, qmap, nullptr);
  const long long nb = n / 2;
  for (long long b = (long long)blockIdx.x * UT + threadIdx.x; b < nb; b += (long long)gridDim.x * UT) {
    const float2 xy = *reinterpret_cast<const float2*>(x + 2 * b);
    out[b] = (uint8_t)(code16(M.mm, xy.x) | (code16(M.mm, xy.y) << 4));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) out[nb] = 0;
}
__global__ void __launch_bounds__(UT) unpack4_kernel(const uint8_t* __restrict__ in, long long n,
                                                      const float* __restrict__ qmap, float* __restrict__ out) {
  __shared__ Maps M;
  load_maps(M, qmap, nullptr);
  const long long nb = n / 2;
  for (long long b = (long long)blockIdx.x * UT + threadIdx.x; b < nb; b += (long long)gridDim.x * UT) {
    const uint8_t c = in[b];
    *reinterpret_cast<float2*>(out + 2 * b) = make_float2(M.qm[c & 15], M.qm[c >> 4]);
  }
}
// mode 0: group-128 scales (computes max1); mode 1: rank-1 scales from given per-axis maxima.
template <int MODE, int ND>
__global__ void __launch_bounds__(UT) quant_kernel(const float* __restrict__ x, long long n, long long units,
                                                    const float* __restrict__ qmap, uint8_t* __restrict__ codes,
                                                    float* __restrict__ max1, const StepArgs a) {
  __shared__ Maps M;
  load_maps(M, qmap, nullptr);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long real_units = (n + 127) / 128;
  for (long long u = (long long)blockIdx.x * (UT / 16) + (threadIdx.x >> 4); u < units;
       u += (long long)gridDim.x * (UT / 16)) {
    const long long e0 = u * 128 + l16 * 8;
    uint32_t* cb = reinterpret_cast<uint32_t*>(codes + (e0 >> 1));
    if (u >= real_units) {
      *cb = 0x11111111u * (uint32_t)M.zero_m;
      continue;
    }
    float xv[8], st[8];
    float ax = 0.0f;
    int co[8];
    if (MODE == 1) decompose<ND>(e0, a.s, co);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      xv[k] = 0.0f;
      st[k] = 1.0f;
      if (e0 + k < n) {
        xv[k] = x[e0 + k];
        ax = fmaxf(ax, fabsf(xv[k]));
        if (MODE == 1) st[k] = axis_min<ND>(a.v_new, co, a.s.nd);
      }
      if (MODE == 1) advance<ND>(co, a.s);
    }
    uint32_t out = 0;
    if (MODE == 0) {
      ax = hmax16(ax, hmask);
      out = codes_by_group_scale(M.mm, xv, ax);
      if (l16 == 0) max1[u] = ax;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int code = (e0 + k < n) ? code16(M.mm, __fdiv_rn(xv[k], st[k])) : M.zero_m;
        out |= (uint32_t)(code & 15) << (4 * k);
      }
    }
    *cb = out;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) codes[units * 64] = 0;
}
template <int MODE, int ND>
__global__ void __launch_bounds__(UT) dequant_kernel(const uint8_t* __restrict__ codes, long long n,
                                                      const float* __restrict__ qmap,
                                                      const float* __restrict__ max1, float* __restrict__ out,
                                                      const StepArgs a) {
  __shared__ Maps M;
  load_maps(M, qmap, nullptr);
  const long long nchunks = (n + 7) / 8;
  for (long long ch = (long long)blockIdx.x * UT + threadIdx.x; ch < nchunks; ch += (long long)gridDim.x * UT) {
    const long long e0 = ch * 8;
    const uint32_t c = *reinterpret_cast<const uint32_t*>(codes + (e0 >> 1));
    int co[8];
    if (MODE == 1) decompose<ND>(e0, a.s, co);
    const float s0 = (MODE == 0) ? max1[e0 >> 7] : 0.0f;
    for (int k = 0; k < 8; ++k) {
      if (e0 + k >= n) break;
      const float sc = (MODE == 0) ? s0 : axis_min<ND>(a.v_old, co, a.s.nd);
      out[e0 + k] = __fmul_rn(M.qm[(c >> (4 * k)) & 15u], sc);
      if (MODE == 1) advance<ND>(co, a.s);
    }
  }
}
template <int ND>
__global__ void __launch_bounds__(UT) axis_absmax_kernel(const float* __restrict__ x, const StepArgs a) {
  const long long n = a.n;
  const long long nchunks = (n + 7) / 8;
  for (long long ch = (long long)blockIdx.x * UT + threadIdx.x; ch < nchunks; ch += (long long)gridDim.x * UT) {
    const long long e0 = ch * 8;
    int co[8];
    decompose<ND>(e0, a.s, co);
    for (int k = 0; k < 8; ++k) {
      if (e0 + k >= n) break;
      const float v = fabsf(x[e0 + k]);
#pragma unroll
      for (int i = 0; i < ND; ++i)
        if (ND < 8 || i < a.s.nd) atomic_max_nonneg(a.v_new[i] + co[i], v);
      advance<ND>(co, a.s);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// Calls `expr` with ND bound to the instantiation that serves `nd` axes: exact for 2, 3, 4, generic for 5..8.
#define LPMM_DISPATCH_ND(nd, ...)        \
  do {                                   \
    if ((nd) == 2) { constexpr int ND = 2; __VA_ARGS__; }        \
    else if ((nd) == 3) { constexpr int ND = 3; __VA_ARGS__; }   \
    else if ((nd) == 4) { constexpr int ND = 4; __VA_ARGS__; }   \
    else { constexpr int ND = 8; __VA_ARGS__; }                  \
  } while (0)
static inline long long pad_to(long long n, long long m) { return (n + m - 1) / m * m; }
static inline unsigned grid_for(long long work_items, int per_cta, int ctas_per_sm = 8) {
  long long g = (work_items + per_cta - 1) / per_cta;
  const long long cap = (long long)num_sms() * ctas_per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (unsigned)g;
}
static int fill_shape(Shape& s, const int64_t* shape, int ndim, long long* numel_out) {
  if (ndim < 1 || ndim > 8 || !shape) return LPMM_B200_ERR_BAD_SIZE;
  s.nd = ndim;
  long long n = 1;
  for (int i = 0; i < 8; ++i) {
    s.dim[i] = i < ndim ? shape[i] : 1;
    if (i < ndim) {
      if (shape[i] < 0 || shape[i] > 0x7fffffffLL) return LPMM_B200_ERR_BAD_SIZE;
      n *= shape[i];
    }
  }
  *numel_out = n;
  return LPMM_B200_OK;
}
static UConsts make_consts(double beta1, double beta2, double lr, double wd, double eps, double step) {
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
  c.fast = (eps >= 0x1p-40 && eps <= 0x1p30 && bc2 >= 0x1p-40);
  return c;
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

extern "C" int64_t lpmm_b200_packed_len(int64_t n_scaled) {
  if (n_scaled < 0) return LPMM_B200_ERR_BAD_SIZE;
  return pad_to(n_scaled, 2048) / 2 + 1;
}

extern "C" int lpmm_b200_pack_nonlinear4(const float* data, int64_t n, const float* qmap, int8_t* packed,
                                         void* stream) {
  if (n < 0 || (n & 1)) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !packed || (n > 0 && !data)) return LPMM_B200_ERR_NULL_POINTER;
  pack4_kernel<<<grid_for(n / 2, UT), UT, 0, (cudaStream_t)stream>>>(data, n, qmap, (uint8_t*)packed);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_unpack_nonlinear4(const int8_t* packed, const float* qmap, int64_t n, float* out,
                                           void* stream) {
  if (n < 0 || (n & 1)) return LPMM_B200_ERR_BAD_SIZE;
  if (n == 0) return LPMM_B200_OK;
  if (!qmap || !packed || !out) return LPMM_B200_ERR_NULL_POINTER;
  unpack4_kernel<<<grid_for(n / 2, UT), UT, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, n, qmap, out);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_quant_group4(const float* x, int64_t numel, const float* qmap, int8_t* codes, float* max1,
                                      void* stream) {
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !codes || (numel > 0 && (!x || !max1))) return LPMM_B200_ERR_NULL_POINTER;
  StepArgs a = {};
  const long long units = pad_to(pad_to(numel, 128), 2048) / 128;
  quant_kernel<0, 2><<<grid_for(units, UT / 16), UT, 0, (cudaStream_t)stream>>>(x, numel, units, qmap, (uint8_t*)codes,
                                                                            max1, a);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_dequant_group4(const int8_t* codes, const float* qmap, const float* max1, int64_t numel,
                                        float* out, void* stream) {
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (numel == 0) return LPMM_B200_OK;
  if (!qmap || !codes || !max1 || !out) return LPMM_B200_ERR_NULL_POINTER;
  StepArgs a = {};
  dequant_kernel<0, 2><<<grid_for((numel + 7) / 8, UT), UT, 0, (cudaStream_t)stream>>>((const uint8_t*)codes, numel,
                                                                                   qmap, max1, out, a);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

static int zero_axes(const Shape& s, float* const* vecs, cudaStream_t st) {
  for (int i = 0; i < s.nd; ++i) {
    if (!vecs[i]) return LPMM_B200_ERR_NULL_POINTER;
    LPMM_CUDA_TRY(cudaMemsetAsync(vecs[i], 0, sizeof(float) * (size_t)s.dim[i], st));
  }
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_axis_absmax(const float* x, const int64_t* shape, int ndim, float* const* max_dims,
                                     void* stream) {
  StepArgs a = {};
  int rc = fill_shape(a.s, shape, ndim, &a.n);
  if (rc) return rc;
  if (!max_dims || (a.n > 0 && !x)) return LPMM_B200_ERR_NULL_POINTER;
  for (int i = 0; i < ndim; ++i) a.v_new[i] = max_dims[i];
  rc = zero_axes(a.s, max_dims, (cudaStream_t)stream);
  if (rc) return rc;
  if (a.n == 0) return LPMM_B200_OK;
  LPMM_DISPATCH_ND(ndim, (axis_absmax_kernel<ND><<<grid_for((a.n + 7) / 8, UT), UT, 0, (cudaStream_t)stream>>>(x, a)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_quant_rank1_4(const float* x, const int64_t* shape, int ndim, const float* qmap,
                                       float* const* max_dims, int8_t* codes, void* stream) {
  if (ndim < 2) return LPMM_B200_ERR_BAD_SIZE;
  int rc = lpmm_b200_axis_absmax(x, shape, ndim, max_dims, stream);
  if (rc) return rc;
  if (!qmap || !codes) return LPMM_B200_ERR_NULL_POINTER;
  StepArgs a = {};
  fill_shape(a.s, shape, ndim, &a.n);
  for (int i = 0; i < ndim; ++i) a.v_new[i] = max_dims[i];
  const long long units = pad_to(a.n, 2048) / 128;
  LPMM_DISPATCH_ND(ndim, (quant_kernel<1, ND><<<grid_for(units, UT / 16), UT, 0, (cudaStream_t)stream>>>(
                              x, a.n, units, qmap, (uint8_t*)codes, nullptr, a)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_dequant_rank1_4(const int8_t* codes, const float* qmap, const float* const* max_dims,
                                         const int64_t* shape, int ndim, float* out, void* stream) {
  if (ndim < 2) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  int rc = fill_shape(a.s, shape, ndim, &a.n);
  if (rc) return rc;
  if (a.n == 0) return LPMM_B200_OK;
  if (!qmap || !codes || !max_dims || !out) return LPMM_B200_ERR_NULL_POINTER;
  for (int i = 0; i < ndim; ++i) {
    if (!max_dims[i]) return LPMM_B200_ERR_NULL_POINTER;
    a.v_old[i] = max_dims[i];
  }
  LPMM_DISPATCH_ND(ndim, (dequant_kernel<1, ND><<<grid_for((a.n + 7) / 8, UT), UT, 0, (cudaStream_t)stream>>>(
                              (const uint8_t*)codes, a.n, qmap, nullptr, out, a)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int64_t lpmm_b200_factored_scratch_bytes(const int64_t* shape, int ndim) {
  if (ndim < 2 || ndim > 8 || !shape) return LPMM_B200_ERR_BAD_SIZE;
  long long B = 1;
  for (int i = 0; i < ndim - 2; ++i) B *= shape[i];
  const long long R = shape[ndim - 2], C = shape[ndim - 1];
  const long long tiles = (R + TR - 1) / TR;
  return (int64_t)sizeof(float) * (B * tiles * C + B);
}

template <int MM>
static cudaError_t launch_unfused(int vm, unsigned grid, cudaStream_t st, const StepArgs& a, const UConsts& c,
                                  const float* qm, const float* qv) {
  switch (vm) {
    case LPMM_B200_STATE_FP32: unfused_adamw_kernel<MM, LPMM_B200_STATE_FP32, 2><<<grid, UT, 0, st>>>(a, c, qm, qv); break;
    case LPMM_B200_STATE_GROUP4: unfused_adamw_kernel<MM, LPMM_B200_STATE_GROUP4, 2><<<grid, UT, 0, st>>>(a, c, qm, qv); break;
    case LPMM_B200_STATE_RANK1_4:
      LPMM_DISPATCH_ND(a.s.nd, (unfused_adamw_kernel<MM, LPMM_B200_STATE_RANK1_4, ND><<<grid, UT, 0, st>>>(a, c, qm, qv)));
      break;
    default: unfused_adamw_kernel<MM, LPMM_B200_STATE_FACTORED, 2><<<grid, UT, 0, st>>>(a, c, qm, qv); break;
  }
  return cudaGetLastError();
}

extern "C" int lpmm_b200_adamw4bit_unfused_step(const lpmm_b200_step_tensor* t, const float* qmap_m,
                                                const float* qmap_v, double beta1, double beta2, double lr,
                                                double weight_decay, double eps, double step, void* scratch,
                                                int64_t scratch_bytes, void* stream) {
  if (!t) return LPMM_B200_ERR_NULL_POINTER;
  if (t->numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (t->numel == 0) return LPMM_B200_OK;
  if (!t->p || !t->g) return LPMM_B200_ERR_NULL_POINTER;
  if (t->m_mode != LPMM_B200_STATE_FP32 && t->m_mode != LPMM_B200_STATE_GROUP4) return LPMM_B200_ERR_BAD_KIND;
  if (t->v_mode < LPMM_B200_STATE_FP32 || t->v_mode > LPMM_B200_STATE_FACTORED) return LPMM_B200_ERR_BAD_KIND;
  if (!t->m) return LPMM_B200_ERR_NULL_POINTER;
  if (t->m_mode == LPMM_B200_STATE_GROUP4 && (!t->m_max1 || !qmap_m)) return LPMM_B200_ERR_NULL_POINTER;
  cudaStream_t st = (cudaStream_t)stream;
  StepArgs a = {};
  a.p = t->p;
  a.g = t->g;
  a.n = t->numel;
  a.first = t->first;
  a.vec_ok = ((((uintptr_t)t->p | (uintptr_t)t->g) & 15) == 0);
  a.m = t->m;
  a.m_max1 = t->m_max1;
  a.v = t->v;
  a.v_max1 = t->v_max1;
  a.row = t->row;
  a.col = t->col;
  a.s.nd = 1;
  a.s.dim[0] = t->numel;
  a.units = pad_to(pad_to(a.n, 128), 2048) / 128;
  const UConsts c = make_consts(beta1, beta2, lr, weight_decay, eps, step);
  if (t->v_mode == LPMM_B200_STATE_RANK1_4 || t->v_mode == LPMM_B200_STATE_FACTORED) {
    long long n2 = 0;
    int rc = fill_shape(a.s, t->shape, t->ndim, &n2);
    if (rc) return rc;
    if (t->ndim < 2 || n2 != t->numel) return LPMM_B200_ERR_BAD_SIZE;
  }
  if (t->v_mode == LPMM_B200_STATE_FP32 || t->v_mode == LPMM_B200_STATE_GROUP4 || t->v_mode == LPMM_B200_STATE_RANK1_4) {
    if (!t->v) return LPMM_B200_ERR_NULL_POINTER;
    if (t->v_mode != LPMM_B200_STATE_FP32 && !qmap_v) return LPMM_B200_ERR_NULL_POINTER;
    if (t->v_mode == LPMM_B200_STATE_GROUP4 && !t->v_max1) return LPMM_B200_ERR_NULL_POINTER;
  }
  if (t->v_mode == LPMM_B200_STATE_RANK1_4) {
    for (int i = 0; i < t->ndim; ++i) {
      if (!t->v_max_dims_new[i] || (!t->first && !t->v_max_dims_old[i])) return LPMM_B200_ERR_NULL_POINTER;
      a.v_old[i] = t->v_max_dims_old[i];
      a.v_new[i] = t->v_max_dims_new[i];
    }
    int rc = zero_axes(a.s, t->v_max_dims_new, st);
    if (rc) return rc;
    if (t->ndim == 2 && t->shape[1] % 8 == 0 && a.vec_ok && (((uintptr_t)t->v & 3) == 0)) {
      const long long R = t->shape[0], C = t->shape[1];
      const long long col_ctas = (C / 8 + UT - 1) / UT;
      long long row_ctas = ((long long)num_sms() * 6 + col_ctas - 1) / col_ctas;
      if (row_ctas > R) row_ctas = R;
      if (row_ctas > 65535) row_ctas = 65535;
      const int rows_per_cta = (int)((R + row_ctas - 1) / row_ctas);
      row_ctas = (R + rows_per_cta - 1) / rows_per_cta;
      rank1_stats2d_kernel<<<dim3((unsigned)col_ctas, (unsigned)row_ctas), UT, 0, st>>>(a, c, qmap_v, rows_per_cta);
    } else {
      LPMM_DISPATCH_ND(t->ndim, (rank1_stats_kernel<ND><<<grid_for((a.n + 7) / 8, UT, 3), UT, 0, st>>>(a, c, qmap_v)));
    }
    LPMM_CUDA_TRY(cudaGetLastError());
  }
  if (t->v_mode == LPMM_B200_STATE_FACTORED) {
    if (!t->row || !t->col) return LPMM_B200_ERR_NULL_POINTER;
    const int64_t need = lpmm_b200_factored_scratch_bytes(t->shape, t->ndim);
    if (!scratch) return LPMM_B200_ERR_NULL_POINTER;
    if (scratch_bytes < need) return LPMM_B200_ERR_BAD_SIZE;
    long long B = 1;
    for (int i = 0; i < t->ndim - 2; ++i) B *= t->shape[i];
    const long long R = t->shape[t->ndim - 2], C = t->shape[t->ndim - 1];
    const long long tiles = (R + TR - 1) / TR;
    float* partial = reinterpret_cast<float*>(scratch);
    float* row_mean = partial + B * tiles * C;
    factored_rows_kernel<<<grid_for(B * R, 8), 256, 0, st>>>(t->g, t->row, B * R, C, c);
    LPMM_CUDA_TRY(cudaGetLastError());
    factored_cols_partial_kernel<<<grid_for(B * tiles * C, 256), 256, 0, st>>>(t->g, partial, B, R, C);
    LPMM_CUDA_TRY(cudaGetLastError());
    factored_cols_final_kernel<<<grid_for(B * C, 256), 256, 0, st>>>(partial, t->col, B, R, C, c);
    LPMM_CUDA_TRY(cudaGetLastError());
    factored_row_mean_kernel<<<(unsigned)B, 256, 0, st>>>(t->row, row_mean, R);
    LPMM_CUDA_TRY(cudaGetLastError());
    a.row_mean = row_mean;
  }
  const unsigned grid = grid_for(a.units, UT / 16);
  cudaError_t e = (t->m_mode == LPMM_B200_STATE_GROUP4) ? launch_unfused<LPMM_B200_STATE_GROUP4>(t->v_mode, grid, st, a, c, qmap_m, qmap_v)
                                                       : launch_unfused<LPMM_B200_STATE_FP32>(t->v_mode, grid, st, a, c, qmap_m, qmap_v);
  LPMM_CUDA_TRY(e);
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_sgd4bit_step(float* p, const float* g, int64_t numel, void* buf, float* buf_max1,
                                      int buf_mode, int first, const float* qmap, double weight_decay,
                                      double momentum, double lr, double dampening, int nesterov, int maximize,
                                      void* stream) {
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (numel == 0) return LPMM_B200_OK;
  if (!p || !g) return LPMM_B200_ERR_NULL_POINTER;
  if (buf_mode != LPMM_B200_STATE_FP32 && buf_mode != LPMM_B200_STATE_GROUP4) return LPMM_B200_ERR_BAD_KIND;
  SgdConsts c;
  c.wd = (float)weight_decay;
  c.momentum = (float)momentum;
  c.omd = (float)(1.0 - dampening);
  c.neg_lr = (float)(-lr);
  c.has_wd = weight_decay != 0.0;
  c.has_momentum = momentum != 0.0;
  c.nesterov = nesterov;
  c.maximize = maximize;
  if (c.has_momentum) {
    if (!buf) return LPMM_B200_ERR_NULL_POINTER;
    if (buf_mode == LPMM_B200_STATE_GROUP4 && (!buf_max1 || !qmap)) return LPMM_B200_ERR_NULL_POINTER;
  }
  const long long units = pad_to(pad_to(numel, 128), 2048) / 128;
  const unsigned grid = grid_for(units, UT / 16);
  if (buf_mode == LPMM_B200_STATE_GROUP4)
    sgd_kernel<LPMM_B200_STATE_GROUP4><<<grid, UT, 0, (cudaStream_t)stream>>>(p, g, numel, units, buf, buf_max1, first, qmap, c);
  else
    sgd_kernel<LPMM_B200_STATE_FP32><<<grid, UT, 0, (cudaStream_t)stream>>>(p, g, numel, units, buf, buf_max1, first, qmap, c);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Factored step without any allocation: the scratch lives in the library image.
// ---------------------------------------------------------------------------------------------
// Device-resident scratch of the allocation-free entry point.  In host code this name is only a
// handle for cudaGetSymbolAddress; it is not itself a device address.
static __device__ __align__(256) unsigned char g_static_scratch[LPMM_B200_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
static int static_scratch_address(void** out) {
  static void* addr[64] = {};
  int dev = -1;
  LPMM_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return LPMM_B200_ERR_UNSUPPORTED;
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    LPMM_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    addr[dev] = p;  // concurrent first calls store the same value
  }
  *out = addr[dev];
  return LPMM_B200_OK;
}

// For callers that may not allocate: same launches as the FACTORED branch of
// lpmm_b200_adamw4bit_unfused_step, scratch taken from g_static_scratch.  Every partial sum and
// row mean the kernels read is written earlier in the same call, so stale contents are harmless;
// calls that overlap on the GPU would overwrite each other's partial sums.
extern "C" int lpmm_b200_adamw4bit_factored_step_noalloc(const lpmm_b200_step_tensor* t, const float* qmap_m,
                                                         double beta1, double beta2, double lr, double weight_decay,
                                                         double eps, double step, void* stream) {
  if (!t) return LPMM_B200_ERR_NULL_POINTER;
  if (t->v_mode != LPMM_B200_STATE_FACTORED) return LPMM_B200_ERR_BAD_KIND;
  const int64_t need = lpmm_b200_factored_scratch_bytes(t->shape, t->ndim);
  if (need < 0) return (int)need;
  if (need > (int64_t)LPMM_B200_STATIC_SCRATCH_BYTES) return LPMM_B200_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != LPMM_B200_OK) return rc;
  return lpmm_b200_adamw4bit_unfused_step(t, qmap_m, nullptr, beta1, beta2, lr, weight_decay, eps, step, scratch,
                                          (int64_t)LPMM_B200_STATIC_SCRATCH_BYTES, stream);
}
