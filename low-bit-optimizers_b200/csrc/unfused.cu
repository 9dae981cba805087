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
// fused step.  Codes live in the reference's padded layout: n' = numel rounded up to the group
// size (group scales) or numel (rank-1 scales), rounded up again to rows of 2048 codes, plus one
// trailing byte.  4-bit maps pack two codes per byte (even element in the low nibble); maps of
// 5 to 8 bits store one code per byte ("wide", template parameter W).  A group of 128 elements is
// one half-warp; larger groups (256 ... 4096, powers of two) are 2 ... 32 adjacent half-warps of one
// CTA whose maxima are combined through shared memory.
#include <cooperative_groups.h>
#include <curand_kernel.h>
#include <math.h>

#include <mutex>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "multi_tensor.cuh"
#include "unfused_math.cuh"

namespace lpmm_b200 {

constexpr int UT = 256;     // threads per CTA
constexpr int UTMAX = 512;  // threads per CTA when a group spans 32 half-warps (4096 elements)

struct Shape {
  int nd;
  long long dim[8];
};

struct StepArgs {
  float* p;
  const float* g;
  long long n;
  long long units;  // loop bound: the larger of units_m and units_v
  long long units_m, units_v;  // padded length / 128 of each quantized state (0 when not quantized)
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
  int bits_m, bits_v;  // 4 ... 8
  int hpg_m, hpg_v;    // half-warps (128-element units) per group: group size / 128, a power of two
  int sh_m, sh_v;      // log2 of the above
};

struct Maps {
  float qm[256];
  float qv[256];
  float mm[256];  // midpoints of qm, padded with +inf
  float mv[256];
  int zero_m, zero_v;  // code of 0.0f in each map (what padding quantizes to)
  int linear_v;        // qv[i] == (i + 1) / 2^bits exactly: the closed-form code applies
};

// Nearest-code rule as a branch-free search over the sorted midpoints: code = #{midpoints < x}.
// A NaN gives what the reference's search gives: 15 in the packed 4-bit kernel, (uint8_t)-1 in the
// one-code-per-byte kernel (quantization_kernel.cu:398-427, :533).
template <bool W>
__device__ __forceinline__ int code_of(const float* __restrict__ mids, int bits, float x) {
  if (!W) return code16(mids, x);
  int c = 0;
  for (int s = 1 << (bits - 1); s; s >>= 1) c += (mids[c + s - 1] < x) ? s : 0;
  return (x != x) ? 255 : c;
}

// The 8 codes of a lane.  W = false: nibbles of one 32-bit word; W = true: bytes of two words.
template <bool W>
struct Codes8 {
  uint32_t lo, hi;
  __device__ __forceinline__ static long long byte_off(long long e0) { return W ? e0 : (e0 >> 1); }
  __device__ __forceinline__ static long long trailing(long long units) { return W ? units * 128 : units * 64; }
  __device__ __forceinline__ void clear() { lo = hi = 0u; }
  __device__ __forceinline__ void fill(int c) {
    lo = hi = (W ? 0x01010101u : 0x11111111u) * (uint32_t)c;
  }
  __device__ __forceinline__ void load(const uint8_t* p) {
    if (W) {
      const uint2 w = *reinterpret_cast<const uint2*>(p);
      lo = w.x;
      hi = w.y;
    } else {
      lo = *reinterpret_cast<const uint32_t*>(p);
      hi = 0u;
    }
  }
  __device__ __forceinline__ void store(uint8_t* p) const {
    if (W) *reinterpret_cast<uint2*>(p) = make_uint2(lo, hi);
    else *reinterpret_cast<uint32_t*>(p) = lo;
  }
  __device__ __forceinline__ int get(int k) const {
    if (W) return (int)(((k < 4 ? lo : hi) >> (8 * (k & 3))) & 255u);
    return (int)((lo >> (4 * k)) & 15u);
  }
  __device__ __forceinline__ void set(int k, int c) {  // into a cleared word
    if (W) {
      if (k < 4) lo |= (uint32_t)(c & 255) << (8 * k);
      else hi |= (uint32_t)(c & 255) << (8 * (k - 4));
    } else {
      lo |= (uint32_t)(c & 15) << (4 * k);
    }
  }
};

// x / d for the 8 values of a lane with a divisor shared by the group: the shared-reciprocal
// division (equal to IEEE division, see common.cuh) when d is in its domain, IEEE division otherwise.
template <bool W>
__device__ __forceinline__ Codes8<W> codes_by_group_scale(const float* __restrict__ mids, int bits, const float* x,
                                                          float d) {
  Codes8<W> out;
  out.clear();
  if (udiv_ok(d)) {
    const f2 r2 = f2_splat(rcp_nr(d)), nd2 = f2_splat(-d);
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // udiv on two elements per instruction
      const f2 xj = f2_pack(x[2 * j], x[2 * j + 1]);
      f2 q = f2_mul(xj, r2);
      q = f2_fma(f2_fma(q, nd2, xj), r2, q);
      float qa, qb;
      f2_unpack(q, qa, qb);
      out.set(2 * j, code_of<W>(mids, bits, qa));
      out.set(2 * j + 1, code_of<W>(mids, bits, qb));
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) out.set(k, code_of<W>(mids, bits, __fdiv_rn(x[k], d)));
  }
  return out;
}

// Copies both maps (2^bits entries each; a null map reads as zeros) into shared memory and derives
// their midpoints.  Entries past the end of a map are NaN (a NaN input's code 255 of a map with
// fewer than 8 bits decodes to NaN instead of reading past the caller's map), midpoints +inf.
template <bool W>
__device__ __forceinline__ void load_maps(Maps& M, const float* __restrict__ qm, const float* __restrict__ qv,
                                          int bits_m, int bits_v) {
  const int nm = 1 << bits_m, nv = 1 << bits_v;
  const float inf = __int_as_float(0x7f800000), nan = __int_as_float(0x7fc00000);
  const int cap = W ? 256 : 16;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) {
    M.qm[i] = (i < nm) ? (qm ? qm[i] : 0.0f) : nan;
    M.qv[i] = (i < nv) ? (qv ? qv[i] : 0.0f) : nan;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cap; i += blockDim.x) {
    M.mm[i] = (i < nm - 1) ? __fmul_rn(__fadd_rn(M.qm[i], M.qm[i + 1]), 0.5f) : inf;
    M.mv[i] = (i < nv - 1) ? __fmul_rn(__fadd_rn(M.qv[i], M.qv[i + 1]), 0.5f) : inf;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    M.zero_m = code_of<W>(M.mm, bits_m, 0.0f);
    M.zero_v = code_of<W>(M.mv, bits_v, 0.0f);
    int lin = qv != nullptr;
    const float step = 1.0f / (float)nv;  // a power of two: (i + 1) * step is exact
    for (int i = 0; i < nv; ++i) lin &= (M.qv[i] == (float)(i + 1) * step);
    M.linear_v = lin;
  }
  __syncthreads();
}

// Closed form of the nearest-code rule for the map q[i] = (i + 1) / N, N = 2^bits (midpoints
// (2k + 1) / (2N)): code = ceil(N x - 1.5) clamped to [0, N - 1].  N x - 1.5 is exact whenever it is
// positive (both terms are multiples of ulp(N x) and the difference is smaller than N x), a negative
// value saturates to 0 in the conversion, so the result equals the search for every x <= 1.
__device__ __forceinline__ int linear_code(float x, float N, int top) {
  const int c = (int)__float2uint_ru(__fmaf_rn(x, N, -1.5f));
  return c < top ? c : top;
}

__device__ __forceinline__ float hmax16(float x, unsigned mask) {
#pragma unroll
  for (int o = 8; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(mask, x, o, 16));
  return x;
}

// Maximum over the hpg adjacent half-warps that form one group (hpg a power of two, the group
// aligned to hpg half-warps inside the CTA).  Every thread of the CTA must call it.
__device__ __forceinline__ float group_max(float a, int hpg, float* red) {
  if (hpg == 1) return a;
  const int hw = threadIdx.x >> 4;
  __syncthreads();
  if ((threadIdx.x & 15) == 0) red[hw] = a;
  __syncthreads();
  const int b = hw & ~(hpg - 1);
  float r = red[b];
  for (int i = 1; i < hpg; ++i) r = fmaxf(r, red[b + i]);
  return r;
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

// e / d for non-negative operands, in 32 bits when both fit.
__device__ __forceinline__ long long div_nn(long long e, long long d) {
  return ((e | d) >> 32) ? e / d : (long long)((unsigned)e / (unsigned)d);
}

// min_i vecs[i][idx_i] for the 8 consecutive elements starting at flat index e0.  2-D tensors whose
// lane stays inside one row read the row value once and the 8 column values as two 128-bit loads.
template <int ND>
__device__ __forceinline__ void lane_scales(const float* const* vecs, long long e0, long long n, const Shape& s,
                                            float* out) {
  if (ND == 2) {
    const long long C = s.dim[1];
    const long long r = div_nn(e0, C);
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


// ---------------------------------------------------------------------------------------------
// AdamW, non-fused semantics.  MM: first-moment storage, VM: second-moment storage / source.
// ---------------------------------------------------------------------------------------------
// Register budget: 64 per thread (4 CTAs of 256 threads per SM) except for the rank-1 variants, whose
// index arithmetic needs more.
// A: the arithmetic of the reference's fused kernel instead of that of its torch operations (scalar path only).
template <int MM, int VM, int ND, bool W, bool A = false>
__global__ void __launch_bounds__(UTMAX, (VM == LPMM_B200_STATE_RANK1_4 && ND != 2) ? 1 : 2) unfused_adamw_kernel(const StepArgs a, const UConsts cin,
                                                               const float* __restrict__ qmap_m,
                                                               const float* __restrict__ qmap_v) {
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  __shared__ Maps M;
  __shared__ float red[UTMAX / 16];
  constexpr bool MQ = (MM == LPMM_B200_STATE_GROUP4);
  constexpr bool VQ = (VM == LPMM_B200_STATE_GROUP4 || VM == LPMM_B200_STATE_RANK1_4);
  if (MQ || VQ) load_maps<W>(M, qmap_m, qmap_v, a.bits_m, a.bits_v);
  const int l16 = threadIdx.x & 15;
  const int hw = threadIdx.x >> 4, hw_per_cta = blockDim.x >> 4;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long n = a.n;
  // units that hold elements or in-group padding (zeros before normalisation); later units are
  // the zeros that fill up the last row of 2048 after normalisation
  const long long in_m = MQ ? (n + 128LL * a.hpg_m - 1) / (128LL * a.hpg_m) * a.hpg_m : (n + 127) / 128;
  const long long in_v = (VM == LPMM_B200_STATE_GROUP4) ? (n + 128LL * a.hpg_v - 1) / (128LL * a.hpg_v) * a.hpg_v
                                                         : (n + 127) / 128;
  const long long C = (VM == LPMM_B200_STATE_FACTORED) ? a.s.dim[a.s.nd - 1] : 1;
  const long long RC = (VM == LPMM_B200_STATE_FACTORED) ? C * a.s.dim[a.s.nd - 2] : 1;
  const UConsts2 c2 = make_consts2(c);
  // a.units is a multiple of the half-warps per CTA, so every half-warp of a CTA makes the same
  // number of trips and the group reductions below may synchronise the CTA.  The two states may
  // have different padded lengths (group padding vs none): each is stored up to its own.
  for (long long u = (long long)blockIdx.x * hw_per_cta + hw; u < a.units; u += (long long)gridDim.x * hw_per_cta) {
    const long long e0 = u * 128 + l16 * 8;
    uint8_t* mb = MQ ? reinterpret_cast<uint8_t*>(a.m) + Codes8<W>::byte_off(e0) : nullptr;
    uint8_t* vb = VQ ? reinterpret_cast<uint8_t*>(a.v) + Codes8<W>::byte_off(e0) : nullptr;
    const bool has_data = e0 < n;  // this lane holds at least one element
    Codes8<W> mcodes, vcodes;
    mcodes.clear();
    vcodes.clear();
    float sm = 0.0f, sv = 0.0f;
    if (!a.first && has_data) {
      if (MQ) {
        mcodes.load(mb);
        sm = a.m_max1[u >> a.sh_m];
      }
      if (VQ) vcodes.load(vb);
      if (VM == LPMM_B200_STATE_GROUP4) sv = a.v_max1[u >> a.sh_v];
    }
    float st_old[8], st_new[8];
    if (VM == LPMM_B200_STATE_RANK1_4 && has_data) {
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
    // the update of the lane's 8 elements; FULL: all 8 exist, no per-element guards
    auto update_lane = [&](auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      if (!A && FULL && VM != LPMM_B200_STATE_FACTORED && c.fast) {  // two elements per instruction
        float* mf = reinterpret_cast<float*>(a.m);
        float* vf = reinterpret_cast<float*>(a.v);
        const f2 sm2 = f2_splat(sm), sv2 = f2_splat(sv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k0 = 2 * j, k1 = 2 * j + 1;
          f2 m0 = f2_splat(0.0f), v0 = f2_splat(0.0f);
          if (!a.first) {
            if (MQ) m0 = f2_mul(f2_pack(M.qm[mcodes.get(k0)], M.qm[mcodes.get(k1)]), sm2);
            else m0 = f2_pack(mf[e0 + k0], mf[e0 + k1]);
            if (VM == LPMM_B200_STATE_GROUP4)
              v0 = f2_mul(f2_pack(M.qv[vcodes.get(k0)], M.qv[vcodes.get(k1)]), sv2);
            else if (VM == LPMM_B200_STATE_RANK1_4)
              v0 = f2_mul(f2_pack(M.qv[vcodes.get(k0)], M.qv[vcodes.get(k1)]), f2_pack(st_old[k0], st_old[k1]));
            else v0 = f2_pack(vf[e0 + k0], vf[e0 + k1]);
          }
          f2 pj = f2_pack(px[k0], px[k1]), mj, vj;
          update_pair(c2, f2_pack(gx[k0], gx[k1]), pj, m0, v0, mj, vj, am, av);
          f2_unpack(pj, px[k0], px[k1]);
          f2_unpack(mj, m[k0], m[k1]);
          f2_unpack(vj, v[k0], v[k1]);
          if (MM == LPMM_B200_STATE_FP32) {
            mf[e0 + k0] = m[k0];
            mf[e0 + k1] = m[k1];
          }
          if (VM == LPMM_B200_STATE_FP32) {
            vf[e0 + k0] = v[k0];
            vf[e0 + k1] = v[k1];
          }
        }
        return;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const long long e = e0 + k;
        m[k] = 0.0f;
        v[k] = 0.0f;
        if (FULL || e < n) {
          const float g = gx[k];
          float m0 = 0.0f, v0 = 0.0f;
          if (!a.first) {
            if (MQ) m0 = __fmul_rn(M.qm[mcodes.get(k)], sm);
            else m0 = reinterpret_cast<const float*>(a.m)[e];
            if (VM == LPMM_B200_STATE_GROUP4) v0 = __fmul_rn(M.qv[vcodes.get(k)], sv);
            else if (VM == LPMM_B200_STATE_RANK1_4) v0 = __fmul_rn(M.qv[vcodes.get(k)], st_old[k]);
            else if (VM == LPMM_B200_STATE_FP32) v0 = reinterpret_cast<const float*>(a.v)[e];
          }
          m[k] = lerp_m<A>(c, m0, g);
          if (VM == LPMM_B200_STATE_FACTORED) {
            const float rf = __fdiv_rn(a.row[rowi], a.row_mean[bi]);
            v[k] = __fmul_rn(rf, a.col[bi * C + cc]);
          } else {
            v[k] = upd_v2<A>(c, v0, g);
          }
          px[k] = upd_param<A>(c, px[k], m[k], v[k]);
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
    };
    if (full) update_lane(std::true_type{});
    else update_lane(std::false_type{});
    if (full) {
      *reinterpret_cast<float4*>(a.p + e0) = make_float4(px[0], px[1], px[2], px[3]);
      *reinterpret_cast<float4*>(a.p + e0 + 4) = make_float4(px[4], px[5], px[6], px[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (e0 + k < n) a.p[e0 + k] = px[k];
    }
    if (MQ) {
      am = group_max(hmax16(am, hmask), a.hpg_m, red);
      Codes8<W> out;
      if (u < in_m) {
        out = codes_by_group_scale<W>(M.mm, a.bits_m, m, am);  // padding inside the last group is 0 / max
        if (l16 == 0 && (u & (a.hpg_m - 1)) == 0) a.m_max1[u >> a.sh_m] = am;
      } else {
        out.fill(M.zero_m);
      }
      if (u < a.units_m) out.store(mb);
    }
    if (VM == LPMM_B200_STATE_GROUP4) {
      av = group_max(hmax16(av, hmask), a.hpg_v, red);
      Codes8<W> out;
      if (u < in_v) {
        out = codes_by_group_scale<W>(M.mv, a.bits_v, v, av);
        if (l16 == 0 && (u & (a.hpg_v - 1)) == 0) a.v_max1[u >> a.sh_v] = av;
      } else {
        out.fill(M.zero_v);
      }
      if (u < a.units_v) out.store(vb);
    }
    if (VM == LPMM_B200_STATE_RANK1_4) {
      Codes8<W> out;
      out.clear();
      bool quick = full && M.linear_v;  // linear map, 8 elements, every divisor in the exact-division domain
      if (quick) {
        float lo = st_new[0], hi = st_new[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
          lo = fminf(lo, st_new[k]);
          hi = fmaxf(hi, st_new[k]);
        }
        quick = (lo >= 0x1p-60f) && (hi <= 0x1p60f);
      }
      if (quick) {
        // v / scale by reciprocal + residual correction (equal to IEEE division for quotients of at
        // least 2^-18; smaller ones are code 0 either way), then the closed-form code
        const int top = (1 << a.bits_v) - 1;
        const float N = (float)(top + 1);
        const f2 N2 = f2_splat(N), k15 = f2_splat(-1.5f), one2 = f2_splat(1.0f), mone2 = f2_splat(-1.0f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f2 d = f2_pack(st_new[2 * j], st_new[2 * j + 1]), x = f2_pack(v[2 * j], v[2 * j + 1]);
          const f2 nd = f2_mul(d, mone2);
          const f2 r0 = f2_pack(mufu_rcp(st_new[2 * j]), mufu_rcp(st_new[2 * j + 1]));
          const f2 r = f2_fma(r0, f2_fma(nd, r0, one2), r0);
          f2 q = f2_mul(x, r);
          q = f2_fma(f2_fma(q, nd, x), r, q);
          float ta, tb;
          f2_unpack(f2_fma(q, N2, k15), ta, tb);
          const int ca = (int)__float2uint_ru(ta), cb = (int)__float2uint_ru(tb);
          out.set(2 * j, ca < top ? ca : top);
          out.set(2 * j + 1, cb < top ? cb : top);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          out.set(k, (e0 + k < n) ? code_of<W>(M.mv, a.bits_v, __fdiv_rn(v[k], st_new[k])) : M.zero_v);
      }
      if (u < a.units_v) out.store(vb);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {  // the trailing byte of the packed layout
    if (MQ) reinterpret_cast<uint8_t*>(a.m)[Codes8<W>::trailing(a.units_m)] = 0;
    if (VQ) reinterpret_cast<uint8_t*>(a.v)[Codes8<W>::trailing(a.units_v)] = 0;
  }
}

// Statistics pass of the rank-1 second moment: recompute v exactly as the update pass will and
// fold it into the (zeroed) per-axis maxima.  The innermost axis changes with every element, so
// its maxima are first combined in shared memory (when the axis has at most STAT_LAST entries) and
// flushed once per CTA; the outer axes change rarely along a lane's 8 consecutive elements, so a
// lane combines runs of equal coordinates in registers before touching global memory.
constexpr int STAT_LAST = 8192;
template <int ND, bool W, bool A = false>
__global__ void __launch_bounds__(UT) rank1_stats_kernel(const StepArgs a, const UConsts cin,
                                                          const float* __restrict__ qmap_v) {
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  __shared__ Maps M;
  __shared__ int lastmax[STAT_LAST];
  load_maps<W>(M, nullptr, qmap_v, 4, a.bits_v);
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
    Codes8<W> vcodes;
    vcodes.clear();
    if (!a.first) vcodes.load(reinterpret_cast<const uint8_t*>(a.v) + Codes8<W>::byte_off(e0));
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
        if (!a.first) v0 = __fmul_rn(M.qv[vcodes.get(k)], st_old[k]);
        const float v = upd_v2<A>(c, v0, gx[k]);
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
// columns for all the rows of its CTA, so column maxima live in registers; a row's maximum is reduced
// across the warp and costs one atomic per warp and row.  Atomics on one 128-byte line serialise (about
// 2 ns each, measured as ~35 us for a 1024 x 1024 matrix cut into 512 row slices), so the column maxima
// of the CTAs of a thread-block cluster (stacked along the rows; the cluster size is a launch
// attribute) are first combined through distributed shared memory and only the cluster's first CTA
// issues atomics.  The host asks for clusters of STATS_CLUSTER when the row slices are thin (many
// CTAs per column, little work each) and for none when they are thick.
constexpr int STATS_CLUSTER = 8;
constexpr int STATS_CLUSTER_MAX_ROWS = 8;  // rows per CTA up to which clusters pay (4096 x 4096 has 12: measured slower)
template <bool W, bool A = false>
__global__ void __launch_bounds__(UT)
rank1_stats2d_kernel(const StepArgs a, const UConsts cin, const float* __restrict__ qmap_v, int rows_per_cta) {
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  __shared__ Maps M;
  __shared__ float colbuf[8 * UT];  // this CTA's column maxima, [k][thread]
  load_maps<W>(M, nullptr, qmap_v, 4, a.bits_v);
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
      Codes8<W> vcodes;
      vcodes.clear();
      float row_old = 0.0f;
      if (!a.first) {
        vcodes.load(reinterpret_cast<const uint8_t*>(a.v) + Codes8<W>::byte_off(e0));
        row_old = __ldg(a.v_old[0] + r);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float v0 = a.first ? 0.0f : __fmul_rn(M.qv[vcodes.get(k)], fminf(row_old, col_old[k]));
        const float v = upd_v2<A>(c, v0, gx[k]);
        col_max[k] = fmaxf(col_max[k], v);
        row_max = fmaxf(row_max, v);
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    if ((threadIdx.x & 31) == 0) atomic_max_nonneg(a.v_new[0] + r, row_max);
  }
  // every CTA of the cluster reaches both barriers (CTAs past the last row have an empty row loop)
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
#pragma unroll
  for (int k = 0; k < 8; ++k) colbuf[k * UT + threadIdx.x] = col_max[k];
  cluster.sync();
  if (cluster.block_rank() == 0 && active) {
    for (unsigned r = 1; r < cluster.num_blocks(); ++r) {
      const float* peer = cluster.map_shared_rank(colbuf, r);
#pragma unroll
      for (int k = 0; k < 8; ++k) col_max[k] = fmaxf(col_max[k], peer[k * UT + threadIdx.x]);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) atomic_max_nonneg(a.v_new[1] + c0 + k, col_max[k]);
  }
  cluster.sync();  // peers keep their shared memory until the first CTA has read it
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

template <int BM, bool W>
__global__ void __launch_bounds__(UTMAX, 2) sgd_kernel(float* __restrict__ p, const float* __restrict__ g, long long n,
                                                     long long units, void* buf, float* __restrict__ buf_max1,
                                                     int first, const float* __restrict__ qmap, int bits, int hpg,
                                                     int sh, const SgdConsts c) {
  __shared__ Maps M;
  __shared__ float red[UTMAX / 16];
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const int l16 = threadIdx.x & 15;
  const int hw = threadIdx.x >> 4, hw_per_cta = blockDim.x >> 4;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long in_units = (n + 128LL * hpg - 1) / (128LL * hpg) * hpg;
  const bool quantized = (BM == LPMM_B200_STATE_GROUP4) && c.has_momentum;
  for (long long u = (long long)blockIdx.x * hw_per_cta + hw; u < units; u += (long long)gridDim.x * hw_per_cta) {
    const long long e0 = u * 128 + l16 * 8;
    uint8_t* bb = quantized ? reinterpret_cast<uint8_t*>(buf) + Codes8<W>::byte_off(e0) : nullptr;
    Codes8<W> codes;
    codes.clear();
    float sc = 0.0f;
    if (bb && !first && e0 < n) {
      codes.load(bb);
      sc = buf_max1[u >> sh];
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
            const float b0 = (BM == LPMM_B200_STATE_GROUP4) ? __fmul_rn(M.qm[codes.get(k)], sc)
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
    if (quantized) {
      ab = group_max(hmax16(ab, hmask), hpg, red);
      Codes8<W> out;
      if (u < in_units) {
        out = codes_by_group_scale<W>(M.mm, bits, b, ab);
        if (l16 == 0 && (u & (hpg - 1)) == 0) buf_max1[u >> sh] = ab;
      } else {
        out.fill(M.zero_m);
      }
      out.store(bb);
    }
  }
  if (quantized && blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<uint8_t*>(buf)[Codes8<W>::trailing(units)] = 0;
}

// ---------------------------------------------------------------------------------------------
// Standalone quantize / dequantize
// ---------------------------------------------------------------------------------------------
// Stochastic rounding as in quantize_bsearch<true> (quantization_kernel.cu:397-427): between the two
// neighbouring map values the upper one is taken with probability (x - lower) / (upper - lower), decided
// by `noise`, a uniform in (0, 1] from the Philox stream of the reference's thread that handles the
// element.  A NaN (where the reference reads before the start of its map) gives the last code.
__device__ __forceinline__ int sr_code(const float* __restrict__ q, int nq, float x, float noise) {
  if (x <= q[0]) return 0;
  if (q[nq - 1] <= x) return nq - 1;
  int lo = 0, hi = nq;
  while (lo < hi) {
    const int mi = (lo + hi) >> 1;
    if (q[mi] <= x) lo = mi + 1;
    else hi = mi;
  }
  if (lo == 0) return nq - 1;
  const float proba = __fdiv_rn(__fsub_rn(x, q[lo - 1]), __fsub_rn(q[lo], q[lo - 1]));
  const int flag = __float2int_rn(__fsub_rn(__fadd_rn(proba, noise), 0.5f));
  return flag ? lo : lo - 1;
}
// The uniforms of the 8 elements that start at padded-layout index e0, drawn exactly as the reference's
// pack kernels draw them: one Philox4_32_10 stream per thread (subsequence = thread index), a thread
// owning 8 consecutive elements in the two-codes-per-byte kernel (quantization_kernel.cu:431-459) and 4
// in the one-code-per-byte kernel (:517-537), one curand_uniform per element in element order.
template <bool W>
__device__ __forceinline__ void sr_noise8(unsigned long long seed, unsigned long long offset, long long e0,
                                          float* noise) {
  curandStatePhilox4_32_10_t st;
  if (W) {
    curand_init(seed, (unsigned long long)(e0 >> 2), offset, &st);
#pragma unroll
    for (int k = 0; k < 4; ++k) noise[k] = curand_uniform(&st);
    curand_init(seed, (unsigned long long)(e0 >> 2) + 1, offset, &st);
#pragma unroll
    for (int k = 4; k < 8; ++k) noise[k] = curand_uniform(&st);
  } else {
    curand_init(seed, (unsigned long long)(e0 >> 3), offset, &st);
#pragma unroll
    for (int k = 0; k < 8; ++k) noise[k] = curand_uniform(&st);
  }
}

// pack / unpack of already normalised values (quantization_kernel.cu:429-460, 515-537, 603-627, 655-672)
// Stochastic pack: one thread per 8 elements (n is a multiple of 8 here, as in the reference).
template <bool W>
__global__ void __launch_bounds__(UT) pack_sr_kernel(const float* __restrict__ x, long long n,
                                                      const float* __restrict__ qmap, int bits,
                                                      uint8_t* __restrict__ out, unsigned long long seed,
                                                      unsigned long long offset) {
  __shared__ Maps M;
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const int nq = 1 << bits;
  for (long long ch = (long long)blockIdx.x * UT + threadIdx.x; ch < n / 8; ch += (long long)gridDim.x * UT) {
    const long long e0 = ch * 8;
    float noise[8];
    sr_noise8<W>(seed, offset, e0, noise);
    Codes8<W> c;
    c.clear();
#pragma unroll
    for (int k = 0; k < 8; ++k) c.set(k, sr_code(M.qm, nq, x[e0 + k], noise[k]));
    c.store(out + Codes8<W>::byte_off(e0));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) out[W ? n : n / 2] = 0;
}
template <bool W>
__global__ void __launch_bounds__(UT) pack_kernel(const float* __restrict__ x, long long n,
                                                   const float* __restrict__ qmap, int bits,
                                                   uint8_t* __restrict__ out) {
  __shared__ Maps M;
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const long long nb = W ? n : n / 2;
  for (long long b = (long long)blockIdx.x * UT + threadIdx.x; b < nb; b += (long long)gridDim.x * UT) {
    if (W) {
      out[b] = (uint8_t)code_of<true>(M.mm, bits, x[b]);
    } else {
      const float2 xy = *reinterpret_cast<const float2*>(x + 2 * b);
      out[b] = (uint8_t)(code16(M.mm, xy.x) | (code16(M.mm, xy.y) << 4));
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) out[nb] = 0;
}
template <bool W>
__global__ void __launch_bounds__(UT) unpack_kernel(const uint8_t* __restrict__ in, long long n,
                                                     const float* __restrict__ qmap, int bits,
                                                     float* __restrict__ out) {
  __shared__ Maps M;
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const long long nb = W ? n : n / 2;
  for (long long b = (long long)blockIdx.x * UT + threadIdx.x; b < nb; b += (long long)gridDim.x * UT) {
    const uint8_t c = in[b];
    if (W) out[b] = M.qm[c];
    else *reinterpret_cast<float2*>(out + 2 * b) = make_float2(M.qm[c & 15], M.qm[c >> 4]);
  }
}
// 4-bit pack / unpack with wide accesses: a lane takes 8 consecutive values with one 256-bit access and their 8
// codes with one 32-bit access (a warp instruction moves 1 KB of values and 128 bytes of codes, both contiguous),
// four such units in flight per thread.  Codes come from the shared-memory table of common.cuh (one read and one
// compare per value) when the map fits it, else from the midpoint search; -inf, which the table files under the
// NaNs, is code 0 as in the reference's search.  The values behind the last whole unit of 8 (n is even) and the
// trailing byte belong to the caller's byte-wise launch.
constexpr int PVT = 256;
__device__ __forceinline__ uint32_t pack8(const f8& v, const LutEnt* __restrict__ lut, const float* __restrict__ mids,
                                          bool lut_ok) {
  const float ninf = __int_as_float(0xff800000);
  uint32_t word = 0;
#pragma unroll
  for (int k = 7; k >= 0; --k) {
    int c = lut_ok ? lut_code(lut, v.x[k]) : code16(mids, v.x[k]);
    if (v.x[k] == ninf) c = 0;
    word = (word << 4) + (uint32_t)c;
  }
  return word;
}
__global__ void __launch_bounds__(PVT) pack4_vec_kernel(const float* __restrict__ x, long long units,
                                                        const float* __restrict__ qmap, uint32_t* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem S;
  LutEnt* lut = reinterpret_cast<LutEnt*>(dyn_smem);
  lut_build(S, lut, qmap);
  const bool lut_ok = S.valid != 0;
  const long long stride = (long long)gridDim.x * PVT;
  long long u = (long long)blockIdx.x * PVT + threadIdx.x;
  for (; u + 3 * stride < units; u += 4 * stride) {
    const f8 a = ldg_f8(x + u * 8), b = ldg_f8(x + (u + stride) * 8), c = ldg_f8(x + (u + 2 * stride) * 8),
             d = ldg_f8(x + (u + 3 * stride) * 8);
    out[u] = pack8(a, lut, S.mids, lut_ok);
    out[u + stride] = pack8(b, lut, S.mids, lut_ok);
    out[u + 2 * stride] = pack8(c, lut, S.mids, lut_ok);
    out[u + 3 * stride] = pack8(d, lut, S.mids, lut_ok);
  }
  for (; u < units; u += stride) out[u] = pack8(ldg_f8(x + u * 8), lut, S.mids, lut_ok);
}
__device__ __forceinline__ void unpack8(uint32_t w, const float* __restrict__ qm, float* dst) {
  f8 r;
#pragma unroll
  for (int k = 0; k < 8; ++k) r.x[k] = qm[(w >> (4 * k)) & 15u];
  stg_f8(dst, r);
}
__global__ void __launch_bounds__(PVT) unpack4_vec_kernel(const uint32_t* __restrict__ in, long long units,
                                                          const float* __restrict__ qmap, float* __restrict__ out) {
  __shared__ float qm[16];
  if (threadIdx.x < 16) qm[threadIdx.x] = qmap[threadIdx.x];
  __syncthreads();
  const long long stride = (long long)gridDim.x * PVT;
  long long u = (long long)blockIdx.x * PVT + threadIdx.x;
  for (; u + 3 * stride < units; u += 4 * stride) {
    const uint32_t a = __ldcs(in + u), b = __ldcs(in + u + stride), c = __ldcs(in + u + 2 * stride),
                   d = __ldcs(in + u + 3 * stride);
    unpack8(a, qm, out + u * 8);
    unpack8(b, qm, out + (u + stride) * 8);
    unpack8(c, qm, out + (u + 2 * stride) * 8);
    unpack8(d, qm, out + (u + 3 * stride) * 8);
  }
  for (; u < units; u += stride) unpack8(__ldcs(in + u), qm, out + u * 8);
}
// mode 0: group scales (computes max1); mode 1: rank-1 scales from given per-axis maxima.
// SR: stochastic rounding with the reference's random stream (seed, offset); else round to nearest.
template <int MODE, int ND, bool W, bool SR = false>
__global__ void __launch_bounds__(UTMAX, 2) quant_kernel(const float* __restrict__ x, long long n, long long units,
                                                       const float* __restrict__ qmap, int bits, int hpg, int sh,
                                                       uint8_t* __restrict__ codes, float* __restrict__ max1,
                                                       const StepArgs a, unsigned long long seed = 0,
                                                       unsigned long long offset = 0) {
  __shared__ Maps M;
  __shared__ float red[UTMAX / 16];
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const int l16 = threadIdx.x & 15;
  const int hw = threadIdx.x >> 4, hw_per_cta = blockDim.x >> 4;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const long long in_units = (MODE == 0) ? (n + 128LL * hpg - 1) / (128LL * hpg) * hpg : (n + 127) / 128;
  for (long long u = (long long)blockIdx.x * hw_per_cta + hw; u < units; u += (long long)gridDim.x * hw_per_cta) {
    const long long e0 = u * 128 + l16 * 8;
    uint8_t* cb = codes + Codes8<W>::byte_off(e0);
    float xv[8], st[8];
    float ax = 0.0f;
    int co[8];
    if (MODE == 1 && e0 < n) decompose<ND>(e0, a.s, co);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      xv[k] = 0.0f;
      st[k] = 1.0f;
      if (e0 + k < n) {
        xv[k] = x[e0 + k];
        ax = fmaxf(ax, fabsf(xv[k]));
        if (MODE == 1) st[k] = axis_min<ND>(a.v_new, co, a.s.nd);
      }
      if (MODE == 1 && e0 < n) advance<ND>(co, a.s);
    }
    Codes8<W> out;
    if (SR) {
      // normalise with IEEE division (torch's div), then the reference's stochastic rule; padding behind
      // the last group is a zero, which the rule maps to the code of zero whatever the noise
      if (MODE == 0) ax = group_max(hmax16(ax, hmask), hpg, red);
      float noise[8];
      sr_noise8<W>(seed, offset, e0, noise);
      const int nq = 1 << bits;
      out.clear();
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const bool inside = (MODE == 0) ? (u < in_units) : (e0 + k < n);
        const float xn = inside ? __fdiv_rn(xv[k], MODE == 0 ? ax : st[k]) : 0.0f;
        out.set(k, sr_code(M.qm, nq, xn, noise[k]));
      }
      if (MODE == 0 && u < in_units && l16 == 0 && (u & (hpg - 1)) == 0) max1[u >> sh] = ax;
    } else if (MODE == 0) {
      ax = group_max(hmax16(ax, hmask), hpg, red);
      if (u < in_units) {
        out = codes_by_group_scale<W>(M.mm, bits, xv, ax);
        if (l16 == 0 && (u & (hpg - 1)) == 0) max1[u >> sh] = ax;
      } else {
        out.fill(M.zero_m);
      }
    } else {
      out.clear();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        out.set(k, (e0 + k < n) ? code_of<W>(M.mm, bits, __fdiv_rn(xv[k], st[k])) : M.zero_m);
    }
    out.store(cb);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) codes[Codes8<W>::trailing(units)] = 0;
}
template <int MODE, int ND, bool W>
__global__ void __launch_bounds__(UT) dequant_kernel(const uint8_t* __restrict__ codes, long long n,
                                                      const float* __restrict__ qmap, int bits, int sh,
                                                      const float* __restrict__ max1, float* __restrict__ out,
                                                      const StepArgs a) {
  __shared__ Maps M;
  load_maps<W>(M, qmap, nullptr, bits, 4);
  const long long nchunks = (n + 7) / 8;
  for (long long ch = (long long)blockIdx.x * UT + threadIdx.x; ch < nchunks; ch += (long long)gridDim.x * UT) {
    const long long e0 = ch * 8;
    Codes8<W> c;
    c.load(codes + Codes8<W>::byte_off(e0));
    int co[8];
    if (MODE == 1) decompose<ND>(e0, a.s, co);
    const float s0 = (MODE == 0) ? max1[(e0 >> 7) >> sh] : 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (e0 + k < n) {
        const float sc = (MODE == 0) ? s0 : axis_min<ND>(a.v_old, co, a.s.nd);
        out[e0 + k] = __fmul_rn(M.qm[c.get(k)], sc);
        if (MODE == 1) advance<ND>(co, a.s);
      }
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

}  // namespace lpmm_b200

using namespace lpmm_b200;

// Code width and group size of one quantized state as the kernels want them.
struct Layout {
  int bits, hpg, sh;
  bool wide;
};
static int make_layout(int bits, long long group_size, Layout* out) {
  if (bits == 0) bits = 4;
  if (group_size == 0) group_size = 128;
  if (bits < 1 || bits > 8) return LPMM_B200_ERR_BAD_KIND;
  if (bits < 4) return LPMM_B200_ERR_UNSUPPORTED;  // several codes per byte other than two
  if (group_size < 128 || group_size > 4096 || (group_size & (group_size - 1))) {
    return (group_size > 0) ? LPMM_B200_ERR_UNSUPPORTED : LPMM_B200_ERR_BAD_SIZE;
  }
  out->bits = bits;
  out->wide = bits > 4;
  out->hpg = (int)(group_size / 128);
  out->sh = 0;
  while ((1 << out->sh) < out->hpg) ++out->sh;
  return LPMM_B200_OK;
}
static inline long long padded_units(long long numel, long long group_size) {
  return pad_to(pad_to(numel, group_size), 2048) / 128;
}
// Threads per CTA: all half-warps of a group must sit in one CTA.
static inline int threads_for(int hpg) { return hpg > UT / 16 ? UTMAX : UT; }
static inline bool aligned_for(const void* p, bool wide) { return ((uintptr_t)p & (wide ? 7 : 3)) == 0; }

#define LPMM_DISPATCH_W(wide, ...)                     \
  do {                                                 \
    if (wide) { constexpr bool W = true; __VA_ARGS__; } \
    else { constexpr bool W = false; __VA_ARGS__; }     \
  } while (0)

extern "C" int64_t lpmm_b200_packed_len_bits(int64_t n_scaled, int bits) {
  if (n_scaled < 0) return LPMM_B200_ERR_BAD_SIZE;
  Layout l;
  const int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  return l.wide ? pad_to(n_scaled, 2048) + 1 : pad_to(n_scaled, 2048) / 2 + 1;
}
extern "C" int64_t lpmm_b200_packed_len(int64_t n_scaled) { return lpmm_b200_packed_len_bits(n_scaled, 4); }

extern "C" int lpmm_b200_pack_nonlinear(const float* data, int64_t n, const float* qmap, int bits, int8_t* packed,
                                        void* stream) {
  Layout l;
  const int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (n < 0 || (!l.wide && (n & 1))) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !packed || (n > 0 && !data)) return LPMM_B200_ERR_NULL_POINTER;
  // two codes per byte, values 32-byte and codes 4-byte aligned: wide accesses for the whole units of 8 values, the
  // byte-wise kernel for what is left (and the trailing byte)
  if (!l.wide && n >= 8 && (((uintptr_t)data & 31) == 0) && (((uintptr_t)packed & 3) == 0)) {
    const long long chunks = n / 8;
    const size_t smem = LUT_ENTRIES * sizeof(LutEnt);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      LPMM_CUDA_TRY(cudaFuncSetAttribute(pack4_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      attr_set[dev] = true;
    }
    pack4_vec_kernel<<<grid_for(chunks, PVT, 4), PVT, smem, (cudaStream_t)stream>>>(data, chunks, qmap, (uint32_t*)packed);
    LPMM_CUDA_TRY(cudaGetLastError());
    const long long rest = n - chunks * 8;  // even; rest == 0 still writes the trailing byte
    pack_kernel<false><<<grid_for(rest / 2, UT), UT, 0, (cudaStream_t)stream>>>(data + chunks * 8, rest, qmap, l.bits,
                                                                               (uint8_t*)packed + chunks * 4);
    LPMM_CUDA_TRY(cudaGetLastError());
    return LPMM_B200_OK;
  }
  LPMM_DISPATCH_W(l.wide, (pack_kernel<W><<<grid_for(l.wide ? n : n / 2, UT), UT, 0, (cudaStream_t)stream>>>(
                              data, n, qmap, l.bits, (uint8_t*)packed)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_pack_nonlinear_sr(const float* data, int64_t n, const float* qmap, int bits, int8_t* packed,
                                           uint64_t seed, uint64_t offset, void* stream) {
  Layout l;
  const int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (n < 0 || (n & 7)) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !packed || (n > 0 && !data)) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(packed, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  LPMM_DISPATCH_W(l.wide, (pack_sr_kernel<W><<<grid_for(n / 8, UT), UT, 0, (cudaStream_t)stream>>>(
                              data, n, qmap, l.bits, (uint8_t*)packed, seed, offset)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_pack_nonlinear4(const float* data, int64_t n, const float* qmap, int8_t* packed,
                                         void* stream) {
  return lpmm_b200_pack_nonlinear(data, n, qmap, 4, packed, stream);
}

extern "C" int lpmm_b200_unpack_nonlinear(const int8_t* packed, const float* qmap, int bits, int64_t n, float* out,
                                          void* stream) {
  Layout l;
  const int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (n < 0 || (!l.wide && (n & 1))) return LPMM_B200_ERR_BAD_SIZE;
  if (n == 0) return LPMM_B200_OK;
  if (!qmap || !packed || !out) return LPMM_B200_ERR_NULL_POINTER;
  if (!l.wide && n >= 8 && (((uintptr_t)out & 31) == 0) && (((uintptr_t)packed & 3) == 0)) {
    const long long chunks = n / 8, rest = n - chunks * 8;
    unpack4_vec_kernel<<<grid_for(chunks, PVT, 4), PVT, 0, (cudaStream_t)stream>>>((const uint32_t*)packed, chunks, qmap, out);
    LPMM_CUDA_TRY(cudaGetLastError());
    if (rest > 0) {
      unpack_kernel<false><<<grid_for(rest / 2, UT), UT, 0, (cudaStream_t)stream>>>((const uint8_t*)packed + chunks * 4, rest,
                                                                                   qmap, l.bits, out + chunks * 8);
      LPMM_CUDA_TRY(cudaGetLastError());
    }
    return LPMM_B200_OK;
  }
  LPMM_DISPATCH_W(l.wide, (unpack_kernel<W><<<grid_for(l.wide ? n : n / 2, UT), UT, 0, (cudaStream_t)stream>>>(
                              (const uint8_t*)packed, n, qmap, l.bits, out)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_unpack_nonlinear4(const int8_t* packed, const float* qmap, int64_t n, float* out,
                                           void* stream) {
  return lpmm_b200_unpack_nonlinear(packed, qmap, 4, n, out, stream);
}

extern "C" int lpmm_b200_quant_group(const float* x, int64_t numel, const float* qmap, int bits, int64_t group_size,
                                     int8_t* codes, float* max1, void* stream) {
  Layout l;
  const int rc = make_layout(bits, group_size, &l);
  if (rc) return rc;
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !codes || (numel > 0 && (!x || !max1))) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  const long long units = padded_units(numel, 128LL * l.hpg);
  const int th = threads_for(l.hpg);
  LPMM_DISPATCH_W(l.wide, (quant_kernel<0, 2, W><<<grid_for(units, th / 16), th, 0, (cudaStream_t)stream>>>(
                              x, numel, units, qmap, l.bits, l.hpg, l.sh, (uint8_t*)codes, max1, a)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_quant_group_sr(const float* x, int64_t numel, const float* qmap, int bits, int64_t group_size,
                                        int8_t* codes, float* max1, uint64_t seed, uint64_t offset, void* stream) {
  Layout l;
  const int rc = make_layout(bits, group_size, &l);
  if (rc) return rc;
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (!qmap || !codes || (numel > 0 && (!x || !max1))) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  const long long units = padded_units(numel, 128LL * l.hpg);
  const int th = threads_for(l.hpg);
  LPMM_DISPATCH_W(l.wide, (quant_kernel<0, 2, W, true><<<grid_for(units, th / 16), th, 0, (cudaStream_t)stream>>>(
                              x, numel, units, qmap, l.bits, l.hpg, l.sh, (uint8_t*)codes, max1, a, seed, offset)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_quant_group4(const float* x, int64_t numel, const float* qmap, int8_t* codes, float* max1,
                                      void* stream) {
  return lpmm_b200_quant_group(x, numel, qmap, 4, 128, codes, max1, stream);
}

extern "C" int lpmm_b200_dequant_group(const int8_t* codes, const float* qmap, int bits, int64_t group_size,
                                       const float* max1, int64_t numel, float* out, void* stream) {
  Layout l;
  const int rc = make_layout(bits, group_size, &l);
  if (rc) return rc;
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (numel == 0) return LPMM_B200_OK;
  if (!qmap || !codes || !max1 || !out) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  LPMM_DISPATCH_W(l.wide, (dequant_kernel<0, 2, W><<<grid_for((numel + 7) / 8, UT), UT, 0, (cudaStream_t)stream>>>(
                              (const uint8_t*)codes, numel, qmap, l.bits, l.sh, max1, out, a)));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_dequant_group4(const int8_t* codes, const float* qmap, const float* max1, int64_t numel,
                                        float* out, void* stream) {
  return lpmm_b200_dequant_group(codes, qmap, 4, 128, max1, numel, out, stream);
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

extern "C" int lpmm_b200_quant_rank1(const float* x, const int64_t* shape, int ndim, const float* qmap, int bits,
                                     float* const* max_dims, int8_t* codes, void* stream) {
  Layout l;
  int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (ndim < 2) return LPMM_B200_ERR_BAD_SIZE;
  rc = lpmm_b200_axis_absmax(x, shape, ndim, max_dims, stream);
  if (rc) return rc;
  if (!qmap || !codes) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  fill_shape(a.s, shape, ndim, &a.n);
  for (int i = 0; i < ndim; ++i) a.v_new[i] = max_dims[i];
  const long long units = pad_to(a.n, 2048) / 128;
  LPMM_DISPATCH_W(l.wide, LPMM_DISPATCH_ND(ndim, (quant_kernel<1, ND, W><<<grid_for(units, UT / 16), UT, 0,
                                                                            (cudaStream_t)stream>>>(
                                                     x, a.n, units, qmap, l.bits, 1, 0, (uint8_t*)codes, nullptr, a))));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_quant_rank1_sr(const float* x, const int64_t* shape, int ndim, const float* qmap, int bits,
                                        float* const* max_dims, int8_t* codes, uint64_t seed, uint64_t offset,
                                        void* stream) {
  Layout l;
  int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (ndim < 2) return LPMM_B200_ERR_BAD_SIZE;
  rc = lpmm_b200_axis_absmax(x, shape, ndim, max_dims, stream);
  if (rc) return rc;
  if (!qmap || !codes) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  fill_shape(a.s, shape, ndim, &a.n);
  for (int i = 0; i < ndim; ++i) a.v_new[i] = max_dims[i];
  const long long units = pad_to(a.n, 2048) / 128;
  LPMM_DISPATCH_W(l.wide, LPMM_DISPATCH_ND(ndim, (quant_kernel<1, ND, W, true><<<grid_for(units, UT / 16), UT, 0,
                                                                                  (cudaStream_t)stream>>>(
                                                     x, a.n, units, qmap, l.bits, 1, 0, (uint8_t*)codes, nullptr, a, seed,
                                                     offset))));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_quant_rank1_4(const float* x, const int64_t* shape, int ndim, const float* qmap,
                                       float* const* max_dims, int8_t* codes, void* stream) {
  return lpmm_b200_quant_rank1(x, shape, ndim, qmap, 4, max_dims, codes, stream);
}

extern "C" int lpmm_b200_dequant_rank1(const int8_t* codes, const float* qmap, int bits,
                                       const float* const* max_dims, const int64_t* shape, int ndim, float* out,
                                       void* stream) {
  Layout l;
  int rc = make_layout(bits, 128, &l);
  if (rc) return rc;
  if (ndim < 2) return LPMM_B200_ERR_BAD_SIZE;
  StepArgs a = {};
  rc = fill_shape(a.s, shape, ndim, &a.n);
  if (rc) return rc;
  if (a.n == 0) return LPMM_B200_OK;
  if (!qmap || !codes || !max_dims || !out) return LPMM_B200_ERR_NULL_POINTER;
  if (!aligned_for(codes, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  for (int i = 0; i < ndim; ++i) {
    if (!max_dims[i]) return LPMM_B200_ERR_NULL_POINTER;
    a.v_old[i] = max_dims[i];
  }
  LPMM_DISPATCH_W(l.wide, LPMM_DISPATCH_ND(ndim, (dequant_kernel<1, ND, W><<<grid_for((a.n + 7) / 8, UT), UT, 0,
                                                                              (cudaStream_t)stream>>>(
                                                     (const uint8_t*)codes, a.n, qmap, l.bits, 0, nullptr, out, a))));
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_dequant_rank1_4(const int8_t* codes, const float* qmap, const float* const* max_dims,
                                         const int64_t* shape, int ndim, float* out, void* stream) {
  return lpmm_b200_dequant_rank1(codes, qmap, 4, max_dims, shape, ndim, out, stream);
}

extern "C" int64_t lpmm_b200_factored_scratch_bytes(const int64_t* shape, int ndim) {
  if (ndim < 2 || ndim > 8 || !shape) return LPMM_B200_ERR_BAD_SIZE;
  long long B = 1;
  for (int i = 0; i < ndim - 2; ++i) B *= shape[i];
  const long long R = shape[ndim - 2], C = shape[ndim - 1];
  const long long tiles = (R + TR - 1) / TR;
  return (int64_t)sizeof(float) * (B * tiles * C + B);
}

template <int MM, bool W>
static cudaError_t launch_unfused(int vm, unsigned grid, int threads, cudaStream_t st, const StepArgs& a,
                                  const UConsts& c, const float* qm, const float* qv) {
  switch (vm) {
    case LPMM_B200_STATE_FP32:
      unfused_adamw_kernel<MM, LPMM_B200_STATE_FP32, 2, W><<<grid, threads, 0, st>>>(a, c, qm, qv);
      break;
    case LPMM_B200_STATE_GROUP4:
      unfused_adamw_kernel<MM, LPMM_B200_STATE_GROUP4, 2, W><<<grid, threads, 0, st>>>(a, c, qm, qv);
      break;
    case LPMM_B200_STATE_RANK1_4:
      LPMM_DISPATCH_ND(a.s.nd, (unfused_adamw_kernel<MM, LPMM_B200_STATE_RANK1_4, ND, W><<<grid, threads, 0, st>>>(a, c, qm, qv)));
      break;
    default:
      unfused_adamw_kernel<MM, LPMM_B200_STATE_FACTORED, 2, W><<<grid, threads, 0, st>>>(a, c, qm, qv);
      break;
  }
  return cudaGetLastError();
}

// The same kernels with the fused kernel's arithmetic: 4-bit codes only; both moments fp32, both in
// groups, or a grouped first moment with a rank-1 second moment.
static cudaError_t launch_fused_arith(bool mq, int vm, unsigned grid, int threads, cudaStream_t st, const StepArgs& a,
                                      const UConsts& c, const float* qm, const float* qv) {
  constexpr int F = LPMM_B200_STATE_FP32, G = LPMM_B200_STATE_GROUP4, R = LPMM_B200_STATE_RANK1_4;
  if (!mq && vm == F) unfused_adamw_kernel<F, F, 2, false, true><<<grid, threads, 0, st>>>(a, c, qm, qv);
  else if (mq && vm == G) unfused_adamw_kernel<G, G, 2, false, true><<<grid, threads, 0, st>>>(a, c, qm, qv);
  else if (mq && vm == R)
    LPMM_DISPATCH_ND(a.s.nd, (unfused_adamw_kernel<G, R, ND, false, true><<<grid, threads, 0, st>>>(a, c, qm, qv)));
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// arith 0: the arithmetic of the reference's torch operations; 1: that of its fused kernel.
static int step_one_tensor(const lpmm_b200_step_tensor* t, const float* qmap_m, const float* qmap_v, double beta1,
                           double beta2, double lr, double weight_decay, double eps, double step, void* scratch,
                           int64_t scratch_bytes, void* stream, int arith) {
  if (!t) return LPMM_B200_ERR_NULL_POINTER;
  if (t->numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (t->m_mode != LPMM_B200_STATE_FP32 && t->m_mode != LPMM_B200_STATE_GROUP4) return LPMM_B200_ERR_BAD_KIND;
  if (t->v_mode < LPMM_B200_STATE_FP32 || t->v_mode > LPMM_B200_STATE_FACTORED) return LPMM_B200_ERR_BAD_KIND;
  const bool mq = t->m_mode == LPMM_B200_STATE_GROUP4;
  const bool vq = t->v_mode == LPMM_B200_STATE_GROUP4 || t->v_mode == LPMM_B200_STATE_RANK1_4;
  Layout lm = {4, 1, 0, false}, lv = {4, 1, 0, false};
  if (mq) {
    const int rc = make_layout(t->m_bits, t->m_group, &lm);
    if (rc) return rc;
  }
  if (vq) {
    const int rc = make_layout(t->v_bits, t->v_mode == LPMM_B200_STATE_GROUP4 ? t->v_group : 128, &lv);
    if (rc) return rc;
  }
  if (mq && vq && lm.wide != lv.wide) return LPMM_B200_ERR_UNSUPPORTED;  // one storage format per launch
  const bool wide = mq ? lm.wide : (vq && lv.wide);
  if (arith) {
    const bool pair_ok = (!mq && t->v_mode == LPMM_B200_STATE_FP32) || (mq && vq);
    if (wide || !pair_ok) return LPMM_B200_ERR_UNSUPPORTED;
  }
  if (t->numel == 0) return LPMM_B200_OK;
  if (!t->p || !t->g) return LPMM_B200_ERR_NULL_POINTER;
  if (!t->m) return LPMM_B200_ERR_NULL_POINTER;
  if (mq && (!t->m_max1 || !qmap_m)) return LPMM_B200_ERR_NULL_POINTER;
  if (mq && !aligned_for(t->m, wide)) return LPMM_B200_ERR_BAD_SIZE;
  if (vq && t->v && !aligned_for(t->v, wide)) return LPMM_B200_ERR_BAD_SIZE;
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
  a.bits_m = lm.bits;
  a.bits_v = lv.bits;
  a.hpg_m = lm.hpg;
  a.sh_m = lm.sh;
  a.hpg_v = lv.hpg;
  a.sh_v = lv.sh;
  const int hpg_max = lm.hpg > lv.hpg ? lm.hpg : lv.hpg;
  a.units_m = mq ? padded_units(a.n, 128LL * lm.hpg) : 0;
  a.units_v = (t->v_mode == LPMM_B200_STATE_GROUP4) ? padded_units(a.n, 128LL * lv.hpg) : (vq ? pad_to(a.n, 2048) / 128 : 0);
  a.units = pad_to(a.n, 2048) / 128;
  if (a.units_m > a.units) a.units = a.units_m;
  if (a.units_v > a.units) a.units = a.units_v;
  const UConsts c = make_consts(beta1, beta2, lr, weight_decay, eps, step);
  if (t->v_mode == LPMM_B200_STATE_RANK1_4 || t->v_mode == LPMM_B200_STATE_FACTORED) {
    long long n2 = 0;
    int rc = fill_shape(a.s, t->shape, t->ndim, &n2);
    if (rc) return rc;
    if (t->ndim < 2 || n2 != t->numel) return LPMM_B200_ERR_BAD_SIZE;
  }
  if (t->v_mode == LPMM_B200_STATE_FP32 || vq) {
    if (!t->v) return LPMM_B200_ERR_NULL_POINTER;
    if (vq && !qmap_v) return LPMM_B200_ERR_NULL_POINTER;
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
    if (t->ndim == 2 && t->shape[1] % 8 == 0 && a.vec_ok) {
      const long long R = t->shape[0], C = t->shape[1];
      const long long col_ctas = (C / 8 + UT - 1) / UT;
      long long row_ctas = ((long long)num_sms() * 6 + col_ctas - 1) / col_ctas;
      if (row_ctas > R) row_ctas = R;
      if (row_ctas > 65528) row_ctas = 65528;  // grid.y limit, rounded down to whole clusters
      const int rows_per_cta = (int)((R + row_ctas - 1) / row_ctas);
      row_ctas = (R + rows_per_cta - 1) / rows_per_cta;
      if (rows_per_cta <= STATS_CLUSTER_MAX_ROWS) {
        row_ctas = (row_ctas + STATS_CLUSTER - 1) / STATS_CLUSTER * STATS_CLUSTER;  // whole clusters; extra CTAs have no rows
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)col_ctas, (unsigned)row_ctas);
        cfg.blockDim = dim3(UT);
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 1;
        attr.val.clusterDim.y = STATS_CLUSTER;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (arith) LPMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, rank1_stats2d_kernel<false, true>, a, c, qmap_v, rows_per_cta));
        else LPMM_DISPATCH_W(lv.wide, LPMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, rank1_stats2d_kernel<W>, a, c, qmap_v, rows_per_cta)));
      } else if (arith) {
        rank1_stats2d_kernel<false, true><<<dim3((unsigned)col_ctas, (unsigned)row_ctas), UT, 0, st>>>(a, c, qmap_v, rows_per_cta);
      } else {
        LPMM_DISPATCH_W(lv.wide, (rank1_stats2d_kernel<W><<<dim3((unsigned)col_ctas, (unsigned)row_ctas), UT, 0, st>>>(
                                     a, c, qmap_v, rows_per_cta)));
      }
    } else if (arith) {
      LPMM_DISPATCH_ND(t->ndim, (rank1_stats_kernel<ND, false, true><<<grid_for((a.n + 7) / 8, UT, 3), UT, 0, st>>>(a, c, qmap_v)));
    } else {
      LPMM_DISPATCH_W(lv.wide, LPMM_DISPATCH_ND(t->ndim, (rank1_stats_kernel<ND, W><<<grid_for((a.n + 7) / 8, UT, 3), UT,
                                                                                    0, st>>>(a, c, qmap_v))));
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
  const int threads = threads_for(hpg_max);
  const unsigned grid = grid_for(a.units, threads / 16, threads == UT ? 8 : 4);
  cudaError_t e = cudaSuccess;
  if (arith) {
    e = launch_fused_arith(mq, t->v_mode, grid, threads, st, a, c, qmap_m, qmap_v);
  } else {
    LPMM_DISPATCH_W(wide, (e = mq ? launch_unfused<LPMM_B200_STATE_GROUP4, W>(t->v_mode, grid, threads, st, a, c, qmap_m, qmap_v)
                                  : launch_unfused<LPMM_B200_STATE_FP32, W>(t->v_mode, grid, threads, st, a, c, qmap_m, qmap_v)));
  }
  LPMM_CUDA_TRY(e);
  return LPMM_B200_OK;
}

extern "C" int lpmm_b200_adamw4bit_unfused_step(const lpmm_b200_step_tensor* t, const float* qmap_m,
                                                const float* qmap_v, double beta1, double beta2, double lr,
                                                double weight_decay, double eps, double step, void* scratch,
                                                int64_t scratch_bytes, void* stream) {
  return step_one_tensor(t, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, scratch, scratch_bytes, stream, 0);
}

extern "C" int lpmm_b200_adamw4bit_fused_arith_step(const lpmm_b200_step_tensor* t, const float* qmap_m,
                                                    const float* qmap_v, double beta1, double beta2, double lr,
                                                    double weight_decay, double eps, double step, void* stream) {
  return step_one_tensor(t, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, nullptr, 0, stream, 1);
}

// adamw_unfused_multi.cu: the shared launch with the fused kernel's arithmetic (internal to the library)
LPMM_INTERNAL int lpmm_b200_fused_arith_multi_tensor(const lpmm_b200_tensor* ts, int n, const float* qmap_m,
                                                  const float* qmap_v, double beta1, double beta2, double lr,
                                                  double weight_decay, double eps, double step, void* stream);
// the shared launch of the torch-operation arithmetic with the tolerance-mode parameter update
LPMM_INTERNAL int lpmm_b200_unfused_multi_tensor_apx(const lpmm_b200_tensor* ts, int n, const float* qmap_m,
                                                  const float* qmap_v, double beta1, double beta2, double lr,
                                                  double weight_decay, double eps, double step, void* stream);

// rank1_multi.cu: all rank-1 matrices of a list in three launches (internal to the library)
LPMM_INTERNAL int lpmm_b200_rank1_multi_ok(const lpmm_b200_step_tensor* t);
LPMM_INTERNAL int lpmm_b200_rank1_multi_step(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m,
                                          const float* qmap_v, double beta1, double beta2, double lr,
                                          double weight_decay, double eps, double step, void* stream, int arith,
                                          int apx);

// factored_multi.cu: all factored matrices of a list in four launches (internal to the library)
LPMM_INTERNAL int lpmm_b200_factored_multi_ok(const lpmm_b200_step_tensor* t);
LPMM_INTERNAL int64_t lpmm_b200_factored_multi_scratch_bytes(const lpmm_b200_step_tensor* const* ts, int n);
LPMM_INTERNAL int lpmm_b200_factored_multi_step(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m,
                                             double beta1, double beta2, double lr, double weight_decay, double eps,
                                             double step, void* scratch, int64_t scratch_bytes, void* stream,
                                             int apx);

// Side streams of lpmm_b200_adamw4bit_unfused_step_many: the tensors of a list are independent and most
// of them are small (a few launches of a few microseconds each, one waiting for the other), so their
// launch chains are spread over SIDE_STREAMS streams that fork from the caller's stream and join it
// again before the call returns; to the caller everything is ordered on `stream` as before.  One set
// per device, created on first use and kept for the life of the process; a mutex serialises callers
// of one device while they enqueue (the events are shared).
constexpr int SIDE_STREAMS = 4;
struct SideStreams {
  cudaStream_t s[SIDE_STREAMS];
  cudaEvent_t fork, join[SIDE_STREAMS];
  int state;  // 0: not tried, 1: ready, -1: could not be created (single-stream operation)
  std::mutex mu;
};
static SideStreams* side_streams_of_current_device() {
  static SideStreams all[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SideStreams& x = all[dev];
  std::lock_guard<std::mutex> lock(x.mu);
  if (x.state == 0) {
    bool ok = cudaEventCreateWithFlags(&x.fork, cudaEventDisableTiming) == cudaSuccess;
    for (int k = 0; ok && k < SIDE_STREAMS; ++k)
      ok = cudaStreamCreateWithFlags(&x.s[k], cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&x.join[k], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) cudaGetLastError();  // leave no sticky "last error" behind
    x.state = ok ? 1 : -1;
  }
  return x.state == 1 ? &x : nullptr;
}

extern "C" int64_t lpmm_b200_unfused_step_many_scratch_bytes(const lpmm_b200_step_tensor* const* tensors, int n) {
  if (n < 0 || (n > 0 && !tensors)) return LPMM_B200_ERR_BAD_SIZE;
  std::vector<const lpmm_b200_step_tensor*> fmv;
  int64_t max_need = 0;
  for (int i = 0; i < n; ++i) {
    const lpmm_b200_step_tensor* t = tensors[i];
    if (!t) return LPMM_B200_ERR_NULL_POINTER;
    if (t->v_mode == LPMM_B200_STATE_FACTORED) {
      const int64_t need = lpmm_b200_factored_scratch_bytes(t->shape, t->ndim);
      if (need > max_need) max_need = need;
      lpmm_b200_step_tensor probe = *t;
      probe.first = 0;  // sized for the steady state
      if (lpmm_b200_factored_multi_ok(&probe)) fmv.push_back(t);
    }
  }
  int64_t total = (int64_t)SIDE_STREAMS * ((max_need + 255) & ~(int64_t)255);
  if (fmv.size() >= 2) total += (lpmm_b200_factored_multi_scratch_bytes(fmv.data(), (int)fmv.size()) + 511) & ~(int64_t)255;
  return total + 1024;
}

static int step_many(const lpmm_b200_step_tensor* const* tensors, int n, const float* qmap_m, const float* qmap_v,
                     double beta1, double beta2, double lr, double weight_decay, double eps, const double* steps,
                     void* scratch, int64_t scratch_bytes, void* stream, int arith, uint32_t flags) {
  if (n < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (n > 0 && (!tensors || !steps)) return LPMM_B200_ERR_NULL_POINTER;
  if (flags & ~(uint32_t)LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) return LPMM_B200_ERR_BAD_KIND;
  // the tolerance mode applies to the list-wide kernels (full aligned groups); tensors stepped on their own stay exact
  const int apx = (flags & LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE) ? 1 : 0;
  cudaStream_t user = (cudaStream_t)stream;
  // which tensors go into the shared multi-tensor launch (both moments fp32, or both 4-bit with
  // groups of 128, already initialised), how many need launches of their own, and the largest
  // scratch need among the factored ones
  auto is_plain = [&](const lpmm_b200_step_tensor* t) {
    if (t->first || t->numel <= 0 || !t->p || !t->g || !t->m || !t->v) return false;
    if (t->m_mode == LPMM_B200_STATE_FP32 && t->v_mode == LPMM_B200_STATE_FP32) return true;
    return t->m_mode == LPMM_B200_STATE_GROUP4 && t->v_mode == LPMM_B200_STATE_GROUP4 &&
           (t->m_bits == 0 || t->m_bits == 4) && (t->v_bits == 0 || t->v_bits == 4) &&
           (t->m_group == 0 || t->m_group == 128) && (t->v_group == 0 || t->v_group == 128) && t->m_max1 &&
           t->v_max1 && qmap_m && qmap_v;
  };
  // rank-1 matrices that share a step count are stepped together (rank1_multi.cu; their descriptors travel in
  // the launch parameters, so this also holds while `stream` is being captured)
  bool capturing = true;
  {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(user, &cap) == cudaSuccess) capturing = cap != cudaStreamCaptureStatusNone;
    else cudaGetLastError();
  }
  static thread_local std::vector<const lpmm_b200_step_tensor*> r1;
  r1.clear();
  double r1_step = 0.0;
  for (int i = 0; i < n; ++i) {
    if (!tensors[i]) return LPMM_B200_ERR_NULL_POINTER;
    if (qmap_m && qmap_v && lpmm_b200_rank1_multi_ok(tensors[i]) && (r1.empty() || steps[i] == r1_step)) {
      r1_step = steps[i];
      r1.push_back(tensors[i]);
    }
  }
  if (r1.size() < 2) r1.clear();
  auto in_r1 = [&](const lpmm_b200_step_tensor* t, double s) {
    return !r1.empty() && s == r1_step && lpmm_b200_rank1_multi_ok(t);
  };
  // factored matrices that share a step count, likewise (factored_multi.cu); their table and partial
  // sums come from the end of what is left of the scratch
  static thread_local std::vector<const lpmm_b200_step_tensor*> fm;
  fm.clear();
  double fm_step = 0.0;
  for (int i = 0; i < n; ++i) {
    if (!arith && lpmm_b200_factored_multi_ok(tensors[i]) && (fm.empty() || steps[i] == fm_step) &&
        (tensors[i]->m_mode == LPMM_B200_STATE_FP32 || qmap_m)) {
      fm_step = steps[i];
      fm.push_back(tensors[i]);
    }
  }
  void* fm_scratch = nullptr;
  int64_t fm_bytes = 0;
  if (fm.size() >= 2 && scratch && (((uintptr_t)scratch & 255) == 0)) {
    fm_bytes = (lpmm_b200_factored_multi_scratch_bytes(fm.data(), (int)fm.size()) + 255) & ~(int64_t)255;
    if (fm_bytes <= scratch_bytes) {
      scratch_bytes = (scratch_bytes - fm_bytes) & ~(int64_t)255;
      fm_scratch = static_cast<char*>(scratch) + scratch_bytes;
    }
  }
  if (!fm_scratch) fm.clear();
  auto in_fm = [&](const lpmm_b200_step_tensor* t, double s) {
    return !fm.empty() && s == fm_step && lpmm_b200_factored_multi_ok(t);
  };
  int own = 0;
  int64_t max_need = 0;
  for (int i = 0; i < n; ++i) {
    if (is_plain(tensors[i]) || in_r1(tensors[i], steps[i]) || in_fm(tensors[i], steps[i])) continue;
    ++own;
    if (tensors[i]->v_mode == LPMM_B200_STATE_FACTORED) {
      const int64_t need = lpmm_b200_factored_scratch_bytes(tensors[i]->shape, tensors[i]->ndim);
      if (need > max_need) max_need = need;
    }
  }
  SideStreams* side = nullptr;
  if (own >= 2 && !capturing) side = side_streams_of_current_device();
  std::unique_lock<std::mutex> lock;
  if (side) {
    lock = std::unique_lock<std::mutex>(side->mu);
    LPMM_CUDA_TRY(cudaEventRecord(side->fork, user));
    for (int k = 0; k < SIDE_STREAMS; ++k) LPMM_CUDA_TRY(cudaStreamWaitEvent(side->s[k], side->fork, 0));
  }
  // factored tensors share `scratch`: each side stream gets its own slice when the largest need fits
  // one, otherwise all factored tensors stay on one stream and use all of it
  const int64_t slice = side ? (scratch_bytes / SIDE_STREAMS) & ~(int64_t)255 : 0;
  const bool sliced = side && scratch && max_need <= slice;
  // the tensors of the shared launch must share a step count (it sets the bias corrections); a tensor
  // with another count is stepped on its own.  Tensors are independent, so the order is free.
  static thread_local std::vector<lpmm_b200_tensor> batch;
  batch.clear();
  double batch_step = 0.0;
  int rr = 0;  // round-robin position
  int rc = LPMM_B200_OK;
  for (int i = 0; i < n && rc == LPMM_B200_OK; ++i) {
    const lpmm_b200_step_tensor* t = tensors[i];
    if (is_plain(t) && (batch.empty() || steps[i] == batch_step)) {
      batch_step = steps[i];
      lpmm_b200_tensor d;
      d.p = t->p;
      d.g = t->g;
      d.m = t->m;
      d.v = t->v;
      d.m_scale = t->m_max1;
      d.v_scale = t->v_max1;
      d.numel = t->numel;
      d.kind = (t->m_mode == LPMM_B200_STATE_FP32) ? LPMM_B200_KIND_FP32 : LPMM_B200_KIND_Q4;
      d.reserved = 0;
      batch.push_back(d);
      continue;
    }
    if (in_r1(t, steps[i]) || in_fm(t, steps[i])) continue;  // stepped together below
    cudaStream_t st = user;
    void* sc = scratch;
    int64_t sc_bytes = scratch_bytes;
    if (side) {
      int k = rr++ % SIDE_STREAMS;
      if (t->v_mode == LPMM_B200_STATE_FACTORED) {
        if (sliced) {
          sc = static_cast<char*>(scratch) + (int64_t)k * slice;
          sc_bytes = slice;
        } else {
          k = 0;
        }
      }
      st = side->s[k];
    }
    rc = step_one_tensor(t, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, steps[i], sc, sc_bytes, st, arith);
  }
  if (rc == LPMM_B200_OK && !r1.empty())
    rc = lpmm_b200_rank1_multi_step(r1.data(), (int)r1.size(), qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps,
                                    r1_step, user, arith, apx);
  if (rc == LPMM_B200_OK && !fm.empty())
    rc = lpmm_b200_factored_multi_step(fm.data(), (int)fm.size(), qmap_m, beta1, beta2, lr, weight_decay, eps, fm_step,
                                       fm_scratch, fm_bytes, user, apx);
  if (rc == LPMM_B200_OK && !batch.empty())
    rc = arith ? lpmm_b200_fused_arith_multi_tensor(batch.data(), (int)batch.size(), qmap_m, qmap_v, beta1, beta2, lr,
                                                    weight_decay, eps, batch_step, user)
         : apx ? lpmm_b200_unfused_multi_tensor_apx(batch.data(), (int)batch.size(), qmap_m, qmap_v, beta1, beta2, lr,
                                                    weight_decay, eps, batch_step, user)
               : lpmm_b200_adamw4bit_unfused_multi_tensor(batch.data(), (int)batch.size(), qmap_m, qmap_v, beta1, beta2,
                                                          lr, weight_decay, eps, batch_step, 0, -1, user);
  if (side) {  // join even after an error: the caller's stream must not run ahead of what was enqueued
    for (int k = 0; k < SIDE_STREAMS; ++k) {
      if (cudaEventRecord(side->join[k], side->s[k]) != cudaSuccess ||
          cudaStreamWaitEvent(user, side->join[k], 0) != cudaSuccess) {
        if (rc == LPMM_B200_OK) rc = set_cuda_error(cudaGetLastError());
      }
    }
  }
  return rc;
}

extern "C" int lpmm_b200_adamw4bit_unfused_step_many(const lpmm_b200_step_tensor* const* tensors, int n,
                                                     const float* qmap_m, const float* qmap_v, double beta1,
                                                     double beta2, double lr, double weight_decay, double eps,
                                                     const double* steps, void* scratch, int64_t scratch_bytes,
                                                     void* stream) {
  return step_many(tensors, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, steps, scratch, scratch_bytes,
                   stream, 0, 0);
}

extern "C" int lpmm_b200_adamw4bit_unfused_step_many_flags(const lpmm_b200_step_tensor* const* tensors, int n,
                                                           const float* qmap_m, const float* qmap_v, double beta1,
                                                           double beta2, double lr, double weight_decay, double eps,
                                                           const double* steps, void* scratch, int64_t scratch_bytes,
                                                           void* stream, uint32_t flags) {
  return step_many(tensors, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, steps, scratch, scratch_bytes,
                   stream, 0, flags);
}

extern "C" int lpmm_b200_adamw4bit_fused_arith_step_many(const lpmm_b200_step_tensor* const* tensors, int n,
                                                         const float* qmap_m, const float* qmap_v, double beta1,
                                                         double beta2, double lr, double weight_decay, double eps,
                                                         const double* steps, void* scratch, int64_t scratch_bytes,
                                                         void* stream) {
  return step_many(tensors, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, steps, scratch, scratch_bytes,
                   stream, 1, 0);
}

extern "C" int lpmm_b200_adamw4bit_fused_arith_step_many_flags(const lpmm_b200_step_tensor* const* tensors, int n,
                                                               const float* qmap_m, const float* qmap_v, double beta1,
                                                               double beta2, double lr, double weight_decay,
                                                               double eps, const double* steps, void* scratch,
                                                               int64_t scratch_bytes, void* stream, uint32_t flags) {
  return step_many(tensors, n, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, steps, scratch, scratch_bytes,
                   stream, 1, flags);
}

extern "C" int lpmm_b200_sgd_lowbit_step(float* p, const float* g, int64_t numel, void* buf, float* buf_max1,
                                         int buf_mode, int bits, int64_t group_size, int first, const float* qmap,
                                         double weight_decay, double momentum, double lr, double dampening,
                                         int nesterov, int maximize, void* stream) {
  if (numel < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (buf_mode != LPMM_B200_STATE_FP32 && buf_mode != LPMM_B200_STATE_GROUP4) return LPMM_B200_ERR_BAD_KIND;
  Layout l = {4, 1, 0, false};
  if (buf_mode == LPMM_B200_STATE_GROUP4) {
    const int rc = make_layout(bits, group_size, &l);
    if (rc) return rc;
  }
  if (numel == 0) return LPMM_B200_OK;
  if (!p || !g) return LPMM_B200_ERR_NULL_POINTER;
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
    if (buf_mode == LPMM_B200_STATE_GROUP4 && !aligned_for(buf, l.wide)) return LPMM_B200_ERR_BAD_SIZE;
  }
  const long long units = padded_units(numel, 128LL * l.hpg);
  const int threads = threads_for(l.hpg);
  const unsigned grid = grid_for(units, threads / 16, threads == UT ? 8 : 4);
  if (buf_mode == LPMM_B200_STATE_GROUP4) {
    LPMM_DISPATCH_W(l.wide, (sgd_kernel<LPMM_B200_STATE_GROUP4, W><<<grid, threads, 0, (cudaStream_t)stream>>>(
                                p, g, numel, units, buf, buf_max1, first, qmap, l.bits, l.hpg, l.sh, c)));
  } else {
    sgd_kernel<LPMM_B200_STATE_FP32, false><<<grid, threads, 0, (cudaStream_t)stream>>>(p, g, numel, units, buf, buf_max1,
                                                                                     first, qmap, 4, 1, 0, c);
  }
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
extern "C" int lpmm_b200_sgd4bit_step(float* p, const float* g, int64_t numel, void* buf, float* buf_max1,
                                      int buf_mode, int first, const float* qmap, double weight_decay,
                                      double momentum, double lr, double dampening, int nesterov, int maximize,
                                      void* stream) {
  return lpmm_b200_sgd_lowbit_step(p, g, numel, buf, buf_max1, buf_mode, 4, 128, first, qmap, weight_decay, momentum,
                                   lr, dampening, nesterov, maximize, stream);
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
