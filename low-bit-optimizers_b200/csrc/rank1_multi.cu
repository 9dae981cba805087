// The non-fused step of the reference's default.yml configuration -- first moment 4-bit with group-128
// scales, second moment 4-bit with rank-1 (per-row / per-column maxima) scales -- for ALL matrices of a
// parameter list in three launches: zero the new maxima, a statistics pass that recomputes every second
// moment and folds it into the new row / column maxima (the first pass of the two-pass grid
// reduction), and the update pass (dequantise with the old maxima, AdamW, requantise with the new).
// The reference does this per parameter in Python (lpmm/optim/adamw.py:332-436 with
// lpmm/functional.py:190-203, 97-106, 512-531); arithmetic and state layout here are those of the
// per-tensor launches in unfused.cu, bit for bit.
//
// The tensors are described by a table carried in the launch parameters (up to R1_MAX per launch; a longer list
// is stepped in windows), so nothing is uploaded and the launches can be captured into a CUDA graph.  Work is
// cut into tiles (statistics) and 128-element units (update) numbered across the whole window, and a fixed
// grid of persistent CTAs strides over them, so small and large matrices share the machine and nothing waits
// for a tiny launch.
#include <math.h>

#include <vector>

#include "common.cuh"
#include "fused_x2.cuh"
#include "multi_tensor.cuh"
#include "unfused_math.cuh"

namespace lpmm_b200 {

constexpr int R1T = 256;                   // threads per CTA
constexpr size_t R1_DYN_SMEM = LUT_ENTRIES * sizeof(LutEnt);

struct R1Desc {
  float* p;
  const float* g;
  uint8_t* m;
  float* m_max1;
  uint8_t* v;
  const float* old_r;  // maxima the stored codes were normalised with: per row, per column
  const float* old_c;
  float* new_r;        // maxima of the updated second moment
  float* new_c;
  long long n;
  long long ustart;    // first global 128-element unit of this tensor
  long long tstart;    // first global statistics tile of this tensor
  int R, C;
  int tiles_x, rows_per_tile;
  int tx_shift;        // statistics: log2 of the column-threads of a tile (8 columns each)
  int pad_;
};


constexpr int R1_MAX = 268;  // descriptors per launch: 120 bytes each, 32 KB of launch parameters in all
struct R1Table {
  int n;
  int first;            // index of the first descriptor the scalar update kernel steps (the wide ones come before)
  long long tiles;      // statistics tiles of the window
  long long units;      // 128-element units of the descriptors from `first` on
  R1Desc t[R1_MAX];
};

// Index of the last descriptor whose `start` field (ustart / tstart) is <= x.
template <bool TILES>
__device__ __forceinline__ int r1_find(const R1Desc* d, int n, long long x) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((TILES ? d[mid].tstart : d[mid].ustart) <= x) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(R1T) r1_zero_kernel(const __grid_constant__ R1Table tab) {
  const R1Desc& t = tab.t[blockIdx.x];
  for (int i = threadIdx.x; i < t.R; i += R1T) t.new_r[i] = 0.0f;
  for (int i = threadIdx.x; i < t.C; i += R1T) t.new_c[i] = 0.0f;
}

// Statistics: a tile is (8 << tx_shift) columns by rows_per_tile rows of one matrix.  The CTA's 256
// threads form 2^tx_shift column-threads (8 columns each) by 256 >> tx_shift row-lanes, so a narrow
// matrix keeps every thread busy; a thread keeps its 8 columns for all its rows of the tile (column
// maxima in registers, one atomic per thread and column at the end), a row's maximum is reduced across
// the lanes that share the row (one atomic per warp and row).  Two rows per thread are in flight.
// Rows are multiples of 8 floats and 16-byte aligned (host-checked).
// One row's 8 elements of a thread: second moments recomputed from codes, old maxima and gradients, folded into
// the thread's column maxima; returns their maximum.  qv_l: this lane's entry of the map (lane & 15), read by
// shuffle with the code as source lane -- every lane of the warp must call this (idle lanes pass zeros, which leave
// every maximum alone).  Pairs of elements share the packed fp32x2 multiply / fma, each half rounding like the
// scalar upd_v2.
template <bool A>
__device__ __forceinline__ float r1_row_pass(float qv_l, const float* col_old, float* col_max, f2 kb2, f2 komb2,
                                             const float4& g0, const float4& g1, uint32_t codes, float row_old) {
  const f2 gx[4] = {f2_pack(g0.x, g0.y), f2_pack(g0.z, g0.w), f2_pack(g1.x, g1.y), f2_pack(g1.z, g1.w)};
  float row_max = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float qa = __shfl_sync(0xffffffffu, qv_l, (int)(codes >> (8 * j)), 16);  // source lane = code (mod 16)
    const float qb = __shfl_sync(0xffffffffu, qv_l, (int)(codes >> (8 * j + 4)), 16);
    const f2 v0 = f2_mul(f2_pack(qa, qb), f2_pack(fminf(row_old, col_old[2 * j]), fminf(row_old, col_old[2 * j + 1])));
    const f2 v = A ? f2_fma(kb2, v0, f2_mul(f2_mul(komb2, gx[j]), gx[j]))       // fma(b2, v0, ((1-b2) g) g)
                   : f2_fma(komb2, f2_mul(gx[j], gx[j]), f2_mul(v0, kb2));     // fma(1-b2, g g, v0 b2)
    float va, vb;
    f2_unpack(v, va, vb);
    col_max[2 * j] = fmaxf(col_max[2 * j], va);
    col_max[2 * j + 1] = fmaxf(col_max[2 * j + 1], vb);
    row_max = fmaxf(row_max, fmaxf(va, vb));
  }
  return row_max;
}

template <bool A>
__global__ void __launch_bounds__(R1T, 3) r1_stats_kernel(const __grid_constant__ R1Table tab,
                                                        const float* __restrict__ qmap_v, const UConsts cin) {
  const R1Desc* d = tab.t;
  const int n = tab.n;
  const long long total_tiles = tab.tiles;
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  const float qv_l = __ldg(qmap_v + (threadIdx.x & 15));
  const f2 kb2 = f2_splat(A ? c.f_beta2 : c.beta2), komb2 = f2_splat(A ? c.f_omb2 : c.omb2);
  for (long long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const R1Desc& t = d[r1_find<true>(d, n, tile)];
    const long long local = tile - t.tstart;
    const int tx_count = 1 << t.tx_shift, ty_count = R1T >> t.tx_shift;
    const int tx = threadIdx.x & (tx_count - 1), ty = threadIdx.x >> t.tx_shift;
    const int tile_x = (int)(local % t.tiles_x);
    const long long tile_y = local / t.tiles_x;
    const long long C = t.C;
    const long long c0 = ((long long)tile_x * tx_count + tx) * 8;
    const bool active = c0 < C;
    float col_old[8], col_max[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      col_old[k] = active ? __ldg(t.old_c + c0 + k) : 0.0f;
      col_max[k] = 0.0f;
    }
    const long long r_begin = tile_y * t.rows_per_tile;
    const long long r_end = (r_begin + t.rows_per_tile < t.R) ? r_begin + t.rows_per_tile : t.R;
    const int seg = tx_count < 32 ? tx_count : 32;  // lanes that share a row inside a warp
    const unsigned segmask = (seg == 32 ? 0xffffffffu : ((1u << seg) - 1u)) << (threadIdx.x & 31 & ~(seg - 1));
    // all lanes of a warp make the same number of trips (the shuffles below need the whole warp); the loads of the
    // next pair of rows are issued before the arithmetic of the current pair
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 nga0 = zero4, nga1 = zero4, ngc0 = zero4, ngc1 = zero4;
    uint32_t nca = 0, ncc = 0;
    float noa = 0.0f, noc = 0.0f;
    {
      const long long ra = r_begin + ty, rc = r_begin + ty_count + ty;
      if (active && ra < r_end) {
        const long long e0 = ra * C + c0;
        nga0 = *reinterpret_cast<const float4*>(t.g + e0);
        nga1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
        nca = *reinterpret_cast<const uint32_t*>(t.v + (e0 >> 1));
        noa = __ldg(t.old_r + ra);
      }
      if (active && rc < r_end) {
        const long long e0 = rc * C + c0;
        ngc0 = *reinterpret_cast<const float4*>(t.g + e0);
        ngc1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
        ncc = *reinterpret_cast<const uint32_t*>(t.v + (e0 >> 1));
        noc = __ldg(t.old_r + rc);
      }
    }
    for (long long rb = r_begin; rb < r_end; rb += 2 * ty_count) {
      const long long ra = rb + ty, rc = rb + ty_count + ty;
      const float4 ga0 = nga0, ga1 = nga1, gc0 = ngc0, gc1 = ngc1;
      const uint32_t ca = nca, cc = ncc;
      const float oa = noa, oc = noc;
      {
        const long long ra2 = ra + 2 * ty_count, rc2 = rc + 2 * ty_count;
        if (active && ra2 < r_end) {
          const long long e0 = ra2 * C + c0;
          nga0 = *reinterpret_cast<const float4*>(t.g + e0);
          nga1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
          nca = *reinterpret_cast<const uint32_t*>(t.v + (e0 >> 1));
          noa = __ldg(t.old_r + ra2);
        }
        if (active && rc2 < r_end) {
          const long long e0 = rc2 * C + c0;
          ngc0 = *reinterpret_cast<const float4*>(t.g + e0);
          ngc1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
          ncc = *reinterpret_cast<const uint32_t*>(t.v + (e0 >> 1));
          noc = __ldg(t.old_r + rc2);
        }
      }
      // rows that do not exist were loaded as zeros: their second moments are zero and change no maximum
      float ma = r1_row_pass<A>(qv_l, col_old, col_max, kb2, komb2, ga0, ga1, ca, oa);
      float mc = r1_row_pass<A>(qv_l, col_old, col_max, kb2, komb2, gc0, gc1, cc, oc);
      // maximum over the lanes that share the row: the values are non-negative floats, whose order is that of their
      // bit patterns, so one integer warp reduction per row replaces a shuffle tree
      ma = __uint_as_float(__reduce_max_sync(segmask, __float_as_uint(ma)));
      mc = __uint_as_float(__reduce_max_sync(segmask, __float_as_uint(mc)));
      if ((threadIdx.x & (seg - 1)) == 0) {
        if (ra < r_end) atomic_max_nonneg(t.new_r + ra, ma);
        if (rc < r_end) atomic_max_nonneg(t.new_r + rc, mc);
      }
    }
    if (active) {
#pragma unroll
      for (int k = 0; k < 8; ++k) atomic_max_nonneg(t.new_c + c0 + k, col_max[k]);
    }
  }
}


// One 128-element unit of one matrix.  FULL lanes (8 elements inside one row, 16-byte aligned, short
// exact sequences applicable) use packed arithmetic; every other lane takes the scalar IEEE path.
// A: the fused kernel's arithmetic (packed for FULL lanes as well, fused_x2.cuh).
template <bool A>
__device__ __forceinline__ void r1_unit(const R1Desc& t, long long u, int l16, unsigned hmask, const UConsts& c,
                                        const UConsts2& c2, const Consts2& kf, const QMapSmem& Sm, const QMapSmem& Sv,
                                        const LutEnt* __restrict__ lut_m, bool lut_ok) {
  const long long n = t.n, C = t.C;
  const long long e0 = u * 128 + l16 * 8;
  uint8_t* mb = t.m + (e0 >> 1);
  uint8_t* vb = t.v + (e0 >> 1);
  const bool has_data = e0 < n;
  uint32_t mcodes = 0, vcodes = 0;
  float sm = 0.0f;
  if (has_data) {
    mcodes = *reinterpret_cast<const uint32_t*>(mb);
    vcodes = *reinterpret_cast<const uint32_t*>(vb);
    sm = t.m_max1[u];
  }
  long long r = 0, col = 0;
  if (has_data) {
    r = ((e0 | C) >> 32) ? e0 / C : (long long)((unsigned)e0 / (unsigned)C);
    col = e0 - r * C;
  }
  const bool full = (A ? c.f_fast : c.fast) && (e0 + 8 <= n) && (col + 8 <= C);  // C % 8 == 0 and aligned bases: host-checked
  float m[8], v[8], st_new[8];
  float am = 0.0f;
  if (full) {
    const float ro = __ldg(t.old_r + r), rn = t.new_r[r];
    const float4 o0 = __ldg(reinterpret_cast<const float4*>(t.old_c + col));
    const float4 o1 = __ldg(reinterpret_cast<const float4*>(t.old_c + col + 4));
    const float4 n0 = *reinterpret_cast<const float4*>(t.new_c + col);
    const float4 n1 = *reinterpret_cast<const float4*>(t.new_c + col + 4);
    const float st_old[8] = {fminf(ro, o0.x), fminf(ro, o0.y), fminf(ro, o0.z), fminf(ro, o0.w),
                             fminf(ro, o1.x), fminf(ro, o1.y), fminf(ro, o1.z), fminf(ro, o1.w)};
    st_new[0] = fminf(rn, n0.x); st_new[1] = fminf(rn, n0.y); st_new[2] = fminf(rn, n0.z); st_new[3] = fminf(rn, n0.w);
    st_new[4] = fminf(rn, n1.x); st_new[5] = fminf(rn, n1.y); st_new[6] = fminf(rn, n1.z); st_new[7] = fminf(rn, n1.w);
    f2x4 g, p;
    {
      const float4 a0 = *reinterpret_cast<const float4*>(t.g + e0), a1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(t.p + e0), b1 = *reinterpret_cast<const float4*>(t.p + e0 + 4);
      g.v[0] = f2_pack(a0.x, a0.y); g.v[1] = f2_pack(a0.z, a0.w); g.v[2] = f2_pack(a1.x, a1.y); g.v[3] = f2_pack(a1.z, a1.w);
      p.v[0] = f2_pack(b0.x, b0.y); p.v[1] = f2_pack(b0.z, b0.w); p.v[2] = f2_pack(b1.x, b1.y); p.v[3] = f2_pack(b1.z, b1.w);
    }
    const f2 sm2 = f2_splat(sm);
    float av = 0.0f;
    float px[8];
    if (A) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k0 = 2 * j, k1 = 2 * j + 1;
        const f2 m0 = f2_mul(f2_pack(Sm.qmap[(mcodes >> (4 * k0)) & 15u], Sm.qmap[(mcodes >> (4 * k1)) & 15u]), sm2);
        const f2 v0 = f2_mul(f2_pack(Sv.qmap[(vcodes >> (4 * k0)) & 15u], Sv.qmap[(vcodes >> (4 * k1)) & 15u]),
                             f2_pack(st_old[k0], st_old[k1]));
        f2 mj, vj;
        const f2 pj = fused_pair_x2(kf, g.v[j], p.v[j], m0, v0, mj, vj, am, av);
        f2_unpack(mj, m[k0], m[k1]);
        f2_unpack(vj, v[k0], v[k1]);
        f2_unpack(pj, px[k0], px[k1]);
      }
    } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k0 = 2 * j, k1 = 2 * j + 1;
      const f2 m0 = f2_mul(f2_pack(Sm.qmap[(mcodes >> (4 * k0)) & 15u], Sm.qmap[(mcodes >> (4 * k1)) & 15u]), sm2);
      const f2 v0 = f2_mul(f2_pack(Sv.qmap[(vcodes >> (4 * k0)) & 15u], Sv.qmap[(vcodes >> (4 * k1)) & 15u]),
                           f2_pack(st_old[k0], st_old[k1]));
      f2 mj, vj;
      update_pair(c2, g.v[j], p.v[j], m0, v0, mj, vj, am, av);
      f2_unpack(mj, m[k0], m[k1]);
      f2_unpack(vj, v[k0], v[k1]);
      f2_unpack(p.v[j], px[k0], px[k1]);
    }
    }
    *reinterpret_cast<float4*>(t.p + e0) = make_float4(px[0], px[1], px[2], px[3]);
    *reinterpret_cast<float4*>(t.p + e0 + 4) = make_float4(px[4], px[5], px[6], px[7]);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const long long e = e0 + k;
      m[k] = 0.0f;
      v[k] = 0.0f;
      st_new[k] = 1.0f;
      if (e < n) {
        const long long rr = e / C, cc = e - rr * C;
        const float so = fminf(__ldg(t.old_r + rr), __ldg(t.old_c + cc));
        st_new[k] = fminf(t.new_r[rr], t.new_c[cc]);
        const float g = t.g[e];
        const float m0 = __fmul_rn(Sm.qmap[(mcodes >> (4 * k)) & 15u], sm);
        const float v0 = __fmul_rn(Sv.qmap[(vcodes >> (4 * k)) & 15u], so);
        m[k] = lerp_m<A>(c, m0, g);
        v[k] = upd_v2<A>(c, v0, g);
        t.p[e] = upd_param<A>(c, t.p[e], m[k], v[k]);
        am = fmaxf(am, fabsf(m[k]));
      }
    }
  }
  // first moment: group maximum over the half-warp (every lane takes part), codes of this lane
  am = hw_max(am, hmask);
  uint32_t mo = 0;
  if (udiv_ok(am)) {
    const f2 r2 = f2_splat(rcp_nr(am)), nam2 = f2_splat(-am);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      const f2 xj = f2_pack(m[2 * j], m[2 * j + 1]);
      f2 q = f2_mul(xj, r2);
      q = f2_fma(f2_fma(q, nam2, xj), r2, q);
      float qa, qb;
      f2_unpack(q, qa, qb);
      mo = (mo << 4) + (uint32_t)(lut_ok ? lut_code(lut_m, qb) : code16(Sm.mids, qb));
      mo = (mo << 4) + (uint32_t)(lut_ok ? lut_code(lut_m, qa) : code16(Sm.mids, qa));
    }
    if (am == 0.0f) mo = 0xFFFFFFFFu;  // 0/0 = NaN -> code 15 for the whole group
  } else {
#pragma unroll
    for (int k = 7; k >= 0; --k) mo = (mo << 4) + (uint32_t)code16(Sm.mids, __fdiv_rn(m[k], am));
  }
  // second moment: v / min(new row max, new column max) per element
  uint32_t vo = 0;
  bool quick = full && Sv.linear16;
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
    const f2 k16 = f2_splat(16.0f), k15 = f2_splat(-1.5f), one2 = f2_splat(1.0f), mone2 = f2_splat(-1.0f);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      const f2 dd = f2_pack(st_new[2 * j], st_new[2 * j + 1]), x = f2_pack(v[2 * j], v[2 * j + 1]);
      const f2 nd = f2_mul(dd, mone2);
      const f2 r0 = f2_pack(mufu_rcp(st_new[2 * j]), mufu_rcp(st_new[2 * j + 1]));
      const f2 rr = f2_fma(r0, f2_fma(nd, r0, one2), r0);
      f2 q = f2_mul(x, rr);
      q = f2_fma(f2_fma(q, nd, x), rr, q);
      float ta, tb;
      f2_unpack(f2_fma(q, k16, k15), ta, tb);
      const uint32_t ca = __float2uint_ru(ta), cb = __float2uint_ru(tb);
      vo = (vo << 4) + (cb < 15u ? cb : 15u);
      vo = (vo << 4) + (ca < 15u ? ca : 15u);
    }
  } else {
    const int zero_v = code16(Sv.mids, 0.0f);
#pragma unroll
    for (int k = 7; k >= 0; --k)
      vo = (vo << 4) + (uint32_t)((e0 + k < n) ? code16(Sv.mids, __fdiv_rn(v[k], st_new[k])) : zero_v);
  }
  // the unit lies inside the padded layout (rows of 2048 codes), so all 16 lanes may store
  *reinterpret_cast<uint32_t*>(mb) = mo;
  *reinterpret_cast<uint32_t*>(vb) = vo;
  if (l16 == 0) t.m_max1[u] = am;
}

template <bool A>
__global__ void __launch_bounds__(R1T, 4) r1_update_kernel(const __grid_constant__ R1Table tab,
                                                            const float* __restrict__ qmap_m,
                                                            const float* __restrict__ qmap_v, const UConsts cin) {
  const R1Desc* d = tab.t + tab.first;
  const int n = tab.n - tab.first;
  const long long total_units = tab.units;
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm, Sv;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  lut_build(Sv, nullptr, qmap_v);
  lut_build(Sm, lut_m, qmap_m);
  const bool lut_ok = Sm.valid != 0;
  const UConsts2 c2 = make_consts2(c);
  const Consts2 kf = make_consts_x2(c.f_beta1, c.f_beta2, c.f_omb1, c.f_omb2, c.f_lr, c.f_wd, c.f_eps, c.c1, c.c2s, c.rc2s);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = (long long)blockIdx.x * (R1T / 16) + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * (R1T / 16);
  // every half-warp walks gi, gi + stride, ... through the tensors in order; the tensor loop is uniform
  for (int ti = 0; ti < n; ++ti) {
    const R1Desc& t = d[ti];
    const long long uend = (ti + 1 < n) ? d[ti + 1].ustart : total_units;
    for (; gi < uend; gi += stride) r1_unit<A>(t, gi - t.ustart, l16, hmask, c, c2, kf, Sm, Sv, lut_m, lut_ok);
  }
}


// ---------------------------------------------------------------------------------------------------------
// Update pass for matrices whose row length is a multiple of 128 (every projection of a transformer): a
// 128-element group then lies inside one row, so the whole half-warp shares the row maxima and a lane's 8
// elements are 8 consecutive columns.  The kernel has the shape of the fused multi-tensor step
// (adamw4bit.cu): descriptors in the launch parameters, persistent 1024-thread CTAs, a half-warp per
// group, 256-bit accesses of parameters and gradients, dequantisation by shuffle (lane i holds map entry i),
// packed fp32x2 arithmetic, table look-up for the first-moment codes.  What differs is the second moment:
// its scale is min(row maximum, column maximum) per element, old ones for dequantisation and the new ones
// from the statistics pass for requantisation.  Arithmetic is that of r1_unit's FULL lanes, bit for bit.
// ---------------------------------------------------------------------------------------------------------
constexpr int R2_MAX = 300;      // descriptors per launch (26.4 KB of the 32 KB parameter space)
constexpr int R2T = 1024;
constexpr int R2_HW = R2T / 16;

struct R2Desc {
  float* p;
  const float* g;
  uint32_t* m;          // first-moment codes, one word per lane and group
  uint32_t* v;
  float* msc;           // first-moment group maxima
  const float* old_r;
  const float* old_c;
  const float* new_r;
  const float* new_c;
  long long ustart;     // first global group of this tensor
  int gpr;              // groups per row: C / 128
  int pad_;
};
struct R2Table {
  int n;
  int pad_;
  long long total;      // groups in this table
  R2Desc t[R2_MAX];
};

// APX: the tolerance mode of the parameter update (fused_x2.cuh / unfused_math.cuh).
template <bool A, bool APX>
__device__ __forceinline__ void r2_group(const R2Desc& t, unsigned u, unsigned r, unsigned cb, int l16, unsigned hmask,
                                         const UConsts2& c2, const Consts2& kf, const QMapSmem& Sm, const QMapSmem& Sv,
                                         const LutEnt* __restrict__ lut_m, bool lut_ok, bool vlin, float qm_l, float qv_l,
                                         unsigned pf) {
  const size_t e0 = (size_t)u * 128 + (size_t)l16 * 8;
  float* pp = t.p + e0;
  const float* gp = t.g + e0;
  uint32_t* mcp = t.m + (size_t)u * 16 + l16;
  uint32_t* vcp = t.v + (size_t)u * 16 + l16;
  f2x4 p = ldg_f2x4(pp);
  const f2x4 g = ldg_f2x4(gp);
  const uint32_t mc = *mcp;
  const uint32_t vc = *vcp;
  const float pm = __fmul_rn(qm_l, t.msc[u]);  // lane i: qmap_m[i] * group maximum
  const float ro = __ldg(t.old_r + r);
  const size_t c0 = (size_t)cb * 128 + (size_t)l16 * 8;
  const float4 o0 = __ldg(reinterpret_cast<const float4*>(t.old_c + c0));
  const float4 o1 = __ldg(reinterpret_cast<const float4*>(t.old_c + c0 + 4));
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 128);
    prefetch_l2(gp + (size_t)pf * 128);
    prefetch_l2(mcp + (size_t)pf * 16);
    prefetch_l2(vcp + (size_t)pf * 16);
  }
  const float oc[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
  f2 m[4], v[4];
  float am = 0.0f, av = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float m0a = __shfl_sync(hmask, pm, (int)(mc >> (8 * j)), 16);  // source lane = code (mod 16)
    const float m0b = __shfl_sync(hmask, pm, (int)(mc >> (8 * j + 4)), 16);
    const float qa = __shfl_sync(hmask, qv_l, (int)(vc >> (8 * j)), 16);
    const float qb = __shfl_sync(hmask, qv_l, (int)(vc >> (8 * j + 4)), 16);
    const f2 v0 = f2_mul(f2_pack(qa, qb), f2_pack(fminf(ro, oc[2 * j]), fminf(ro, oc[2 * j + 1])));
    if (A) p.v[j] = fused_pair_x2<APX>(kf, g.v[j], p.v[j], f2_pack(m0a, m0b), v0, m[j], v[j], am, av);
    else update_pair<APX>(c2, g.v[j], p.v[j], f2_pack(m0a, m0b), v0, m[j], v[j], am, av);
  }
  stg_f2x4(pp, p);
  // first moment: group maximum over the half-warp, codes of this lane
  am = hw_max(am, hmask);
  uint32_t mo = 0;
  if (udiv_ok(am)) {
    const f2 r2 = f2_splat(rcp_nr(am)), nam2 = f2_splat(-am);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      f2 q = f2_mul(m[j], r2);
      q = f2_fma(f2_fma(q, nam2, m[j]), r2, q);
      float qa, qb;
      f2_unpack(q, qa, qb);
      mo = (mo << 4) + (uint32_t)(lut_ok ? lut_code(lut_m, qb) : code16(Sm.mids, qb));
      mo = (mo << 4) + (uint32_t)(lut_ok ? lut_code(lut_m, qa) : code16(Sm.mids, qa));
    }
    if (am == 0.0f) mo = 0xFFFFFFFFu;  // 0/0 = NaN -> code 15 for the whole group
  } else {
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      float ma, mb;
      f2_unpack(m[j], ma, mb);
      mo = (mo << 4) + (uint32_t)code16(Sm.mids, __fdiv_rn(mb, am));
      mo = (mo << 4) + (uint32_t)code16(Sm.mids, __fdiv_rn(ma, am));
    }
  }
  // second moment: v / min(new row maximum, new column maximum) per element
  const float rn = __ldg(t.new_r + r);
  const float4 n0 = __ldg(reinterpret_cast<const float4*>(t.new_c + c0));
  const float4 n1 = __ldg(reinterpret_cast<const float4*>(t.new_c + c0 + 4));
  const float nc[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
  const float cmin = fminf(fminf(fminf(nc[0], nc[1]), fminf(nc[2], nc[3])), fminf(fminf(nc[4], nc[5]), fminf(nc[6], nc[7])));
  uint32_t vo = 0;
  if (vlin && rn <= 0x1p60f && fminf(rn, cmin) >= 0x1p-60f) {  // every divisor inside the short division's domain
    const f2 k16 = f2_splat(16.0f), k15 = f2_splat(-1.5f), one2 = f2_splat(1.0f), mone2 = f2_splat(-1.0f);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      const float da = fminf(rn, nc[2 * j]), db = fminf(rn, nc[2 * j + 1]);
      const f2 nd = f2_mul(f2_pack(da, db), mone2);
      const f2 r0 = f2_pack(mufu_rcp(da), mufu_rcp(db));
      const f2 rr = f2_fma(r0, f2_fma(nd, r0, one2), r0);
      f2 q = f2_mul(v[j], rr);
      q = f2_fma(f2_fma(q, nd, v[j]), rr, q);
      float ta, tb;
      f2_unpack(f2_fma(q, k16, k15), ta, tb);
      // no clamp: every v is at most its row and its column maximum (the statistics pass computed them from the
      // same values with the same roundings), so the quotient is at most 1 and the code at most 15
      vo = vo * 16u + __float2uint_ru(tb);
      vo = vo * 16u + __float2uint_ru(ta);
    }
  } else {
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      float va, vb;
      f2_unpack(v[j], va, vb);
      vo = (vo << 4) + (uint32_t)code16(Sv.mids, __fdiv_rn(vb, fminf(rn, nc[2 * j + 1])));
      vo = (vo << 4) + (uint32_t)code16(Sv.mids, __fdiv_rn(va, fminf(rn, nc[2 * j])));
    }
  }
  *mcp = mo;
  *vcp = vo;
  if (l16 == 0) t.msc[u] = am;
}

template <bool A, bool APX>
__global__ void __launch_bounds__(R2T, 1) r1_update2_kernel(const __grid_constant__ R2Table tab,
                                                            const float* __restrict__ qmap_m,
                                                            const float* __restrict__ qmap_v, const UConsts cin) {
  UConsts cf;
  if (A) cf = fused_consts(cin);
  const UConsts& c = A ? cf : cin;
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm, Sv;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  lut_build(Sv, nullptr, qmap_v);
  lut_build(Sm, lut_m, qmap_m);
  const bool lut_ok = Sm.valid != 0, vlin = Sv.linear16 != 0;
  const UConsts2 c2 = make_consts2(c);
  const Consts2 kf = make_consts_x2(c.f_beta1, c.f_beta2, c.f_omb1, c.f_omb2, c.f_lr, c.f_wd, c.f_eps, c.c1, c.c2s, c.rc2s);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const float qm_l = Sm.qmap[l16], qv_l = Sv.qmap[l16];
  long long gi = (long long)blockIdx.x * R2_HW + (threadIdx.x >> 4);
  const unsigned stride = gridDim.x * R2_HW;
  // every half-warp walks gi, gi + stride, ... through the tensors in order; the tensor loop is uniform
  for (int ti = 0; ti < tab.n; ++ti) {
    const R2Desc& t = tab.t[ti];
    const long long uend = (ti + 1 < tab.n) ? tab.t[ti + 1].ustart : tab.total;
    if (gi >= uend) continue;
    unsigned u = (unsigned)(gi - t.ustart);
    const unsigned lim = (unsigned)(uend - t.ustart);
    const unsigned gpr = (unsigned)t.gpr;
    unsigned r = u / gpr, cb = u - r * gpr;          // row and column block of the group; advanced incrementally
    const unsigned sr = stride / gpr, sc = stride - sr * gpr;
    for (; u < lim; u += stride) {
      r2_group<A, APX>(t, u, r, cb, l16, hmask, c2, kf, Sm, Sv, lut_m, lut_ok, vlin, qm_l, qv_l, (u + stride < lim) ? stride : 0u);
      cb += sc;
      r += sr;
      if (cb >= gpr) {
        cb -= gpr;
        ++r;
      }
    }
    gi = t.ustart + u;
  }
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

// Host side.  `ts`: n tensors that all satisfy lpmm_b200_rank1_multi_ok.  Not part of the public header: called
// by lpmm_b200_adamw4bit_unfused_step_many.  The descriptors travel in the launch parameters: no scratch is needed.

LPMM_INTERNAL int lpmm_b200_rank1_multi_ok(const lpmm_b200_step_tensor* t) {
  if (!t || t->first || t->numel <= 0 || t->ndim != 2) return 0;
  if (t->m_mode != LPMM_B200_STATE_GROUP4 || t->v_mode != LPMM_B200_STATE_RANK1_4) return 0;
  if ((t->m_bits != 0 && t->m_bits != 4) || (t->v_bits != 0 && t->v_bits != 4)) return 0;
  if (t->m_group != 0 && t->m_group != 128) return 0;
  if (t->shape[1] % 8 != 0 || t->shape[0] <= 0 || t->shape[0] > 0x7fffffffLL || t->shape[1] > 0x7fffffffLL) return 0;
  if (t->shape[0] * t->shape[1] != t->numel) return 0;
  if (!t->p || !t->g || !t->m || !t->m_max1 || !t->v) return 0;
  for (int i = 0; i < 2; ++i)
    if (!t->v_max_dims_old[i] || !t->v_max_dims_new[i]) return 0;
  const uintptr_t a16 = (uintptr_t)t->p | (uintptr_t)t->g | (uintptr_t)t->v_max_dims_old[1] | (uintptr_t)t->v_max_dims_new[1];
  if (a16 & 15) return 0;
  if (((uintptr_t)t->m | (uintptr_t)t->v) & 3) return 0;
  return 1;
}

static int r1_occupancy(int* out) {
  static int stats_ctas[64] = {};  // CTAs of the statistics kernel one SM holds, per device
  int cur = 0;
  cudaGetDevice(&cur);
  int per_sm = (cur >= 0 && cur < 64) ? stats_ctas[cur] : 0;
  if (per_sm == 0) {
    LPMM_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, r1_stats_kernel<false>, R1T, 0));
    if (per_sm < 1) per_sm = 1;
    if (cur >= 0 && cur < 64) stats_ctas[cur] = per_sm;
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update2_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update2_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update2_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(r1_update2_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R1_DYN_SMEM));
  }
  *out = per_sm;
  return LPMM_B200_OK;
}

// One window of at most R1_MAX tensors: zero, statistics, update.
static int r1_window(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m, const float* qmap_v,
                     const UConsts& c, cudaStream_t st, int arith, int apx) {
  static thread_local R1Table tab;   // 32 KB; copied into the launch parameters by the runtime
  static thread_local R2Table tab2;
  static thread_local std::vector<int> order;
  order.clear();
  long long total_elems = 0;
  for (int i = 0; i < n; ++i) total_elems += ts[i]->numel;
  // Matrices whose rows are whole 128-element groups take the update kernel shaped like the fused step
  // (r1_update2_kernel); they come first in the table.  It has no scalar path, so it needs the short exact
  // sequences (hyper-parameters inside their domain) and 32-byte aligned parameters and gradients.
  const bool fast = arith ? c.f_fast != 0 : c.fast != 0;
  auto wide = [&](const lpmm_b200_step_tensor* t) {
    return fast && t->shape[1] % 128 == 0 && t->numel < ((long long)1 << 37) &&
           ((((uintptr_t)t->p | (uintptr_t)t->g | (uintptr_t)t->v_max_dims_old[1] | (uintptr_t)t->v_max_dims_new[1]) & 31) == 0);
  };
  for (int i = 0; i < n; ++i)
    if (wide(ts[i])) order.push_back(i);
  const int n_wide = (int)order.size();
  for (int i = 0; i < n; ++i)
    if (!wide(ts[i])) order.push_back(i);
  // statistics tiles: about sixteen per SM over the whole window, at least 4 rows each; a grid of resident CTAs
  // (as many of 256 threads as an SM holds) strides over them, so the last tiles level the load
  const long long target_tiles = (long long)num_sms() * 16;
  long long per_tile = (total_elems + target_tiles - 1) / target_tiles;
  if (per_tile < 8192) per_tile = 8192;
  long long units = 0, tiles = 0;  // units: 128-element units of the matrices that are NOT wide (numbered from 0)
  for (int k = 0; k < n; ++k) {
    const lpmm_b200_step_tensor* t = ts[order[k]];
    R1Desc& d = tab.t[k];
    d.p = t->p;
    d.g = t->g;
    d.m = reinterpret_cast<uint8_t*>(t->m);
    d.m_max1 = t->m_max1;
    d.v = reinterpret_cast<uint8_t*>(t->v);
    d.old_r = t->v_max_dims_old[0];
    d.old_c = t->v_max_dims_old[1];
    d.new_r = t->v_max_dims_new[0];
    d.new_c = t->v_max_dims_new[1];
    d.n = t->numel;
    d.R = (int)t->shape[0];
    d.C = (int)t->shape[1];
    d.ustart = units;
    d.tstart = tiles;
    const int shift = tile_shift(d.C);
    d.tx_shift = shift;
    d.pad_ = 0;
    const int tile_cols = 8 << shift;
    d.tiles_x = (d.C + tile_cols - 1) / tile_cols;
    const long long width = d.C < tile_cols ? d.C : tile_cols;
    long long rows = (per_tile + width - 1) / width;
    if (rows < 4) rows = 4;
    if (rows > d.R) rows = d.R;
    d.rows_per_tile = (int)rows;
    if (k >= n_wide) units += (t->numel + 127) / 128;
    tiles += (long long)d.tiles_x * ((d.R + rows - 1) / rows);
  }
  tab.n = n;
  tab.first = n_wide;
  tab.tiles = tiles;
  tab.units = units;
  int per_sm = 1;
  const int rc = r1_occupancy(&per_sm);
  if (rc != LPMM_B200_OK) return rc;
  r1_zero_kernel<<<(unsigned)n, R1T, 0, st>>>(tab);
  LPMM_CUDA_TRY(cudaGetLastError());
  const long long resident = (long long)num_sms() * per_sm;
  const long long sgrid = tiles < resident ? tiles : resident;
  if (arith) r1_stats_kernel<true><<<(unsigned)sgrid, R1T, 0, st>>>(tab, qmap_v, c);
  else r1_stats_kernel<false><<<(unsigned)sgrid, R1T, 0, st>>>(tab, qmap_v, c);
  LPMM_CUDA_TRY(cudaGetLastError());
  if (n_wide > 0) {
    long long g2 = 0;
    for (int k = 0; k < n_wide; ++k) {
      const R1Desc& d = tab.t[k];
      R2Desc& w = tab2.t[k];
      w.p = d.p;
      w.g = d.g;
      w.m = reinterpret_cast<uint32_t*>(d.m);
      w.v = reinterpret_cast<uint32_t*>(d.v);
      w.msc = d.m_max1;
      w.old_r = d.old_r;
      w.old_c = d.old_c;
      w.new_r = d.new_r;
      w.new_c = d.new_c;
      w.ustart = g2;
      w.gpr = d.C / 128;
      w.pad_ = 0;
      g2 += d.n / 128;
    }
    tab2.n = n_wide;
    tab2.pad_ = 0;
    tab2.total = g2;
    long long grid2 = (g2 + R2_HW - 1) / R2_HW;
    if (grid2 > num_sms()) grid2 = num_sms();
    // the folded constants of the fused arithmetic's tolerance mode need a finite 1 / lr
    const bool apx_ok = apx && (!arith || (c.f_lr >= 0x1p-60f && c.f_lr <= 0x1p30f && c.f_wd <= 0x1p30f));
    if (arith && apx_ok) r1_update2_kernel<true, true><<<(unsigned)grid2, R2T, R1_DYN_SMEM, st>>>(tab2, qmap_m, qmap_v, c);
    else if (arith) r1_update2_kernel<true, false><<<(unsigned)grid2, R2T, R1_DYN_SMEM, st>>>(tab2, qmap_m, qmap_v, c);
    else if (apx_ok) r1_update2_kernel<false, true><<<(unsigned)grid2, R2T, R1_DYN_SMEM, st>>>(tab2, qmap_m, qmap_v, c);
    else r1_update2_kernel<false, false><<<(unsigned)grid2, R2T, R1_DYN_SMEM, st>>>(tab2, qmap_m, qmap_v, c);
    LPMM_CUDA_TRY(cudaGetLastError());
  }
  if (n > n_wide) {
    long long ugrid = (units + R1T / 16 - 1) / (R1T / 16);
    const long long ucap = (long long)num_sms() * 4;
    if (ugrid > ucap) ugrid = ucap;
    if (arith) r1_update_kernel<true><<<(unsigned)ugrid, R1T, R1_DYN_SMEM, st>>>(tab, qmap_m, qmap_v, c);
    else r1_update_kernel<false><<<(unsigned)ugrid, R1T, R1_DYN_SMEM, st>>>(tab, qmap_m, qmap_v, c);
    LPMM_CUDA_TRY(cudaGetLastError());
  }
  return LPMM_B200_OK;
}

LPMM_INTERNAL int lpmm_b200_rank1_multi_step(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m,
                                          const float* qmap_v, double beta1, double beta2, double lr,
                                          double weight_decay, double eps, double step, void* stream, int arith,
                                          int apx) {
  if (n <= 0) return LPMM_B200_OK;
  if (!ts || !qmap_m || !qmap_v) return LPMM_B200_ERR_NULL_POINTER;
  for (int i = 0; i < n; ++i)
    if (!lpmm_b200_rank1_multi_ok(ts[i])) return LPMM_B200_ERR_UNSUPPORTED;
  const UConsts c = make_consts(beta1, beta2, lr, weight_decay, eps, step);
  static_assert(R1_MAX <= R2_MAX, "a window of wide matrices must fit the second table");
  for (int i = 0; i < n; i += R1_MAX) {
    const int cnt = (n - i < R1_MAX) ? n - i : R1_MAX;
    const int rc = r1_window(ts + i, cnt, qmap_m, qmap_v, c, (cudaStream_t)stream, arith, apx);
    if (rc != LPMM_B200_OK) return rc;
  }
  return LPMM_B200_OK;
}
