// The factored second moment (lpmm/optim/adamw.py:571-627: fp32 row and column accumulators of g^2,
// v reconstructed as row / mean(row) * col) for ALL matrices of a parameter list in four launches:
// partial row / column sums of g^2 over tiles, their reduction into the accumulators, the mean of each
// matrix's row accumulator, and the update pass (first moment 4-bit with group-128 scales or fp32).
// The reference does this per parameter in Python with a dozen torch kernels each.
//
// Everything is summed in a fixed order (no atomics), so results are reproducible; the order differs
// from torch's reductions, which is why the accumulators and parameters agree with the reference to
// 1e-6 relative rather than bit for bit (first-moment codes are still identical in the tests).
//
// The tensors are described by a table carried in the launch parameters (up to F_MAX per launch; a longer list is
// stepped in windows), so nothing is uploaded and the launches can be captured into a CUDA graph; tiles, rows,
// column blocks and 128-element units are numbered across the whole window and fixed grids stride over them.
#include <math.h>

#include <vector>

#include "common.cuh"
#include "multi_tensor.cuh"
#include "unfused_math.cuh"

namespace lpmm_b200 {

constexpr int FT = 256;  // threads per CTA
constexpr size_t F_DYN_SMEM = LUT_ENTRIES * sizeof(LutEnt);
constexpr int F_MIN_ROWS = 64;  // rows per tile at least: bounds the column partials by numel / 64 floats

struct FDesc {
  float* p;
  const float* g;
  uint8_t* m;       // codes (m_quant) or float[n]
  float* m_max1;
  float* row;       // accumulators
  float* col;
  float* row_part;  // [slots][R] partial row sums of g^2, slot = 256-column segment
  float* col_part;  // [tiles_y][C] partial column sums
  float* row_mean;  // one float
  long long n;
  long long ustart;  // first global 128-element unit
  long long tstart;  // first global tile
  long long rstart;  // first global row index among the rows of all tensors (finalize pass)
  long long cstart;  // first global 32-column block among the column blocks of all tensors (finalize pass)
  int R, C;
  int tiles_x, tiles_y, rows_per_tile, tx_shift, slots, m_quant;
};

constexpr int F_MAX = 224;  // descriptors per launch: 144 bytes each, 32 KB of launch parameters in all
struct FTable {
  int n;
  int first;            // index of the first descriptor the scalar update kernel steps (the wide ones come before)
  long long tiles;      // tiles of the sums pass
  long long units;      // 128-element units of the descriptors from `first` on
  long long rows;       // rows of all matrices of the window
  long long row_blocks; // CTAs of the finalize pass that take rows (the others take 32-column blocks)
  FDesc t[F_MAX];
};

template <int WHICH>  // 0: ustart, 1: tstart, 2: rstart, 3: cstart
__device__ __forceinline__ int f_find(const FDesc* d, int n, long long x) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    const long long s = WHICH == 0 ? d[mid].ustart : (WHICH == 1 ? d[mid].tstart : (WHICH == 2 ? d[mid].rstart : d[mid].cstart));
    if (s <= x) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// Pass 1.  A tile is (8 << tx_shift) columns by rows_per_tile rows; 2^tx_shift column-threads (8 columns
// each) by 256 >> tx_shift row-lanes.  Column sums: per thread over its rows (in row order), then over the
// row-lanes in lane order through shared memory.  Row sums: the thread's 8 squares in column order, then a
// butterfly over the lanes that share the row inside a warp; one partial per 256-column segment.
__global__ void __launch_bounds__(FT) f_sums_kernel(const __grid_constant__ FTable tab) {
  const FDesc* d = tab.t;
  const int n = tab.n;
  const long long total_tiles = tab.tiles;
  __shared__ float colbuf[8 * FT];
  for (long long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const FDesc& t = d[f_find<1>(d, n, tile)];
    const long long local = tile - t.tstart;
    const int tx_count = 1 << t.tx_shift, ty_count = FT >> t.tx_shift;
    const int tx = threadIdx.x & (tx_count - 1), ty = threadIdx.x >> t.tx_shift;
    const int tile_x = (int)(local % t.tiles_x);
    const long long tile_y = local / t.tiles_x;
    const long long C = t.C;
    const long long c0 = ((long long)tile_x * tx_count + tx) * 8;
    const bool active = c0 < C;
    const long long r_begin = tile_y * t.rows_per_tile;
    const long long r_end = (r_begin + t.rows_per_tile < t.R) ? r_begin + t.rows_per_tile : t.R;
    const int seg = tx_count < 32 ? tx_count : 32;
    const int slot = (int)(c0 >> 8);  // 256-column segment of this thread's columns (seg * 8 columns each when seg == 32)
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    // the loads of the next pair of rows are issued before the sums of the current pair (two pairs in flight)
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 na0 = zero4, na1 = zero4, nb0 = zero4, nb1 = zero4;
    {
      const long long ra = r_begin + ty, rc = r_begin + ty_count + ty;
      if (active && ra < r_end) {
        na0 = *reinterpret_cast<const float4*>(t.g + ra * C + c0);
        na1 = *reinterpret_cast<const float4*>(t.g + ra * C + c0 + 4);
      }
      if (active && rc < r_end) {
        nb0 = *reinterpret_cast<const float4*>(t.g + rc * C + c0);
        nb1 = *reinterpret_cast<const float4*>(t.g + rc * C + c0 + 4);
      }
    }
    for (long long rb = r_begin; rb < r_end; rb += 2 * ty_count) {
      const long long ra = rb + ty, rc = rb + ty_count + ty;
      const float4 a0 = na0, a1 = na1, b0 = nb0, b1 = nb1;
      {
        const long long rn = rb + 2 * ty_count;
        const long long ra2 = rn + ty, rc2 = rn + ty_count + ty;
        na0 = na1 = nb0 = nb1 = zero4;
        if (active && ra2 < r_end) {
          na0 = *reinterpret_cast<const float4*>(t.g + ra2 * C + c0);
          na1 = *reinterpret_cast<const float4*>(t.g + ra2 * C + c0 + 4);
        }
        if (active && rc2 < r_end) {
          nb0 = *reinterpret_cast<const float4*>(t.g + rc2 * C + c0);
          nb1 = *reinterpret_cast<const float4*>(t.g + rc2 * C + c0 + 4);
        }
      }
      const float ga[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float gb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      float sa = 0.0f, sb = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float qa = __fmul_rn(ga[k], ga[k]), qb = __fmul_rn(gb[k], gb[k]);
        acc[k] = __fadd_rn(__fadd_rn(acc[k], qa), qb);  // rows ra then rc: ascending row order per thread
        sa = __fadd_rn(sa, qa);
        sb = __fadd_rn(sb, qb);
      }
      for (int o = seg >> 1; o; o >>= 1) {
        sa = __fadd_rn(sa, __shfl_xor_sync(0xffffffffu, sa, o));
        sb = __fadd_rn(sb, __shfl_xor_sync(0xffffffffu, sb, o));
      }
      if ((threadIdx.x & (seg - 1)) == 0 && active) {
        if (ra < r_end) t.row_part[(long long)slot * t.R + ra] = sa;
        if (rc < r_end) t.row_part[(long long)slot * t.R + rc] = sb;
      }
    }
    // column sums of the tile: row-lanes in order
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) colbuf[k * FT + threadIdx.x] = acc[k];
    __syncthreads();
    if (ty == 0 && active) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float s = acc[k];
        for (int j = 1; j < ty_count; ++j) s = __fadd_rn(s, colbuf[k * FT + j * tx_count + tx]);
        t.col_part[tile_y * C + c0 + k] = s;
      }
    }
  }
}

// Pass 2: partials into the accumulators,  acc = fma(1 - beta2, mean, acc * beta2)  (adamw.py:609-610:
// mul_(beta2).add_(mean, alpha=1-beta2)).  The first row_blocks CTAs take 256 rows each (any matrix): a row's
// few segment partials in slot order.  The other CTAs take 32 columns of one matrix each: a tall matrix has
// hundreds of tile partials per column, so the CTA's 8 warps share them (warp w sums tiles w, w + 8, ... in
// order) and the 8 sums are added in warp order.  Fixed order throughout: results are reproducible.
__global__ void __launch_bounds__(FT) f_finalize_kernel(const __grid_constant__ FTable tab, const UConsts c) {
  const FDesc* d = tab.t;
  const int n = tab.n;
  const long long total_rows = tab.rows, row_blocks = tab.row_blocks;
  __shared__ float part[8][32];
  if ((long long)blockIdx.x < row_blocks) {
    const long long i = (long long)blockIdx.x * FT + threadIdx.x;
    if (i >= total_rows) return;
    const FDesc& t = d[f_find<2>(d, n, i)];
    const long long j = i - t.rstart;
    float s = 0.0f;
    for (int k = 0; k < t.slots; ++k) s = __fadd_rn(s, t.row_part[(long long)k * t.R + j]);
    t.row[j] = __fmaf_rn(c.omb2, __fdiv_rn(s, (float)t.C), __fmul_rn(t.row[j], c.beta2));
    return;
  }
  const long long cblock = (long long)blockIdx.x - row_blocks;
  const FDesc& t = d[f_find<3>(d, n, cblock)];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long cc = (cblock - t.cstart) * 32 + lane;
  float s = 0.0f;
  if (cc < t.C)
    for (int k = w; k < t.tiles_y; k += 8) s = __fadd_rn(s, t.col_part[(long long)k * t.C + cc]);
  part[w][lane] = s;
  __syncthreads();
  if (w == 0 && cc < t.C) {
    float sum = part[0][lane];
#pragma unroll
    for (int k = 1; k < 8; ++k) sum = __fadd_rn(sum, part[k][lane]);
    t.col[cc] = __fmaf_rn(c.omb2, __fdiv_rn(sum, (float)t.R), __fmul_rn(t.col[cc], c.beta2));
  }
}

// Pass 3: mean of each matrix's updated row accumulator, one CTA of 1024 threads per matrix, fixed order; then
// row[r] / mean for every row, for the update pass of wide matrices (f_update2_kernel): the first slot of the row
// partials is free again after pass 2.
constexpr int FMT = 1024;
__global__ void __launch_bounds__(FMT) f_row_mean_kernel(const __grid_constant__ FTable tab) {
  __shared__ float red[FMT];
  const FDesc& t = tab.t[blockIdx.x];
  float acc = 0.0f;
  for (long long j = threadIdx.x; j < t.R; j += FMT) acc = __fadd_rn(acc, t.row[j]);
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = FMT / 2; o; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    red[0] = __fdiv_rn(red[0], (float)t.R);
    *t.row_mean = red[0];
  }
  __syncthreads();
  const float mean = red[0];
  for (long long j = threadIdx.x; j < t.R; j += FMT) t.row_part[j] = __fdiv_rn(t.row[j], mean);
}


// Pass 4: one 128-element unit: v = (row / row_mean) * col, AdamW, first moment requantised.
__device__ __forceinline__ void f_unit(const FDesc& t, long long u, int l16, unsigned hmask, const UConsts& c,
                                       const UConsts2& c2, const QMapSmem& Sm, const LutEnt* __restrict__ lut_m,
                                       bool lut_ok) {
  const long long n = t.n, C = t.C;
  const long long e0 = u * 128 + l16 * 8;
  const bool has_data = e0 < n;
  const bool mq = t.m_quant != 0;
  uint8_t* mb = t.m + (e0 >> 1);
  float* mf = reinterpret_cast<float*>(t.m);
  uint32_t mcodes = 0;
  float sm = 0.0f;
  if (has_data && mq) {
    mcodes = *reinterpret_cast<const uint32_t*>(mb);
    sm = t.m_max1[u];
  }
  const float mean = *t.row_mean;
  float m[8];
  float am = 0.0f;
  const bool full = c.fast && (e0 + 8 <= n);  // C % 8 == 0: the lane lies inside one row; bases 16-byte aligned
  if (full) {
    const long long r = ((e0 | C) >> 32) ? e0 / C : (long long)((unsigned)e0 / (unsigned)C);
    const long long col = e0 - r * C;
    const float rf = __fdiv_rn(t.row[r], mean);
    const float4 c0 = *reinterpret_cast<const float4*>(t.col + col), c1 = *reinterpret_cast<const float4*>(t.col + col + 4);
    const float4 a0 = *reinterpret_cast<const float4*>(t.g + e0), a1 = *reinterpret_cast<const float4*>(t.g + e0 + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(t.p + e0), b1 = *reinterpret_cast<const float4*>(t.p + e0 + 4);
    const f2 g[4] = {f2_pack(a0.x, a0.y), f2_pack(a0.z, a0.w), f2_pack(a1.x, a1.y), f2_pack(a1.z, a1.w)};
    f2 p[4] = {f2_pack(b0.x, b0.y), f2_pack(b0.z, b0.w), f2_pack(b1.x, b1.y), f2_pack(b1.z, b1.w)};
    const f2 cv[4] = {f2_pack(c0.x, c0.y), f2_pack(c0.z, c0.w), f2_pack(c1.x, c1.y), f2_pack(c1.z, c1.w)};
    const f2 rf2 = f2_splat(rf), sm2 = f2_splat(sm);
    float px[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k0 = 2 * j, k1 = 2 * j + 1;
      f2 m0;
      if (mq) m0 = f2_mul(f2_pack(Sm.qmap[(mcodes >> (4 * k0)) & 15u], Sm.qmap[(mcodes >> (4 * k1)) & 15u]), sm2);
      else m0 = f2_pack(mf[e0 + k0], mf[e0 + k1]);
      const f2 mj = lerp_pair(c2, g[j], m0, am);
      const f2 vj = f2_mul(rf2, cv[j]);
      param_pair(c2, p[j], mj, vj);
      f2_unpack(mj, m[k0], m[k1]);
      f2_unpack(p[j], px[k0], px[k1]);
      if (!mq) {
        mf[e0 + k0] = m[k0];
        mf[e0 + k1] = m[k1];
      }
    }
    *reinterpret_cast<float4*>(t.p + e0) = make_float4(px[0], px[1], px[2], px[3]);
    *reinterpret_cast<float4*>(t.p + e0 + 4) = make_float4(px[4], px[5], px[6], px[7]);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const long long e = e0 + k;
      m[k] = 0.0f;
      if (e < n) {
        const long long rr = e / C, cc = e - rr * C;
        const float v = __fmul_rn(__fdiv_rn(t.row[rr], mean), t.col[cc]);
        const float g = t.g[e];
        const float m0 = mq ? __fmul_rn(Sm.qmap[(mcodes >> (4 * k)) & 15u], sm) : mf[e];
        m[k] = lerp_m(c, m0, g);
        t.p[e] = upd_param(c, t.p[e], m[k], v);
        am = fmaxf(am, fabsf(m[k]));
        if (!mq) mf[e] = m[k];
      }
    }
  }
  if (!mq) return;  // uniform per tensor
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
  *reinterpret_cast<uint32_t*>(mb) = mo;  // inside the padded layout for every lane of the unit
  if (l16 == 0) t.m_max1[u] = am;
}

__global__ void __launch_bounds__(FT, 4) f_update_kernel(const __grid_constant__ FTable tab,
                                                          const float* __restrict__ qmap_m, const UConsts c) {
  const FDesc* d = tab.t + tab.first;
  const int n = tab.n - tab.first;
  const long long total_units = tab.units;
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  bool lut_ok = false;
  if (qmap_m) {
    lut_build(Sm, lut_m, qmap_m);
    lut_ok = Sm.valid != 0;
  }
  const UConsts2 c2 = make_consts2(c);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  long long gi = (long long)blockIdx.x * (FT / 16) + (threadIdx.x >> 4);
  const long long stride = (long long)gridDim.x * (FT / 16);
  for (int ti = 0; ti < n; ++ti) {
    const FDesc& t = d[ti];
    const long long uend = (ti + 1 < n) ? d[ti + 1].ustart : total_units;
    for (; gi < uend; gi += stride) f_unit(t, gi - t.ustart, l16, hmask, c, c2, Sm, lut_m, lut_ok);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Pass 4 for matrices whose row length is a multiple of 128 with a 4-bit first moment: a 128-element group lies
// inside one row, so the half-warp shares row[r] / mean(row) (read from the vector pass 3 left in row_part) and a
// lane's 8 elements are 8 consecutive columns.  Shape of the fused multi-tensor step (adamw4bit.cu): descriptors in
// the launch parameters, persistent 1024-thread CTAs, 256-bit accesses, dequantisation by shuffle, packed fp32x2
// arithmetic, table look-up for the codes.  Arithmetic is that of f_unit's FULL lanes, bit for bit.
// ---------------------------------------------------------------------------------------------------------
constexpr int F2_MAX = 400;
constexpr int F2T = 1024;
constexpr int F2_HW = F2T / 16;

struct F2Desc {
  float* p;
  const float* g;
  uint32_t* m;
  float* msc;
  const float* rowf;   // row[r] / mean(row)
  const float* col;
  long long ustart;
  int gpr;             // groups per row: C / 128
  int pad_;
};
struct F2Table {
  int n;
  int pad_;
  long long total;
  F2Desc t[F2_MAX];
};

template <bool APX>  // APX: the tolerance mode of the parameter update (unfused_math.cuh)
__device__ __forceinline__ void f2_group(const F2Desc& t, unsigned u, unsigned r, unsigned cb, int l16, unsigned hmask,
                                         const UConsts2& c2, const QMapSmem& Sm, const LutEnt* __restrict__ lut_m,
                                         bool lut_ok, float qm_l, unsigned pf) {
  const size_t e0 = (size_t)u * 128 + (size_t)l16 * 8;
  float* pp = t.p + e0;
  const float* gp = t.g + e0;
  uint32_t* mcp = t.m + (size_t)u * 16 + l16;
  f2x4 p = ldg_f2x4(pp);
  const f2x4 g = ldg_f2x4(gp);
  const uint32_t mc = *mcp;
  const float pm = __fmul_rn(qm_l, t.msc[u]);
  const f2 rf2 = f2_splat(__ldg(t.rowf + r));
  const f2x4 cv = ldg_f2x4(t.col + (size_t)cb * 128 + (size_t)l16 * 8);
  if (pf) {
    prefetch_l2(pp + (size_t)pf * 128);
    prefetch_l2(gp + (size_t)pf * 128);
    prefetch_l2(mcp + (size_t)pf * 16);
  }
  f2 m[4];
  float am = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float m0a = __shfl_sync(hmask, pm, (int)(mc >> (8 * j)), 16);
    const float m0b = __shfl_sync(hmask, pm, (int)(mc >> (8 * j + 4)), 16);
    m[j] = lerp_pair(c2, g.v[j], f2_pack(m0a, m0b), am);
    if (APX) param_pair_apx(c2, p.v[j], m[j], f2_mul(rf2, cv.v[j]));
    else param_pair(c2, p.v[j], m[j], f2_mul(rf2, cv.v[j]));
  }
  stg_f2x4(pp, p);
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
  *mcp = mo;
  if (l16 == 0) t.msc[u] = am;
}

template <bool APX>
__global__ void __launch_bounds__(F2T, 1) f_update2_kernel(const __grid_constant__ F2Table tab,
                                                           const float* __restrict__ qmap_m, const UConsts c) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem Sm;
  LutEnt* lut_m = reinterpret_cast<LutEnt*>(dyn_smem);
  lut_build(Sm, lut_m, qmap_m);
  const bool lut_ok = Sm.valid != 0;
  const UConsts2 c2 = make_consts2(c);
  const int l16 = threadIdx.x & 15;
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const float qm_l = Sm.qmap[l16];
  long long gi = (long long)blockIdx.x * F2_HW + (threadIdx.x >> 4);
  const unsigned stride = gridDim.x * F2_HW;
  for (int ti = 0; ti < tab.n; ++ti) {
    const F2Desc& t = tab.t[ti];
    const long long uend = (ti + 1 < tab.n) ? tab.t[ti + 1].ustart : tab.total;
    if (gi >= uend) continue;
    unsigned u = (unsigned)(gi - t.ustart);
    const unsigned lim = (unsigned)(uend - t.ustart);
    const unsigned gpr = (unsigned)t.gpr;
    unsigned r = u / gpr, cb = u - r * gpr;
    const unsigned sr = stride / gpr, sc = stride - sr * gpr;
    for (; u < lim; u += stride) {
      f2_group<APX>(t, u, r, cb, l16, hmask, c2, Sm, lut_m, lut_ok, qm_l, (u + stride < lim) ? stride : 0u);
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

static inline int64_t f_align(int64_t x) { return (x + 63) & ~(int64_t)63; }  // floats: 256-byte granules

}  // namespace lpmm_b200

using namespace lpmm_b200;

// Host side; internal to the library (called by lpmm_b200_adamw4bit_unfused_step_many).
LPMM_INTERNAL int lpmm_b200_factored_multi_ok(const lpmm_b200_step_tensor* t) {
  if (!t || t->first || t->numel <= 0 || t->ndim != 2 || t->v_mode != LPMM_B200_STATE_FACTORED) return 0;
  if (t->m_mode != LPMM_B200_STATE_FP32 && t->m_mode != LPMM_B200_STATE_GROUP4) return 0;
  if (t->m_mode == LPMM_B200_STATE_GROUP4) {
    if ((t->m_bits != 0 && t->m_bits != 4) || (t->m_group != 0 && t->m_group != 128) || !t->m_max1) return 0;
    if ((uintptr_t)t->m & 3) return 0;
  }
  if (t->shape[1] % 8 != 0 || t->shape[0] <= 0 || t->shape[0] > 0x7fffffffLL || t->shape[1] > 0x7fffffffLL) return 0;
  if (t->shape[0] * t->shape[1] != t->numel) return 0;
  if (!t->p || !t->g || !t->m || !t->row || !t->col) return 0;
  if (((uintptr_t)t->p | (uintptr_t)t->g | (uintptr_t)t->col) & 15) return 0;
  return 1;
}

// Bytes of device scratch the list needs: one row-mean slot per tensor and the partial sums (column partials for
// tiles of at least F_MIN_ROWS rows, row partials per 256-column segment).
LPMM_INTERNAL int64_t lpmm_b200_factored_multi_scratch_bytes(const lpmm_b200_step_tensor* const* ts, int n) {
  int64_t floats = 0;
  for (int i = 0; i < n; ++i) {
    const int64_t R = ts[i]->shape[0], C = ts[i]->shape[1];
    floats += f_align(((R + F_MIN_ROWS - 1) / F_MIN_ROWS) * C) + f_align(((C + 255) / 256) * R) + 64;
  }
  return 4 * floats;
}

static int f_occupancy(int* out) {
  static int sums_ctas[64] = {};  // CTAs of the sums kernel one SM holds, per device
  int cur = 0;
  cudaGetDevice(&cur);
  int per_sm = (cur >= 0 && cur < 64) ? sums_ctas[cur] : 0;
  if (per_sm == 0) {
    LPMM_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, f_sums_kernel, FT, 0));
    if (per_sm < 1) per_sm = 1;
    if (cur >= 0 && cur < 64) sums_ctas[cur] = per_sm;
    LPMM_CUDA_TRY(cudaFuncSetAttribute(f_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(f_update2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_DYN_SMEM));
    LPMM_CUDA_TRY(cudaFuncSetAttribute(f_update2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_DYN_SMEM));
  }
  *out = per_sm;
  return LPMM_B200_OK;
}

// One window of at most F_MAX tensors; fbase: this window's slice of the partial-sum scratch.
static int f_window(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m, bool any_q, const UConsts& c,
                    float* fbase, cudaStream_t st, int apx) {
  static thread_local FTable tab;  // 32 KB; copied into the launch parameters by the runtime
  static thread_local F2Table tab2;
  static thread_local std::vector<int> order;
  order.clear();
  long long total_elems = 0;
  for (int i = 0; i < n; ++i) total_elems += ts[i]->numel;
  // Matrices whose rows are whole 128-element groups, with a 4-bit first moment, take f_update2_kernel; they come
  // first in the table.  That kernel has no scalar path: it needs the short exact sequences and 32-byte alignment.
  auto wide = [&](const lpmm_b200_step_tensor* t) {
    return c.fast != 0 && t->m_mode == LPMM_B200_STATE_GROUP4 && t->shape[1] % 128 == 0 && t->numel < ((long long)1 << 37) &&
           ((((uintptr_t)t->p | (uintptr_t)t->g | (uintptr_t)t->col) & 31) == 0);
  };
  for (int i = 0; i < n; ++i)
    if (wide(ts[i])) order.push_back(i);
  const int n_wide = (int)order.size();
  for (int i = 0; i < n; ++i)
    if (!wide(ts[i])) order.push_back(i);
  // about twenty tiles per SM; a grid of resident CTAs (as many as the SMs hold) strides over them
  const long long target_tiles = (long long)num_sms() * 20;
  long long per_tile = (total_elems + target_tiles - 1) / target_tiles;
  if (per_tile < 8192) per_tile = 8192;
  long long units = 0, tiles = 0, rows_total = 0, cblocks = 0;  // units: of the matrices that are NOT wide, from 0
  int64_t foff = 0;
  for (int k = 0; k < n; ++k) {
    const lpmm_b200_step_tensor* t = ts[order[k]];
    FDesc& d = tab.t[k];
    d.p = t->p;
    d.g = t->g;
    d.m = reinterpret_cast<uint8_t*>(t->m);
    d.m_max1 = t->m_max1;
    d.row = t->row;
    d.col = t->col;
    d.n = t->numel;
    d.R = (int)t->shape[0];
    d.C = (int)t->shape[1];
    d.m_quant = t->m_mode == LPMM_B200_STATE_GROUP4;
    const int shift = tile_shift(d.C);
    d.tx_shift = shift;
    const int tile_cols = 8 << shift;
    d.tiles_x = (d.C + tile_cols - 1) / tile_cols;
    const long long width = d.C < tile_cols ? d.C : tile_cols;
    long long rows = (per_tile + width - 1) / width;
    if (rows < F_MIN_ROWS) rows = F_MIN_ROWS;
    if (rows > d.R) rows = d.R;
    d.rows_per_tile = (int)rows;
    d.tiles_y = (int)((d.R + rows - 1) / rows);
    d.slots = (d.C + 255) / 256;
    d.col_part = fbase + foff;
    foff += f_align((int64_t)d.tiles_y * d.C);
    d.row_part = fbase + foff;
    foff += f_align((int64_t)d.slots * d.R);
    d.row_mean = fbase + foff;
    foff += 64;
    d.ustart = units;
    d.tstart = tiles;
    d.rstart = rows_total;
    d.cstart = cblocks;
    if (k >= n_wide) units += (t->numel + 127) / 128;
    tiles += (long long)d.tiles_x * d.tiles_y;
    rows_total += d.R;
    cblocks += (d.C + 31) / 32;
  }
  tab.n = n;
  tab.first = n_wide;
  tab.tiles = tiles;
  tab.units = units;
  tab.rows = rows_total;
  tab.row_blocks = (rows_total + FT - 1) / FT;
  int per_sm = 1;
  const int rc = f_occupancy(&per_sm);
  if (rc != LPMM_B200_OK) return rc;
  const long long resident = (long long)num_sms() * per_sm;
  const long long sgrid = tiles < resident ? tiles : resident;
  f_sums_kernel<<<(unsigned)sgrid, FT, 0, st>>>(tab);
  LPMM_CUDA_TRY(cudaGetLastError());
  f_finalize_kernel<<<(unsigned)(tab.row_blocks + cblocks), FT, 0, st>>>(tab, c);
  LPMM_CUDA_TRY(cudaGetLastError());
  f_row_mean_kernel<<<(unsigned)n, FMT, 0, st>>>(tab);
  LPMM_CUDA_TRY(cudaGetLastError());
  if (n_wide > 0) {
    long long g2 = 0;
    for (int k = 0; k < n_wide; ++k) {
      const FDesc& d = tab.t[k];
      F2Desc& w = tab2.t[k];
      w.p = d.p;
      w.g = d.g;
      w.m = reinterpret_cast<uint32_t*>(d.m);
      w.msc = d.m_max1;
      w.rowf = d.row_part;
      w.col = d.col;
      w.ustart = g2;
      w.gpr = d.C / 128;
      w.pad_ = 0;
      g2 += d.n / 128;
    }
    tab2.n = n_wide;
    tab2.pad_ = 0;
    tab2.total = g2;
    long long grid2 = (g2 + F2_HW - 1) / F2_HW;
    if (grid2 > num_sms()) grid2 = num_sms();
    if (apx) f_update2_kernel<true><<<(unsigned)grid2, F2T, F_DYN_SMEM, st>>>(tab2, qmap_m, c);
    else f_update2_kernel<false><<<(unsigned)grid2, F2T, F_DYN_SMEM, st>>>(tab2, qmap_m, c);
    LPMM_CUDA_TRY(cudaGetLastError());
  }
  if (n > n_wide) {
    long long ugrid = (units + FT / 16 - 1) / (FT / 16);
    const long long ucap = (long long)num_sms() * 4;
    if (ugrid > ucap) ugrid = ucap;
    f_update_kernel<<<(unsigned)ugrid, FT, F_DYN_SMEM, st>>>(tab, any_q ? qmap_m : nullptr, c);
    LPMM_CUDA_TRY(cudaGetLastError());
  }
  return LPMM_B200_OK;
}

LPMM_INTERNAL int lpmm_b200_factored_multi_step(const lpmm_b200_step_tensor* const* ts, int n, const float* qmap_m,
                                             double beta1, double beta2, double lr, double weight_decay, double eps,
                                             double step, void* scratch, int64_t scratch_bytes, void* stream, int apx) {
  if (n <= 0) return LPMM_B200_OK;
  if (!ts || !scratch) return LPMM_B200_ERR_NULL_POINTER;
  bool any_q = false;
  for (int i = 0; i < n; ++i) {
    if (!lpmm_b200_factored_multi_ok(ts[i])) return LPMM_B200_ERR_UNSUPPORTED;
    any_q = any_q || ts[i]->m_mode == LPMM_B200_STATE_GROUP4;
  }
  if (any_q && !qmap_m) return LPMM_B200_ERR_NULL_POINTER;
  if (scratch_bytes < lpmm_b200_factored_multi_scratch_bytes(ts, n)) return LPMM_B200_ERR_BAD_SIZE;
  if ((uintptr_t)scratch & 255) return LPMM_B200_ERR_BAD_SIZE;
  const UConsts c = make_consts(beta1, beta2, lr, weight_decay, eps, step);
  static_assert(F_MAX <= F2_MAX, "a window of wide matrices must fit the second table");
  char* base = static_cast<char*>(scratch);
  for (int i = 0; i < n; i += F_MAX) {
    const int cnt = (n - i < F_MAX) ? n - i : F_MAX;
    const int rc = f_window(ts + i, cnt, qmap_m, any_q, c, reinterpret_cast<float*>(base), (cudaStream_t)stream, apx);
    if (rc != LPMM_B200_OK) return rc;
    base += lpmm_b200_factored_multi_scratch_bytes(ts + i, cnt);  // multiples of 256 bytes
  }
  return LPMM_B200_OK;
}
