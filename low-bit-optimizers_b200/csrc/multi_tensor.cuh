// Descriptor table of the one-launch multi-tensor steps (AdamW and SGD): the whole parameter list
// travels in the kernel parameters, and every half-warp walks the global sequence of 128-element
// groups through it.
#pragma once
#include "common.cuh"

namespace lpmm_b200 {

constexpr int MAX_TENSORS = 400;  // descriptors per launch (28.9 KB of the 32 KB parameter space)
// One 1024-thread CTA per SM: measured faster than 2 x 512 or 3 x 256 (6.2 vs 5.9 vs 5.3 TB/s in a burst).
// Tuning knobs, overridable at compile time for experiments; the defaults are the measured best.
#ifndef LPMM_PF_DIST
#define LPMM_PF_DIST 1
#endif
#ifndef LPMM_CTA_THREADS
#define LPMM_CTA_THREADS 1024
#endif
#ifndef LPMM_CTAS_PER_SM
#define LPMM_CTAS_PER_SM 1
#endif
constexpr unsigned PF_DIST = LPMM_PF_DIST;  // the L2 prefetch runs this many of a half-warp's iterations ahead (0: none; 2: same, 3: slower)
constexpr int CTA_THREADS = LPMM_CTA_THREADS;
constexpr int CTAS_PER_SM = LPMM_CTAS_PER_SM;
constexpr int HW_PER_CTA = CTA_THREADS / 16;

struct TDesc {
  float* p;
  const float* g;
  void* m;
  void* v;
  float* sm;
  float* sv;
  long long numel;
  long long gstart;  // first global group index of this tensor
  int kind;          // LPMM_B200_KIND_*
  int aligned;       // all pointers satisfy the vector-access alignment
};

struct Table {
  int n;
  int pad;
  long long gtotal;  // groups in this table
  TDesc t[MAX_TENSORS];
};


// Peers of a ZeRO-1 step for 16-bit parameters: byte offsets from an address in this GPU's flat parameter buffer to
// the same element in each peer's buffer (peer-mapped memory).  Every updated parameter is stored locally and at
// each of these offsets.
struct PeerStores {
  int n;
  int pad_;
  long long off[7];
};

// Maximum of a non-negative value over the half-warp.
__device__ __forceinline__ float hw_max(float x, unsigned mask) {
#ifdef LPMM_HWMAX_REDUX  // one integer warp reduction on the bit patterns (experiment; measured no faster)
  return __uint_as_float(__reduce_max_sync(mask, __float_as_uint(x)));
#else
#pragma unroll
  for (int o = 8; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(mask, x, o, 16));
  return x;
#endif
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

static inline int64_t groups_of(int64_t numel) { return (numel + 127) / 128; }

// Column-threads of a statistics / sums tile of the list-wide rank-1 and factored passes: a tile is 8 << shift
// columns wide (each of 2^shift column-threads owns 8 columns).  A row shorter than 2048 columns takes the power
// of two that covers it; a longer one the width among 2048, 1024, 512, 256 that leaves the fewest idle columns in
// its last tile (3072 -> 1024, 11008 -> 256), the wider one on a tie.
static inline int tile_shift(long long C) {
  int shift = 0;
  while (shift < 8 && (8LL << shift) < C) ++shift;
  if ((8LL << shift) >= C) return shift;
  int best = 8;
  long long best_waste = -1;
  for (int sh = 8; sh >= 5; --sh) {
    const long long w = 8LL << sh;
    const long long waste = (C + w - 1) / w * w - C;
    if (best_waste < 0 || waste < best_waste) {
      best = sh;
      best_waste = waste;
    }
  }
  return best;
}

// Host side of every multi-tensor launch.  A list may hold more tensors than a table: it is walked in
// windows of at most MAX_TENSORS non-empty tensors, one launch per window over the part of the
// caller's group range [gbeg, gend) that falls inside it.
struct Window {
  int64_t lo, hi;  // the launch's group range, relative to the window
  bool any_q4;     // the window holds a 4-bit tensor (tables needed)
  bool work;       // false: nothing of [gbeg, gend) lies in this window
};
// Fills `tab` from ts[i...] and advances i and gcursor (global group index of the next window's first
// tensor).  uses_v: the step has a second state (AdamW); otherwise v / v_scale are ignored (SGD).
// `aligned` of a 4-bit tensor: p, g 32-byte aligned (256-bit accesses), codes 4-byte aligned; of an
// fp32-state tensor: everything 32-byte aligned.
static inline Window next_window(const lpmm_b200_tensor* ts, int n, int& i, int64_t& gcursor, int64_t gbeg, int64_t gend,
                                 bool uses_v, Table& tab) {
  int cnt = 0;
  int64_t g = 0;
  Window w = {0, 0, false, false};
  for (; i < n && cnt < MAX_TENSORS; ++i) {
    const lpmm_b200_tensor& s = ts[i];
    if (s.numel == 0) continue;
    TDesc& d = tab.t[cnt++];
    d.p = s.p;
    d.g = s.g;
    d.m = s.m;
    d.v = uses_v ? s.v : nullptr;
    d.sm = s.m_scale;
    d.sv = uses_v ? s.v_scale : nullptr;
    d.numel = s.numel;
    d.gstart = g;
    d.kind = s.kind;
    w.any_q4 = w.any_q4 || s.kind == LPMM_B200_KIND_Q4;
    const uintptr_t pg = (uintptr_t)s.p | (uintptr_t)s.g;
    const uintptr_t states = (uintptr_t)s.m | (uses_v ? (uintptr_t)s.v : 0);
    d.aligned = (s.kind == LPMM_B200_KIND_Q4) ? (((pg & 31) == 0) && ((states & 3) == 0)) : (((pg | states) & 31) == 0);
    g += groups_of(s.numel);
  }
  tab.n = cnt;
  tab.pad = 0;
  tab.gtotal = g;
  w.lo = (gbeg > gcursor ? gbeg : gcursor) - gcursor;
  w.hi = (gend < gcursor + g ? gend : gcursor + g) - gcursor;
  gcursor += g;
  w.work = cnt > 0 && w.hi > w.lo;
  return w;
}
// One CTA per SM at most (persistent CTAs stride over the groups).
static inline unsigned multi_grid(const Window& w) {
  int64_t grid = (w.hi - w.lo + HW_PER_CTA - 1) / HW_PER_CTA;
  const int64_t cap = (int64_t)num_sms() * CTAS_PER_SM;
  return (unsigned)(grid > cap ? cap : grid);
}
// Argument checks shared by the list entry points; total receives the list's group count.
static inline int check_tensor_list(const lpmm_b200_tensor* ts, int n, bool uses_v, bool* any_q4, int64_t* total) {
  if (n < 0) return LPMM_B200_ERR_BAD_SIZE;
  if (n > 0 && !ts) return LPMM_B200_ERR_NULL_POINTER;
  *any_q4 = false;
  *total = 0;
  for (int i = 0; i < n; ++i) {
    const lpmm_b200_tensor& s = ts[i];
    if (s.numel < 0) return LPMM_B200_ERR_BAD_SIZE;
    if (s.numel > (int64_t)1 << 37) return LPMM_B200_ERR_TOO_LARGE;  // 32-bit group index per tensor
    if (s.kind != LPMM_B200_KIND_Q4 && s.kind != LPMM_B200_KIND_FP32) return LPMM_B200_ERR_BAD_KIND;
    *total += groups_of(s.numel);
    if (s.numel == 0) continue;
    if (!s.p || !s.g || !s.m || (uses_v && !s.v)) return LPMM_B200_ERR_NULL_POINTER;
    if (s.kind == LPMM_B200_KIND_Q4) {
      *any_q4 = true;
      if (!s.m_scale || (uses_v && !s.v_scale)) return LPMM_B200_ERR_NULL_POINTER;
    }
  }
  return LPMM_B200_OK;
}

}  // namespace lpmm_b200
