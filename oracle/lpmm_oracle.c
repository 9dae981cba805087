/*
 * lpmm_oracle.c -- CPU restatement of the reference's 4-bit optimizer-step arithmetic.
 *
 * TEST INFRASTRUCTURE.  Only tests, the smoke check and the CPU-baseline legs of the benchmark
 * may call this; the product (the CUDA library) never does and has no CPU path.
 *
 * Parity status: PINNED.  The fused step below reproduces, bit for bit, the outputs of the
 * reference's own CUDA kernels compiled unmodified for sm_100a and run on a B200 (fixtures under
 * tests/golden/fused_*.npz, made by tests/golden/make_fused_golden.py), and the pack/unpack pair
 * reproduces the reference's pack_nonlinear/unpack_nonlinear the same way.
 *
 * Every function cites the reference lines it follows (paths within thu-ml/low-bit-optimizers).
 * Compile with -ffp-contract=off: each fused multiply-add the GPU compiler forms out of the
 * reference's expressions is written here as an explicit fmaf(), everything else must round
 * operation by operation.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define GROUP 128

/* Nearest-code rule of q_mapping (lpmm/cpp_extension/fused_adamw_kernel.cu:27-49) and of
 * quantize_bsearch<false> (lpmm/cpp_extension/quantization_kernel.cu:397-427): clamp at the
 * ends, upper-bound binary search, then the midpoint of the two neighbours decides; a tie goes to
 * the lower code.  A NaN fails every comparison, leaves lo = 0 and makes the reference return
 * -1, which its callers mask to 15 (fused_adamw_kernel.cu:157, quantization_kernel.cu:454). */
int lpmm_oracle_code(const float* qmap, int bits, float x) {
  int lo = 0, hi = 1 << bits;
  if (x <= qmap[lo]) return lo;
  if (qmap[hi - 1] <= x) return hi - 1;
  while (lo < hi) {
    int mi = (lo + hi) >> 1;
    if (qmap[mi] <= x) lo = mi + 1;
    else hi = mi;
  }
  if (lo == 0) return (1 << bits) - 1; /* NaN: (-1) & mask */
  float mid = (qmap[lo - 1] + qmap[lo]) * 0.5f;
  return (mid < x) ? lo : lo - 1;
}

/* pack_nonlinear_4bit_kernel<float,false> (quantization_kernel.cu:430-459) for bits = 4: two
 * codes per byte, element 2k in the low nibble.  `n` elements (the reference always passes a
 * multiple of 2048) give n/2 bytes; the caller provides the extra trailing byte of
 * pack_nonlinear_4bit_cuda's (total_bits + 8) / 8 allocation (quantization_kernel.cu:475-477),
 * which the reference leaves unwritten. */
void lpmm_oracle_pack4(const float* data, int64_t n, const float* qmap, uint8_t* packed) {
  int64_t nb = n / 2;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    int c0 = lpmm_oracle_code(qmap, 4, data[2 * b]) & 15;
    int c1 = lpmm_oracle_code(qmap, 4, data[2 * b + 1]) & 15;
    packed[b] = (uint8_t)(c0 | (c1 << 4));
  }
}

/* unpack_nonlinear_4bit_kernel<float> (quantization_kernel.cu:604-628): out[i] = qmap[nibble]. */
void lpmm_oracle_unpack4(const uint8_t* packed, int64_t n, const float* qmap, float* out) {
  int64_t nb = n / 2;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    out[2 * b] = qmap[packed[b] & 15];
    out[2 * b + 1] = qmap[(packed[b] >> 4) & 15];
  }
}

/* pack_nonlinear_8bit_kernel<float,false> (quantization_kernel.cu:515-537) for bits 5 ... 8: one code
 * per byte, the search's result cast to uint8_t without a mask, so a NaN (search result -1) is
 * stored as 255 whatever the width.  n bytes; the caller provides the trailing byte of the
 * (total_bits + 8) / 8 allocation (quantization_kernel.cu:552-554). */
void lpmm_oracle_pack8(const float* data, int64_t n, const float* qmap, int bits, uint8_t* packed) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float x = data[i];
    packed[i] = (x != x) ? (uint8_t)255 : (uint8_t)lpmm_oracle_code(qmap, bits, x);
  }
}

/* unpack_nonlinear_8bit_kernel<float> (quantization_kernel.cu:655-672): out[i] = qmap[byte].  A byte
 * beyond the map (the 255 of a NaN in a map of fewer than 8 bits), which the reference reads from
 * whatever follows its map, decodes to NaN here. */
void lpmm_oracle_unpack8(const uint8_t* packed, int64_t n, const float* qmap, int bits, float* out) {
  const int entries = 1 << bits;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = (packed[i] < entries) ? qmap[packed[i]] : NAN;
}

/* Bias corrections of the fused kernels (fused_adamw_kernel.cu:103-104, 72-73), with the host's
 * powf.  The device's powf may differ in the last bit, so tests that want bit-equal parameters
 * pass the device's values to the *_c variants below instead. */
void lpmm_oracle_bias_corrections(float beta1, float beta2, float step, float* out) {
  out[0] = 1.0f - powf(beta1, step);
  out[1] = sqrtf(1.0f - powf(beta2, step));
}

/* The moment and parameter updates of both fused kernels (fused_adamw_kernel.cu:121,124,126-128
 * and 69-77).  nvcc's default -fmad=true contracts
 *   beta1*m + (1-beta1)*g           into fma(beta1, m, (1-beta1)*g)
 *   beta2*v + (1-beta2)*g*g         into fma(beta2, v, ((1-beta2)*g)*g)
 *   m/denom + wd*p                  into fma(wd, p, m/denom)
 *   p - lr*update                   into fma(-lr, update, p)
 * `variant` bit 0 / bit 1 select the other possible contraction of the first / second line
 * (fma(1-beta1, g, beta1*m) / fma((1-beta2)*g, g, beta2*v)); variant 0 is what the reference
 * binary does (established against its outputs on a B200). */
static inline float upd_m(float b1, float omb1, float m0, float g, int variant) {
  if (variant & 1) return fmaf(omb1, g, b1 * m0);
  return fmaf(b1, m0, omb1 * g);
}
static inline float upd_v(float b2, float omb2, float v0, float g, int variant) {
  if (variant & 2) return fmaf(omb2 * g, g, b2 * v0);
  return fmaf(b2, v0, (omb2 * g) * g);
}
static inline float upd_p(float p, float m, float v, float lr, float wd, float eps, float c1, float c2s) {
  float denom = (sqrtf(v) / c2s + eps) * c1;
  float update = fmaf(wd, p, m / denom);
  return fmaf(-lr, update, p);
}

/* adamw4bit_cuda_kernel<float> (fused_adamw_kernel.cu:81-174) over a whole tensor, in place.
 * One iteration of the outer loop is one CTA of the reference: a group of 128 elements, its two
 * scales, 64 code bytes per moment.  Elements past numel take no part (:114, :132); an odd numel
 * leaves the last high nibble 0 (:153-165).  c1 = 1 - beta1^step, c2s = sqrt(1 - beta2^step). */
void lpmm_oracle_adamw4bit_c(float* p, const float* g, uint8_t* mq, uint8_t* vq, float* ms, float* vs,
                             const float* qmap_m, const float* qmap_v, float beta1, float beta2, float lr,
                             float wd, float eps, float c1, float c2s, int64_t numel, int variant) {
  const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
  const int64_t ngroups = (numel + GROUP - 1) / GROUP;
#pragma omp parallel for schedule(static)
  for (int64_t gi = 0; gi < ngroups; ++gi) {
    const int64_t e0 = gi * GROUP;
    const int cnt = (int)((numel - e0) < GROUP ? (numel - e0) : GROUP);
    float m[GROUP], v[GROUP];
    float am = 0.0f, av = 0.0f;
    const float sm = ms[gi], sv = vs[gi];
    for (int k = 0; k < cnt; ++k) {
      const int64_t e = e0 + k;
      const uint8_t mb = mq[e >> 1], vb = vq[e >> 1];
      const float m0 = qmap_m[(mb >> (4 * (e & 1))) & 15] * sm; /* :120, :134 */
      const float v0 = qmap_v[(vb >> (4 * (e & 1))) & 15] * sv; /* :123, :137 */
      m[k] = upd_m(beta1, omb1, m0, g[e], variant);
      v[k] = upd_v(beta2, omb2, v0, g[e], variant);
      p[e] = upd_p(p[e], m[k], v[k], lr, wd, eps, c1, c2s);
      am = fmaxf(am, fabsf(m[k])); /* :146-149 */
      av = fmaxf(av, v[k]);
    }
    for (int k = 0; k < cnt; k += 2) {
      const int64_t e = e0 + k;
      int c0 = lpmm_oracle_code(qmap_m, 4, m[k] / am) & 15; /* :155 */
      int d0 = lpmm_oracle_code(qmap_v, 4, v[k] / av) & 15; /* :156 */
      int c1n = 0, d1n = 0;
      if (k + 1 < cnt) {
        c1n = lpmm_oracle_code(qmap_m, 4, m[k + 1] / am) & 15; /* :161 */
        d1n = lpmm_oracle_code(qmap_v, 4, v[k + 1] / av) & 15; /* :162 */
      }
      mq[e >> 1] = (uint8_t)(c0 | (c1n << 4));
      vq[e >> 1] = (uint8_t)(d0 | (d1n << 4));
    }
    ms[gi] = am; /* :169-172 */
    vs[gi] = av;
  }
}

void lpmm_oracle_adamw4bit(float* p, const float* g, uint8_t* mq, uint8_t* vq, float* ms, float* vs,
                           const float* qmap_m, const float* qmap_v, float beta1, float beta2, float lr,
                           float wd, float eps, float step, int64_t numel, int variant) {
  float c[2];
  lpmm_oracle_bias_corrections(beta1, beta2, step, c);
  lpmm_oracle_adamw4bit_c(p, g, mq, vq, ms, vs, qmap_m, qmap_v, beta1, beta2, lr, wd, eps, c[0], c[1], numel,
                          variant);
}

/* adamw_cuda_kernel<float> (fused_adamw_kernel.cu:52-78): fp32 moments, same update. */
void lpmm_oracle_adamw_fp32_c(float* p, const float* g, float* m, float* v, float beta1, float beta2, float lr,
                              float wd, float eps, float c1, float c2s, int64_t numel, int variant) {
  const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
#pragma omp parallel for schedule(static)
  for (int64_t e = 0; e < numel; ++e) {
    m[e] = upd_m(beta1, omb1, m[e], g[e], variant);
    v[e] = upd_v(beta2, omb2, v[e], g[e], variant);
    p[e] = upd_p(p[e], m[e], v[e], lr, wd, eps, c1, c2s);
  }
}

void lpmm_oracle_adamw_fp32(float* p, const float* g, float* m, float* v, float beta1, float beta2, float lr,
                            float wd, float eps, float step, int64_t numel, int variant) {
  float c[2];
  lpmm_oracle_bias_corrections(beta1, beta2, step, c);
  lpmm_oracle_adamw_fp32_c(p, g, m, v, beta1, beta2, lr, wd, eps, c[0], c[1], numel, variant);
}

int lpmm_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void lpmm_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
