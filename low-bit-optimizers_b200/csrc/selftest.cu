// Self-test of the short arithmetic sequences the step kernels rely on (common.cuh): each one is compared, on the
// GPU, with the IEEE instruction or the reference's search it stands in for, over pseudo-random and adversarial
// operands of its stated domain.  Exported for the test-suite (lpmm_b200_test_exactness); not on any step's path.
#include "common.cuh"

namespace lpmm_b200 {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {  // splitmix64 finaliser: one independent word per index
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// A float with a uniformly random mantissa, the given sign bit and an exponent drawn uniformly from [elo, ehi]
// (unbiased); `bits` supplies the randomness.
__device__ __forceinline__ float rand_float(uint64_t bits, int elo, int ehi, bool neg) {
  const unsigned mant = (unsigned)bits & 0x7FFFFFu;
  const int e = elo + (int)((bits >> 23) % (uint64_t)(ehi - elo + 1));
  return __uint_as_float((neg ? 0x80000000u : 0u) | ((unsigned)(e + 127) << 23) | mant);
}

__device__ __forceinline__ float step_ulps(float x, int k) {  // k ulps up (k > 0) or down in magnitude order of the bits
  return __int_as_float(__float_as_int(x) + (x >= 0.0f ? k : -k));
}

// check 0: udiv(x, d, rcp_nr(d)) == x / d (as values) for 2^-60 <= d <= 2^60, |x| <= d, |x / d| >= 2^-18 or x == 0
// check 1: code from udiv + table / closed form == the reference's search on x / d, any |x| <= d (tiny quotients too);
//          `qmap` decides which: the linear map k/16 takes linear16_code, any other map the table
// check 2: sqrt_rn_fast(v) == sqrt(v)                 for v >= 2^-102 and v == 0
// check 3: div_rn_fast(m, d) == m / d                 for 2^-60 <= d <= 2^60, 2^-60 <= |m| <= 2^30 or m == 0
// check 4: lut_code / linear16_code == the search     for arbitrary bit patterns x (linear map: x in [-1e30, 1]; -inf left out)
__global__ void exactness_kernel(int check, const float* __restrict__ qmap_g, uint64_t seed, long long n,
                                 unsigned long long* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ QMapSmem S;
  LutEnt* lut = reinterpret_cast<LutEnt*>(dyn_smem);
  bool linear = false;
  if (qmap_g != nullptr) {
    lut_build(S, lut, qmap_g);
    linear = S.linear16 != 0;
  }
  unsigned long long bad = 0, tested = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const uint64_t a = mix64(seed + 3ull * (uint64_t)i), b = mix64(seed + 3ull * (uint64_t)i + 1), c = mix64(seed + 3ull * (uint64_t)i + 2);
    if (check == 0 || check == 1) {
      float d = rand_float(a, -60, 59, false);
      if ((c & 1023u) == 0) d = 0x1p60f;                    // the upper guard itself
      if ((c & 1023u) == 1) d = 0x1p-60f;                   // the lower guard itself
      float x;
      const unsigned mode = (unsigned)(c >> 10) & 3u;
      if (mode == 0 && qmap_g != nullptr) {                  // adversarial: x / d lands within 2 ulps of a midpoint
        const float mid = S.mids[(b >> 40) % 15u];
        x = __fmul_rn(step_ulps(mid, (int)((b >> 50) % 5u) - 2), d);
      } else if (mode == 1) {                                // quotient of any size down to 2^-18 (check 0) / 2^-40 (check 1)
        x = __fmul_rn(rand_float(b, check == 0 ? -18 : -40, -1, (b >> 63) != 0), d);
      } else if (mode == 2) {                                // |x| == d, x == 0, x tiny
        const unsigned k = (unsigned)(b >> 20) % 3u;
        x = k == 0 ? d : (k == 1 ? 0.0f : rand_float(b, -126, -100, false));
        if ((b >> 63) != 0) x = -x;
      } else {                                               // same binade neighbourhood: mantissa pairs
        x = __fmul_rn(rand_float(b, -3, -1, (b >> 63) != 0), d);
      }
      if (!(fabsf(x) <= d)) continue;
      const float q = udiv(x, d, rcp_nr(d));
      const float ref = __fdiv_rn(x, d);
      ++tested;
      if (check == 0) {
        if (x != 0.0f && fabsf(ref) < 0x1p-18f) { --tested; continue; }
        if (!(q == ref)) ++bad;  // as values: a zero quotient may come out as +0 where IEEE gives -0 (same code either way)
      } else {
        const int want = bsearch_code(S.qmap, ref);
        const int got = linear ? (int)linear16_code(q) : lut_code(lut, q);
        if (want != got) ++bad;
      }
    } else if (check == 2) {
      float v = rand_float(a, -102, 127, false);
      if ((c & 255u) == 0) v = 0.0f;
      if ((c & 255u) == 1) v = 0x1p-102f;
      if ((c & 255u) == 2) v = __uint_as_float(0x7F7FFFFFu);
      if ((c & 255u) == 3) {                                 // perfect squares and their neighbours
        const float r = rand_float(b, -50, 60, false);
        v = step_ulps(__fmul_rn(r, r), (int)((b >> 50) % 3u) - 1);
      }
      ++tested;
      if (__float_as_uint(sqrt_rn_fast(v)) != __float_as_uint(__fsqrt_rn(v))) ++bad;
    } else if (check == 3) {
      float d = rand_float(a, -60, 59, false);
      if ((c & 1023u) == 0) d = 0x1p60f;
      if ((c & 1023u) == 1) d = 0x1p-60f;
      float m = rand_float(b, -60, 29, (b >> 63) != 0);
      if ((c & 1023u) == 2) m = 0.0f;
      if ((c & 1023u) == 3) m = 0x1p30f;
      if ((c & 1023u) == 4) m = -0x1p-60f;
      ++tested;
      if (__float_as_uint(div_rn_fast(m, d)) != __float_as_uint(__fdiv_rn(m, d))) ++bad;
    } else if (check == 4) {
      float x = __uint_as_float((unsigned)a);
      if ((c & 3u) == 0) x = step_ulps(S.mids[(b >> 40) % 15u], (int)((b >> 50) % 5u) - 2);  // around every midpoint
      if ((c & 3u) == 1) x = S.qmap[(b >> 40) % 16u];                                        // the map values themselves
      if (x == __int_as_float(0xff800000)) continue;         // -inf: documented exception of the table
      if (linear && !(x <= 1.0f && x >= -1e30f)) continue;   // closed form: stated domain (NaN is the caller's case)
      ++tested;
      const int want = bsearch_code(S.qmap, x);
      const int got = linear ? (int)linear16_code(x) : lut_code(lut, x);
      if (want != got) ++bad;
    }
  }
  for (int o = 16; o; o >>= 1) {
    bad += __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    tested += __shfl_xor_sync(0xFFFFFFFFu, tested, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out, bad);
    atomicAdd(out + 1, tested);
  }
}

}  // namespace lpmm_b200

using namespace lpmm_b200;

extern "C" int lpmm_b200_test_exactness(int check, const float* qmap, uint64_t seed, int64_t n_samples,
                                        unsigned long long* out, void* stream) {
  if (check < 0 || check > 4) return LPMM_B200_ERR_BAD_KIND;
  if (!out || ((check == 1 || check == 4) && !qmap)) return LPMM_B200_ERR_NULL_POINTER;
  if (n_samples < 0) return LPMM_B200_ERR_BAD_SIZE;
  const size_t smem = LUT_ENTRIES * sizeof(LutEnt);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    LPMM_CUDA_TRY(cudaFuncSetAttribute(exactness_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev] = true;
  }
  LPMM_CUDA_TRY(cudaMemsetAsync(out, 0, 2 * sizeof(unsigned long long), (cudaStream_t)stream));
  exactness_kernel<<<num_sms() * 4, 256, smem, (cudaStream_t)stream>>>(check, qmap, seed, n_samples, out);
  LPMM_CUDA_TRY(cudaGetLastError());
  return LPMM_B200_OK;
}
