/*
 * lpmm_b200.h -- C ABI of the B200 (sm_100a) implementation of lpmm's 4-bit optimizer-step path.
 *
 * Every entry point takes plain device pointers, element counts and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL means the legacy default stream) and returns an int
 * status: 0 on success, a negative LPMM_B200_ERR_* otherwise.  Argument errors are detected on
 * the host before anything is launched.  No entry point allocates or frees device memory unless
 * its comment says otherwise, none synchronises the device, and all launches are asynchronous on
 * the given stream.  The caller owns every buffer.
 *
 * Each declaration cites the interface of the reference (thu-ml/low-bit-optimizers, paths
 * relative to that project) that it stands in for.
 *
 * Data formats shared by all entry points
 *   - 4-bit codes: two per byte, element 2k in bits 0-3 and element 2k+1 in bits 4-7 of byte k
 *     (lpmm/cpp_extension/fused_adamw_kernel.cu:119,133,157,163; quantization_kernel.cu:454,623).
 *   - quantization map ("qmap"): 16 ascending fp32 values in device memory.
 *   - nearest-code rule: code(x) = number of midpoints (q[i]+q[i+1])*0.5f that are < x, ties to
 *     the lower code, NaN -> 15 (fused_adamw_kernel.cu:27-49, quantization_kernel.cu:397-427).
 *   - group scale: one fp32 absmax per 128 consecutive elements of the flattened tensor.
 */
#ifndef LPMM_B200_H
#define LPMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LPMM_B200_OK 0
#define LPMM_B200_ERR_NULL_POINTER (-1)   /* a required pointer is NULL                        */
#define LPMM_B200_ERR_BAD_SIZE (-2)       /* negative / inconsistent element count or range    */
#define LPMM_B200_ERR_BAD_KIND (-3)       /* unknown tensor kind / option value                */
#define LPMM_B200_ERR_CUDA (-4)           /* a CUDA runtime call failed, see last_cuda_error   */
#define LPMM_B200_ERR_UNSUPPORTED (-5)    /* valid in the reference, not built here            */
#define LPMM_B200_ERR_TOO_LARGE (-6)      /* size beyond a documented static limit             */

#define LPMM_B200_GROUP 128               /* elements per scale group of the fused step        */
#define LPMM_B200_PACK_GROUP 2048         /* elements per row of the pack/unpack layout        */

/* Tensor kinds of the multi-tensor step. */
#define LPMM_B200_KIND_Q4 0               /* 4-bit m and v, group-128 absmax scales            */
#define LPMM_B200_KIND_FP32 1             /* fp32 m and v (the numel <= threshold fallback)    */

/* element type of p and g in lpmm_b200_adamw4bit_multi_tensor_16bit */
#define LPMM_B200_DTYPE_BF16 1
#define LPMM_B200_DTYPE_FP16 2

/* One parameter tensor of a multi-tensor step.  All pointers are device pointers into
 * contiguous arrays.  kind Q4: m, v are int8[(numel+1)/2] packed codes, m_scale, v_scale are
 * float[(numel+127)/128].  kind FP32: m, v are float[numel], the scale pointers are ignored. */
typedef struct lpmm_b200_tensor {
  float* p;
  const float* g;
  void* m;
  void* v;
  float* m_scale;
  float* v_scale;
  int64_t numel;
  int32_t kind;
  int32_t reserved;
} lpmm_b200_tensor;

/* AdamW hyper-parameters, as the C floats the reference's bindings receive
 * (lpmm/cpp_extension/fused_adamw.cc:44-58). */
typedef struct lpmm_b200_hyper {
  float beta1;
  float beta2;
  float lr;
  float weight_decay;
  float eps;
  float step;
} lpmm_b200_hyper;

/* Human-readable text for a status code. */
const char* lpmm_b200_strerror(int status);
/* Text of the CUDA error behind the calling thread's last LPMM_B200_ERR_CUDA ("" if none). */
const char* lpmm_b200_last_cuda_error(void);
/* ABI version of this library (bumped on any signature change). */
int lpmm_b200_abi_version(void);

/* Fused 4-bit AdamW step of one tensor, in place.
 * Replaces fused_adamw.adamw4bit_single_tensor (lpmm/cpp_extension/fused_adamw.cc:44-78 ->
 * fused_adamw_kernel.cu:81-174, 208-243).  Unlike the reference (fused_adamw.cc:68-71) an odd
 * numel is accepted; the unused high nibble of the last byte is written as 0. */
int lpmm_b200_adamw4bit_single_tensor(float* p, const float* g, int8_t* exp_avg, int8_t* exp_avg_sq,
                                      float* exp_avg_scale, float* exp_avg_sq_scale,
                                      const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                      float beta1, float beta2, float lr, float weight_decay, float eps,
                                      float step, int64_t numel, void* stream);

/* Fused fp32-state AdamW step of one tensor, in place.
 * Replaces fused_adamw.adamw_single_tensor (lpmm/cpp_extension/fused_adamw.cc:15-41 ->
 * fused_adamw_kernel.cu:52-78, 177-205). */
int lpmm_b200_adamw_single_tensor(float* p, const float* g, float* exp_avg, float* exp_avg_sq, float beta1,
                                  float beta2, float lr, float weight_decay, float eps, float step,
                                  int64_t numel, void* stream);

/* Fused step over a whole parameter list in one launch per <= 400 tensors.
 * Replaces the per-tensor Python loop of _fused_adamw4bit (lpmm/optim/adamw.py:463-561) and the
 * per-tensor launches behind it.  `tensors` is a HOST array of n descriptors (copied into the
 * launch parameters; nothing is read from it after return).  The flattened list defines a global
 * index space of 128-element groups (tensor t contributes ceil(numel_t/128) groups, in list
 * order); only groups in [group_begin, group_end) are updated, which is how a ZeRO-1 rank
 * updates its shard.  Pass group_begin = 0, group_end = -1 for the whole list. */
int lpmm_b200_adamw4bit_multi_tensor(const lpmm_b200_tensor* tensors, int n_tensors, const float* exp_avg_qmap,
                                     const float* exp_avg_sq_qmap, lpmm_b200_hyper hyper, int64_t group_begin,
                                     int64_t group_end, void* stream);

/* Options of the fused step (the ..._flags entry points; 0 = the behaviour of the plain ones).
 *
 * LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE: moments, group maxima and packed codes are computed exactly as without
 * the flag (they never depend on the parameter: fused_adamw_kernel.cu:120-124,146-162), but the parameter
 * update p -= lr * (m / ((sqrt(v)/c2s + eps) * c1) + wd * p) (fused_adamw_kernel.cu:126-128) uses the GPU's
 * approximate square root and reciprocal (2^-23 relative each) with lr, c1 and c2s folded into constants,
 * instead of correctly rounded operations.  A step lr*m/d then differs from the reference's by less than 1e-6
 * of its own size, a parameter by a few 1e-10 per step at lr = 1e-3.  Full, aligned 4-bit groups take it;
 * ragged groups, fp32-state tensors and hyper-parameters outside lr in [2^-60, 2^30] keep the exact update. */
#define LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE 1u
int lpmm_b200_adamw4bit_multi_tensor_flags(const lpmm_b200_tensor* tensors, int n_tensors, const float* exp_avg_qmap,
                                           const float* exp_avg_sq_qmap, lpmm_b200_hyper hyper, int64_t group_begin,
                                           int64_t group_end, uint32_t flags, void* stream);

/* The fused step for 16-bit parameters and gradients: `p` and `g` of every tensor point to bf16 or fp16
 * arrays (dtype = LPMM_B200_DTYPE_*; the struct's float* is reinterpreted), everything else is as in
 * lpmm_b200_adamw4bit_multi_tensor: 4-bit codes, fp32 scales, fp32 moments for kind FP32.
 * Parameters and gradients are widened to fp32 on load, the step is the fp32 step to the bit, the new
 * parameter is rounded to nearest-even on store.  The reference instantiates its kernel for half
 * (fused_adamw_kernel.cu:188,222) but cannot reach it: the launcher wants half scale tensors where
 * lpmm/optim/adamw.py:515-521 allocates fp32 ones, and bf16 is not dispatched. */
int lpmm_b200_adamw4bit_multi_tensor_16bit(const lpmm_b200_tensor* tensors, int n_tensors, int dtype,
                                           const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                           lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end, void* stream);

int lpmm_b200_adamw4bit_multi_tensor_16bit_flags(const lpmm_b200_tensor* tensors, int n_tensors, int dtype,
                                                 const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                 lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                 uint32_t flags, void* stream);

/* The same step for a ZeRO-1 rank, with the all-gather of the updated parameters folded into the
 * kernel.  It has no counterpart in the reference (which has no distributed step).
 * Every parameter this call updates is stored at its own address AND at that address plus each of
 * the n_peers (<= 7) byte offsets, which must lead to the same element of the other ranks' copies
 * of the parameter buffer in peer-mapped memory (offsets multiples of 32).  The transfer over
 * NVLink thus overlaps the update group by group.  The caller orders the ranks afterwards (any
 * stream-ordered barrier across the ranks) before parameters are read. */
int lpmm_b200_adamw4bit_multi_tensor_peers(const lpmm_b200_tensor* tensors, int n_tensors, const float* exp_avg_qmap,
                                           const float* exp_avg_sq_qmap, lpmm_b200_hyper hyper, int64_t group_begin,
                                           int64_t group_end, const int64_t* peer_byte_offsets, int n_peers,
                                           void* stream);

int lpmm_b200_adamw4bit_multi_tensor_peers_flags(const lpmm_b200_tensor* tensors, int n_tensors,
                                                 const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                 lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                 const int64_t* peer_byte_offsets, int n_peers, uint32_t flags,
                                                 void* stream);

/* The ZeRO-1 step with the all-gather folded in, for 16-bit parameters and gradients (dtype = LPMM_B200_DTYPE_*):
 * lpmm_b200_adamw4bit_multi_tensor_16bit_flags whose every updated parameter is also stored at its address plus each
 * of the n_peers (<= 7) byte offsets (multiples of 16) -- half the NVLink bytes of the fp32 form.  No counterpart in
 * the reference.  Both quantization maps are required whenever n_peers > 0. */
int lpmm_b200_adamw4bit_multi_tensor_16bit_peers(const lpmm_b200_tensor* tensors, int n_tensors, int dtype,
                                                 const float* exp_avg_qmap, const float* exp_avg_sq_qmap,
                                                 lpmm_b200_hyper hyper, int64_t group_begin, int64_t group_end,
                                                 const int64_t* peer_byte_offsets, int n_peers, uint32_t flags,
                                                 void* stream);

/* The whole ZeRO-1 step in one kernel: additionally to the above, the gradient of every element of
 * this rank's range is the sum, in the order given, of the values found at the n_grads (<= 8) byte
 * offsets from its address in this GPU's gradient buffer (tensors[i].g; offset 0 is this GPU's own
 * copy, the others lead to the same element of the peers' gradient buffers in peer-mapped memory),
 * multiplied by grad_scale (1/world for a mean).  Each rank thus reads only the gradients of its own
 * groups from every peer over NVLink (the reduce-scatter) while it stores its updated parameters into
 * the peers' parameter buffers (the all-gather), both inside the update kernel.  All ranks must have
 * finished writing their gradients before any rank's call starts reading them, and must not overwrite
 * them before every call has finished (order with a barrier on the stream).  Offsets must be multiples
 * of 32.  n_grads == 0: gradients are read from tensors[i].g alone, as in the entry point above. */
int lpmm_b200_adamw4bit_multi_tensor_zero1(const lpmm_b200_tensor* tensors, int n_tensors, const float* exp_avg_qmap,
                                           const float* exp_avg_sq_qmap, lpmm_b200_hyper hyper, int64_t group_begin,
                                           int64_t group_end, const int64_t* peer_byte_offsets, int n_peers,
                                           const int64_t* grad_byte_offsets, int n_grads, float grad_scale,
                                           void* stream);

/* Number of 128-element groups of a tensor list (the size of the index space above), or a
 * negative status.  Host-only arithmetic. */
int64_t lpmm_b200_count_groups(const lpmm_b200_tensor* tensors, int n_tensors);

/* The two bias-correction terms exactly as the fused step computes them on the device:
 * out[0] = 1 - powf(beta1, step), out[1] = sqrtf(1 - powf(beta2, step))
 * (fused_adamw_kernel.cu:103-104).  out is a device pointer to 2 floats.  For tests that feed a
 * CPU model the device's own powf result. */
int lpmm_b200_bias_corrections(float beta1, float beta2, float step, float* out, void* stream);

/* ------------------------------------------------------------------------------------------- */
/* Standalone quantize / dequantize (the kernels behind lpmm.functional)                        */
/* ------------------------------------------------------------------------------------------- */

/* Bytes of the packed-code tensor the reference allocates for n_scaled normalised values:
 * rows of 2048 values, two codes per byte, plus one trailing byte
 * (lpmm/functional.py:362; lpmm/cpp_extension/quantization_kernel.cu:475-477). */
int64_t lpmm_b200_packed_len(int64_t n_scaled);

/* Replaces quantization.pack_nonlinear(data[G, S], qmap, 4, False)
 * (lpmm/cpp_extension/quantization.cc:54-63 -> quantization_kernel.cu:430-513).  n = G*S values,
 * n even; packed holds n/2 + 1 bytes, the last one (never written by the reference) is set to 0.
 * This is the 4-bit round-to-nearest form; lpmm_b200_pack_nonlinear takes 4 to 8 bits and
 * lpmm_b200_pack_nonlinear_sr rounds stochastically. */
int lpmm_b200_pack_nonlinear4(const float* data, int64_t n, const float* qmap, int8_t* packed, void* stream);

/* Replaces quantization.unpack_nonlinear(packed, qmap, 4, G, S)
 * (lpmm/cpp_extension/quantization.cc:65-76 -> quantization_kernel.cu:604-653): out[i] = qmap[code_i]
 * for i < n = G*S, n even. */
int lpmm_b200_unpack_nonlinear4(const int8_t* packed, const float* qmap, int64_t n, float* out, void* stream);

/* Group-128 quantization of a flattened tensor: what vectorwise_quant does for scale_type
 * 'group' with gp_sz 128, and for 'rank1' on 1-D tensors (lpmm/functional.py:26-59, 184-197,
 * 359-369).  max1 receives ceil(numel/128) group maxima of |x|; codes receives
 * lpmm_b200_packed_len(ceil(numel/128)*128) bytes (zero padding quantized as the reference's
 * padded zeros are). */
int lpmm_b200_quant_group4(const float* x, int64_t numel, const float* qmap, int8_t* codes, float* max1, void* stream);

/* Inverse (vectorwise_dequant, lpmm/functional.py:62-151, group branch): out[i] = qmap[code_i] *
 * max1[i / 128], i < numel. */
int lpmm_b200_dequant_group4(const int8_t* codes, const float* qmap, const float* max1, int64_t numel, float* out,
                             void* stream);

/* Per-axis maxima of |x| of a contiguous ndim-D tensor (ndim <= 8): max_dims[i] points to
 * shape[i] floats and receives the maximum over all other axes (get_sm3_statistics,
 * lpmm/functional.py:512-531).  shape and max_dims are HOST arrays. */
int lpmm_b200_axis_absmax(const float* x, const int64_t* shape, int ndim, float* const* max_dims, void* stream);

/* Rank-1 quantization (vectorwise_quant, scale_type 'rank1', ndim >= 2; functional.py:190-203):
 * fills max_dims as above, then codes = rule(x / min_i max_dims[i][idx_i]) in the packed layout
 * of lpmm_b200_packed_len(numel) bytes. */
int lpmm_b200_quant_rank1_4(const float* x, const int64_t* shape, int ndim, const float* qmap,
                            float* const* max_dims, int8_t* codes, void* stream);

/* Inverse (vectorwise_dequant, rank1 branch, functional.py:97-106). */
int lpmm_b200_dequant_rank1_4(const int8_t* codes, const float* qmap, const float* const* max_dims,
                              const int64_t* shape, int ndim, float* out, void* stream);

/* The same six operations for every code width and group size of the reference's configuration
 * files (lpmm/configs/default_{5,6,7,8}b.yml, 1st_moment_group_{256,...,4096}.yml):
 *   bits        4 ... 8.  4: two codes per byte as above.  5 ... 8: one code per byte, the map has
 *               2^bits entries (pack_nonlinear_8bit_kernel / unpack_nonlinear_8bit_kernel,
 *               quantization_kernel.cu:515-537, 655-672); a NaN is stored as 255 like there.
 *               1 ... 3 bits return LPMM_B200_ERR_UNSUPPORTED.
 *   group_size  128, 256, ..., 4096 (a power of two): x is zero-padded to a multiple of it before
 *               normalisation, max1 holds ceil(numel/group_size) maxima
 *               (group_tensor, lpmm/functional.py:359-369).
 * Packed length: rows of 2048 codes, (bits == 4 ? 1/2 : 1) byte per code, plus one trailing byte.
 * The ...4 entry points above are these with bits = 4 and group_size = 128. */
int64_t lpmm_b200_packed_len_bits(int64_t n_scaled, int bits);
int lpmm_b200_pack_nonlinear(const float* data, int64_t n, const float* qmap, int bits, int8_t* packed, void* stream);
int lpmm_b200_unpack_nonlinear(const int8_t* packed, const float* qmap, int bits, int64_t n, float* out,
                               void* stream);
int lpmm_b200_quant_group(const float* x, int64_t numel, const float* qmap, int bits, int64_t group_size,
                          int8_t* codes, float* max1, void* stream);
int lpmm_b200_dequant_group(const int8_t* codes, const float* qmap, int bits, int64_t group_size, const float* max1,
                            int64_t numel, float* out, void* stream);
int lpmm_b200_quant_rank1(const float* x, const int64_t* shape, int ndim, const float* qmap, int bits,
                          float* const* max_dims, int8_t* codes, void* stream);
int lpmm_b200_dequant_rank1(const int8_t* codes, const float* qmap, int bits, const float* const* max_dims,
                            const int64_t* shape, int ndim, float* out, void* stream);

/* Stochastic rounding (round_type 'real-sr': pack_nonlinear(..., stochastic=True),
 * quantization_kernel.cu:397-427, 431-459, 517-537).  Between the two neighbouring map values the
 * upper one is taken with probability (x - lower) / (upper - lower).  The uniforms are those of the
 * reference: curand Philox4_32_10, one subsequence per reference thread (8 consecutive elements of the
 * padded layout for 4-bit codes, 4 for wider ones), started at (seed, offset) -- the pair the reference
 * takes from torch's default CUDA generator with philox_engine_inputs(16384) (4-bit) or (8192) (wider)
 * on every pack_nonlinear call, stochastic or not.  The caller reads and advances the generator.  With
 * the same (seed, offset) the codes equal the reference's bit for bit; a NaN gives the last code (the
 * reference reads before the start of its map there).  n must be a multiple of 8 in the pack call. */
int lpmm_b200_pack_nonlinear_sr(const float* data, int64_t n, const float* qmap, int bits, int8_t* packed,
                                uint64_t seed, uint64_t offset, void* stream);
int lpmm_b200_quant_group_sr(const float* x, int64_t numel, const float* qmap, int bits, int64_t group_size,
                             int8_t* codes, float* max1, uint64_t seed, uint64_t offset, void* stream);
int lpmm_b200_quant_rank1_sr(const float* x, const int64_t* shape, int ndim, const float* qmap, int bits,
                             float* const* max_dims, int8_t* codes, uint64_t seed, uint64_t offset, void* stream);

/* ------------------------------------------------------------------------------------------- */
/* One-launch-per-tensor steps with the arithmetic of the reference's non-fused Python path     */
/* ------------------------------------------------------------------------------------------- */

#define LPMM_B200_STATE_FP32 0    /* float[numel]                                               */
#define LPMM_B200_STATE_GROUP4 1  /* codes + group scales, vectorwise_quant layout (4 bits, groups of 128 unless the bits / group fields say otherwise) */
#define LPMM_B200_STATE_RANK1_4 2 /* codes + per-axis maxima (ndim >= 2)                        */
#define LPMM_B200_STATE_FACTORED 3/* fp32 row / column accumulators (ndim >= 2), no codes       */

typedef struct lpmm_b200_step_tensor {
  float* p;
  const float* g;
  int64_t numel;
  int32_t ndim;                 /* <= 8; needed for RANK1_4 and FACTORED, else may be 1        */
  int32_t first;                /* nonzero: the moments are not initialised yet, read as zero   */
  int64_t shape[8];
  int32_t m_mode;               /* FP32 or GROUP4                                               */
  int32_t v_mode;               /* any LPMM_B200_STATE_*                                        */
  void* m;                      /* float[numel] or int8[packed_len]                             */
  float* m_max1;                /* GROUP4: float[ceil(numel/128)]                               */
  void* v;                      /* float[numel] or int8[packed_len]; unused when FACTORED       */
  float* v_max1;                /* GROUP4: float[ceil(numel/128)]                               */
  const float* v_max_dims_old[8]; /* RANK1_4: maxima the current codes were normalised with     */
  float* v_max_dims_new[8];       /* RANK1_4: receives the maxima of the updated second moment  */
  float* row;                   /* FACTORED: float[prod(shape[:-1])]                            */
  float* col;                   /* FACTORED: float[prod(shape[:-2]) * shape[-1]]                */
  int32_t m_bits, v_bits;       /* code width of a quantized state, 4 ... 8; 0 means 4            */
  int32_t m_group, v_group;     /* group size of a GROUP4 state: 128 ... 4096, power of two; 0 = 128 */
} lpmm_b200_step_tensor;

/* One AdamW step of one tensor with the arithmetic and state layout of the reference's
 * non-fused path: _single_tensor_adamw4bit (lpmm/optim/adamw.py:332-436) for v_mode FP32 /
 * GROUP4 / RANK1_4 and _single_quantized_factored_update (adamw.py:579-627, after the decay at
 * :369/:478) for FACTORED.  Hyper-parameters arrive as the Python doubles the reference computes
 * its scalar constants from.  FACTORED needs `scratch` (device memory, at least
 * lpmm_b200_factored_scratch_bytes() bytes, contents irrelevant before and after); other modes
 * ignore it. */
int lpmm_b200_adamw4bit_unfused_step(const lpmm_b200_step_tensor* t, const float* qmap_m, const float* qmap_v,
                                     double beta1, double beta2, double lr, double weight_decay, double eps,
                                     double step, void* scratch, int64_t scratch_bytes, void* stream);
int64_t lpmm_b200_factored_scratch_bytes(const int64_t* shape, int ndim);

/* The non-fused step of a whole list in ONE launch, for tensors whose two moments are both 4-bit with
 * group-128 scales (the reference's configuration when no qconfig is given; kind LPMM_B200_KIND_Q4: m, v
 * = packed codes in the vectorwise_quant layout of lpmm_b200_packed_len(ceil(numel/128)*128) bytes,
 * m_scale, v_scale = float[ceil(numel/128)]) or both fp32 (LPMM_B200_KIND_FP32).  Arithmetic and layout
 * are those of lpmm_b200_adamw4bit_unfused_step with GROUP4 / GROUP4 or FP32 / FP32 states, so a tensor
 * may be stepped by either; the states must already be initialised (a tensor's first step belongs to
 * lpmm_b200_adamw4bit_unfused_step, which also writes the layout's padding).  All tensors share `step`.
 * [group_begin, group_end) selects a range of the list's 128-element group sequence (group_end < 0: all). */
int lpmm_b200_adamw4bit_unfused_multi_tensor(const lpmm_b200_tensor* tensors, int n_tensors, const float* qmap_m,
                                             const float* qmap_v, double beta1, double beta2, double lr,
                                             double weight_decay, double eps, double step, int64_t group_begin,
                                             int64_t group_end, void* stream);

/* The same step for n tensors in one call: tensors[i] is stepped with steps[i] (the reference keeps
 * one step counter per parameter), all with the same maps and hyper-parameters, in order, on
 * `stream`; `scratch` must serve the largest FACTORED tensor of the list.  It replaces the reference's
 * per-parameter Python loop (lpmm/optim/adamw.py:332-436); results are those of n single calls. The
 * first non-zero status ends the call (earlier tensors have been stepped).
 * Tensors that lpmm_b200_adamw4bit_unfused_multi_tensor covers and that share a step count are updated
 * by one launch of it; 2-D RANK1_4 tensors (4-bit codes, group-128 first moment, row length a multiple
 * of 8, 16-byte aligned) that share a step count are stepped together in three or four launches (zero,
 * statistics, update; matrices whose rows are multiples of 128 elements take an update kernel of their own),
 * their descriptors carried in the launch parameters.  2-D FACTORED tensors (fp32 or 4-bit group-128 first
 * moment, same shape conditions) that share a step count are likewise stepped together in four or five
 * launches, their partial sums taken from `scratch` (lpmm_b200_unfused_step_many_scratch_bytes gives a size
 * that serves everything; without enough scratch they are stepped one by one).  Nothing is uploaded, so both
 * list-wide paths also run while `stream` is being captured.  `scratch` should be 256-byte aligned.  The launch
 * chains of the other tensors are spread over four streams owned by the library (created on
 * the first such call on a device, never destroyed); they start after everything already enqueued on
 * `stream`, and `stream` waits for them before the call returns, so the caller's ordering is that of
 * a call that used `stream` alone.  While `stream` is being captured the library's streams are not used.
 * FACTORED tensors run concurrently only if `scratch_bytes` / 4 (rounded down to 256) covers the
 * largest lpmm_b200_factored_scratch_bytes() of the list; otherwise they run one after the other. */
/* Scratch size with which lpmm_b200_adamw4bit_unfused_step_many takes all its list-wide paths for
 * these tensors (shapes, modes and pointers alignment are read; `first` is ignored). */
int64_t lpmm_b200_unfused_step_many_scratch_bytes(const lpmm_b200_step_tensor* const* tensors, int n);
int lpmm_b200_adamw4bit_unfused_step_many(const lpmm_b200_step_tensor* const* tensors, int n, const float* qmap_m,
                                          const float* qmap_v, double beta1, double beta2, double lr,
                                          double weight_decay, double eps, const double* steps, void* scratch,
                                          int64_t scratch_bytes, void* stream);
/* The same with `flags` (0, or LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE).  With the flag, the list-wide kernels (the
 * shared launch of the plain tensors, and the update kernels of the rank-1 and factored matrices whose rows are
 * multiples of 128 elements) compute the new parameter with the GPU's approximate square root and reciprocal;
 * moments, maxima, row / column statistics and codes are unchanged, tensors stepped on their own stay exact.  Any
 * other bit: LPMM_B200_ERR_BAD_KIND.  No counterpart in the reference. */
int lpmm_b200_adamw4bit_unfused_step_many_flags(const lpmm_b200_step_tensor* const* tensors, int n,
                                                const float* qmap_m, const float* qmap_v, double beta1, double beta2,
                                                double lr, double weight_decay, double eps, const double* steps,
                                                void* scratch, int64_t scratch_bytes, void* stream, uint32_t flags);

/* The fused step on the non-fused state layout: the arithmetic of the reference's fused kernel
 * (lpmm/cpp_extension/fused_adamw_kernel.cu:103-128: float hyper-parameters, bias corrections by the
 * device's powf, m = fma(b1, m0, (1-b1)g), v = fma(b2, v0, ((1-b2)g)g), d = (sqrt(v)/c2s + eps)c1,
 * p = fma(-lr, fma(wd, p, m/d), p)) on the states of lpmm_b200_adamw4bit_unfused_step, which the
 * fused kernel itself cannot hold: above all a RANK1_4 second moment (per-axis maxima by the two-pass
 * grid reduction).  The reference has no such step: with a rank-1 configuration its fused=True warns
 * and uses group scales (lpmm/optim/adamw.py:503-506).  4-bit codes only; the moments are both FP32,
 * both GROUP4, or GROUP4 + RANK1_4; FACTORED is not covered (LPMM_B200_ERR_UNSUPPORTED).  States that
 * are all zero (zero maxima) step like first != 0.  The _many form follows
 * lpmm_b200_adamw4bit_unfused_step_many: eligible 2-D RANK1_4 tensors that share a step count take
 * three launches together, the others a launch chain each on the library's streams. */
int lpmm_b200_adamw4bit_fused_arith_step(const lpmm_b200_step_tensor* t, const float* qmap_m, const float* qmap_v,
                                         double beta1, double beta2, double lr, double weight_decay, double eps,
                                         double step, void* stream);
int lpmm_b200_adamw4bit_fused_arith_step_many(const lpmm_b200_step_tensor* const* tensors, int n, const float* qmap_m,
                                              const float* qmap_v, double beta1, double beta2, double lr,
                                              double weight_decay, double eps, const double* steps, void* scratch,
                                              int64_t scratch_bytes, void* stream);
/* The same with `flags`, as lpmm_b200_adamw4bit_unfused_step_many_flags (the rank-1 update kernel of matrices whose
 * rows are multiples of 128 elements takes the tolerance mode; learning rate in [2^-60, 2^30] as for the fused step,
 * otherwise the flag is ignored). */
int lpmm_b200_adamw4bit_fused_arith_step_many_flags(const lpmm_b200_step_tensor* const* tensors, int n,
                                                    const float* qmap_m, const float* qmap_v, double beta1,
                                                    double beta2, double lr, double weight_decay, double eps,
                                                    const double* steps, void* scratch, int64_t scratch_bytes,
                                                    void* stream, uint32_t flags);

/* fp32 -> bf16 / fp16 copy of `numel` elements, round to nearest even (dtype = LPMM_B200_DTYPE_*): the 16-bit replicas
 * of fp32 master parameters in a sharded step (a rank keeps fp32 parameters for its own range and publishes them at
 * half the bytes).  src 4-byte, dst 2-byte aligned; 256-bit loads / 128-bit stores where both are 32- / 16-byte aligned
 * at the same element.  No counterpart in the reference (torch's `.to(dtype)` gives the same values). */
int lpmm_b200_narrow_fp32(const float* src, void* dst, int64_t numel, int dtype, void* stream);

/* One momentum-SGD step of one tensor with the arithmetic of _single_tensor_sgd4bit
 * (lpmm/optim/sgd.py:133-187).  buf_mode FP32 or GROUP4; first != 0: the buffer is created from
 * the (decayed) gradient.  momentum == 0 ignores the buffer. */
int lpmm_b200_sgd4bit_step(float* p, const float* g, int64_t numel, void* buf, float* buf_max1, int buf_mode,
                           int first, const float* qmap, double weight_decay, double momentum, double lr,
                           double dampening, int nesterov, int maximize, void* stream);
/* The same with the buffer's code width (4 ... 8) and group size (128 ... 4096) given. */
int lpmm_b200_sgd_lowbit_step(float* p, const float* g, int64_t numel, void* buf, float* buf_max1, int buf_mode,
                              int bits, int64_t group_size, int first, const float* qmap, double weight_decay,
                              double momentum, double lr, double dampening, int nesterov, int maximize,
                              void* stream);

/* Momentum SGD of a whole parameter list in one launch (the reference has no fused SGD: sgd.py:31-32
 * raises for fused=True).  Arithmetic and state layout are those of lpmm_b200_sgd4bit_step, i.e. of
 * _single_tensor_sgd4bit (lpmm/optim/sgd.py:133-187), so a buffer may be stepped by either entry
 * point.  Per tensor: p, g, m = the momentum buffer (KIND_Q4: packed 4-bit codes in the
 * vectorwise_quant layout of lpmm_b200_packed_len(ceil(numel/128)*128) bytes, m_scale = float[ceil(
 * numel/128)]; KIND_FP32: float[numel]); v and v_scale are ignored.  Buffers must already be
 * initialised (the first step of a tensor, buffer = clone of the decayed gradient, belongs to
 * lpmm_b200_sgd4bit_step, which also writes the layout's padding).  momentum must be non-zero.
 * [group_begin, group_end) selects a range of the list's global 128-element group sequence
 * (group_end < 0: all), as in lpmm_b200_adamw4bit_multi_tensor. */
int lpmm_b200_sgd4bit_multi_tensor(const lpmm_b200_tensor* tensors, int n_tensors, const float* qmap,
                                   double weight_decay, double momentum, double lr, double dampening, int nesterov,
                                   int maximize, int64_t group_begin, int64_t group_end, void* stream);

/* Allocation-free variant of the factored step, for callers that cannot allocate device memory.
 * It has no counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a training loop whose memory is
 * entirely owned by a framework allocator or fixed up front, a process running under a memory
 * budget that forbids growth after start-up, or a caller that simply has no handle on a device
 * allocator and therefore cannot provide the scratch buffer that
 * lpmm_b200_adamw4bit_unfused_step wants for v_mode == LPMM_B200_STATE_FACTORED.
 *
 * What it does: exactly that step (same kernels, same results), with the column partial sums and
 * row means kept in a fixed array of LPMM_B200_STATIC_SCRATCH_BYTES that lives inside the library
 * image on every GPU that loads it, from load until the process exits.  The caller passes only
 * inputs and outputs.  Nothing is allocated or freed here, by this library or by any library it
 * calls.
 *
 * Limits and rules:
 *  - a tensor whose scratch need (lpmm_b200_factored_scratch_bytes) exceeds
 *    LPMM_B200_STATIC_SCRATCH_BYTES is refused with LPMM_B200_ERR_TOO_LARGE and nothing is launched
 *    (8 MiB covers a 32000 x 4096 matrix);
 *  - t->v_mode must be LPMM_B200_STATE_FACTORED (LPMM_B200_ERR_BAD_KIND otherwise);
 *  - the first call on each device looks up the array's device address; make that first call
 *    with the device current and before starting any stream capture;
 *  - all calls on a device share the one array: two calls that may overlap on the GPU (different
 *    streams, no dependency) race on it -- order them.  The array keeps whatever the last call
 *    left; no call relies on its previous contents. */
#define LPMM_B200_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int lpmm_b200_adamw4bit_factored_step_noalloc(const lpmm_b200_step_tensor* t, const float* qmap_m, double beta1,
                                              double beta2, double lr, double weight_decay, double eps, double step,
                                              void* stream);

/* Self-test hook (no counterpart in the reference; not part of any step).  The step kernels replace IEEE
 * division and square root and the reference's nearest-code search (fused_adamw_kernel.cu:27-49) by shorter
 * sequences that give the same result on a stated domain.  This runs one of those comparisons on the GPU over
 * n_samples pseudo-random and adversarial operands (seeded) and writes to out[0] the number of mismatches and to
 * out[1] the number of operands inside the domain (out: device pointer to two 64-bit counters, zeroed here).
 *   check 0  x / d by the shared reciprocal with residual correction  vs  div.rn   (2^-60 <= d <= 2^60, |x| <= d)
 *   check 1  the code of x / d (table, or closed form for the map k/16) vs the search on div.rn's quotient
 *   check 2  the short square root  vs  sqrt.rn    (v >= 2^-102 or v == 0)
 *   check 3  the short division     vs  div.rn     (2^-60 <= d <= 2^60, 2^-60 <= |m| <= 2^30 or m == 0)
 *   check 4  the code of an arbitrary float (table / closed form)  vs  the search
 * qmap (16 floats, device) selects the map of checks 1 and 4. */
int lpmm_b200_test_exactness(int check, const float* qmap, uint64_t seed, int64_t n_samples, unsigned long long* out,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LPMM_B200_H */
