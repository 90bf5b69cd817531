/*
 * aqt_b200.h -- C ABI of libaqt_b200.so: the quantized dot_general hot path of
 * google/aqt's aqt.jax.v2 as sm_100a CUDA kernels.
 *
 * The reference is pure Python on JAX and has no native boundary; the calls
 * below are what an XLA FFI custom-call handler (or any other host) binds in
 * place of the jnp/lax ops the reference traces. Each entry point names the
 * reference code it replaces (paths relative to aqt/jax/v2/).
 *
 * Conventions
 *  - every function returns 0 on success, a negative AQTB200_E* code for a bad
 *    argument / unsupported configuration, or a positive cudaError_t value;
 *    aqtb200_last_error() gives a human-readable message for the calling thread;
 *  - compute calls only ENQUEUE work on the caller's stream: no allocation, no
 *    synchronisation, no host readback. Scratch memory comes from the caller
 *    (size it with the matching *_workspace_bytes call);
 *  - all pointers in views/descriptors are device pointers unless stated;
 *  - strides are in ELEMENTS of the tensor they describe.
 */
#ifndef AQT_B200_H_
#define AQT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AQTB200_VERSION 1

/* error codes (negative); positive return values are cudaError_t */
#define AQTB200_OK 0
#define AQTB200_EINVAL (-1)      /* malformed argument (null pointer, bad extent, bad stride) */
#define AQTB200_EUNSUPPORTED (-2) /* valid request outside what the kernels cover */
#define AQTB200_EWORKSPACE (-3)  /* workspace too small or misaligned */
#define AQTB200_EDRIVER (-4)     /* CUDA driver entry point / tensor-map encode failed */
#define AQTB200_EDEVICE (-5)     /* a kernel reported a bounded wait that ran out */

typedef enum aqtb200_dtype {
  AQTB200_F32 = 0,
  AQTB200_BF16 = 1,
  AQTB200_S8 = 2,   /* also the container of int4 / intN values, N < 8 */
  AQTB200_E4M3 = 3, /* float8_e4m3fn */
  AQTB200_E5M2 = 4, /* float8_e5m2 */
  AQTB200_S32 = 5
} aqtb200_dtype;

typedef enum aqtb200_numerics_kind {
  AQTB200_NUM_NONE = 0, /* no_numerics.NoNumerics: value passes through as float */
  AQTB200_NUM_INT = 1,  /* int_numerics.IntSymmetric, preserve_zero, clip, round */
  AQTB200_NUM_FP8 = 2   /* fp8_numerics.Fp8Numerics, round-to-nearest-even */
} aqtb200_numerics_kind;

/*
 * A strided 4-D view [b0][b1][rows][cols] of one tensor.
 *   cols = the contraction index of the dot (the axis AbsMax shares a scale
 *          over, calibration.py:149), rows = the kept ("remaining") index,
 *   b0,b1 = up to two batch indices (extent 1 when unused).
 * Either col_stride == 1 (contraction contiguous) or row_stride == 1; the
 * latter makes the quantize kernel transpose through shared memory, because
 * its OUTPUT always has the contraction index contiguous.
 */
typedef struct aqtb200_view {
  const void* ptr;
  int32_t dtype; /* aqtb200_dtype */
  int32_t reserved;
  int64_t b0, b1, rows, cols;
  int64_t b0_stride, b1_stride, row_stride, col_stride;
} aqtb200_view;

/*
 * How one operand is calibrated and quantized. Mirrors aqt_quantizer.Quantizer
 * + calibration.AbsMaxCalibration + the numerics object
 * (aqt_quantizer.py:37-176, calibration.py:106-157, numerics/int_numerics.py:
 * 24-111, numerics/fp8_numerics.py:67-123).
 */
typedef struct aqtb200_quant_spec {
  int32_t kind;          /* aqtb200_numerics_kind */
  int32_t qdtype;        /* container: AQTB200_S8, _E4M3, _E5M2 (NONE: = compute_dtype) */
  float quant_bound;     /* numerics.get_quant_bound(): 127.5, 7.5, 448, 57344, ... */
  float clip_bound;      /* forward clip: 127, 7, 448, 57344, ... */
  int32_t per_tensor;    /* calib_shared_axes == "per_tensor": one scale for everything */
  int32_t compute_dtype; /* T: dtype the operand has when arithmetic starts (F32|BF16);
                            int8/fp8 inputs are widened to it exactly first */
  int32_t scale_dtype;   /* dtype of the scale array (F32|BF16); T unless scale_dtype set */
  int32_t po2_scale;     /* calibration.ceil_to_po2 */
  float clipping_scale;  /* AbsMaxCalibration.clipping_scale ALREADY ROUNDED to T; 0 = unset */
  int32_t reserved;
} aqtb200_quant_spec;

/*
 * aqtb200_quantize: AbsMax calibrate + quantize one operand.
 * Replaces: AbsMaxCalibration.get_scale_and_bias_and_sparsity (calibration.py:
 * 117-157), QTensor.quant (aqt_tensor.py:125-159), IntSymmetric.vjp_fwd
 * (numerics/int_numerics.py:81-111) / Fp8Numerics.vjp_fwd (numerics/
 * fp8_numerics.py:88-123) and, when `prescale` is given, the cotangent
 * pre-scaling of _maybe_use_fwd_quant (aqt_dot_general.py:714-720).
 *
 *   v      = widen(x) [* cast_T(prescale[b0,b1,col])]            (rounded to T)
 *   scale  = where(max|v|==0, 1, max|v|) [* clipping_scale] / quant_bound   (in T, stored as scale_dtype)
 *   q      = cast(round_half_even(clip(v * (1/scale) [+ noise])))           (int)
 *          = cast_fp8(clip(v * (1/scale)))                                  (fp8)
 *
 * x        : input view (dtype F32/BF16, or S8/E4M3/E5M2 when re-quantizing a
 *            stored QTensor as the backward pass does with use_fwd_quant).
 * prescale : optional (ptr may be NULL). Indexed [b0][b1][col] through its
 *            b0/b1/col strides (rows, row_stride ignored); dtype F32/BF16.
 * noise    : optional f32 view with x's extents (stochastic rounding input,
 *            U[-0.5,0.5)); int numerics only.
 * scale_in : optional. When non-NULL calibration is skipped and this scale
 *            (layout of scale_out) is used: Quantizer.calculate_qvalue on a
 *            caller-supplied incomplete QTensor (aqt_dot_general.py:645-653).
 * q_out    : [b0][b1][rows][ldq] bytes, contraction contiguous, ldq =
 *            aqtb200_round_up(cols,16); batch strides rows*ldq and b1*rows*ldq;
 *            bytes past `cols` in each row are written as zero.
 * scale_out: [b0][b1][rows] of scale_dtype, or a single element when
 *            spec->per_tensor.
 * workspace: aqtb200_quantize_workspace_bytes() bytes, 256-byte aligned.
 */
int aqtb200_quantize(const aqtb200_view* x, const aqtb200_view* prescale,
                     const aqtb200_view* noise, const aqtb200_quant_spec* spec,
                     const void* scale_in, void* q_out, void* scale_out,
                     void* workspace, size_t workspace_bytes, void* stream);

size_t aqtb200_quantize_workspace_bytes(const aqtb200_view* x,
                                        const aqtb200_quant_spec* spec);

/*
 * aqtb200_quantize_static: aqtb200_quantize for callers that cannot hand over
 * scratch memory. (No counterpart in the reference: it exists for the hosts
 * this library gets embedded in, not for AQT's semantics.)
 *
 * Who needs it: a host that owns every byte of device memory through its own
 * allocator and passes a custom call only its operands and results -- an XLA
 * custom call registered without a scratch result is the typical case -- or a
 * serving loop that forbids calls into the CUDA allocator once it is warm.
 * Such a caller has nowhere to get the amax cells and reciprocal scales that
 * aqtb200_quantize wants in `workspace`, and must not cudaMalloc them.
 *
 * The scratch therefore lives inside the library: one fixed device array per
 * GPU (2 x 256 KiB, resident from library load to process exit). Consequences:
 *  - at most AQTB200_STATIC_MAX_SCALES scales per call (b0*b1*rows, or 1 with
 *    a per-tensor scale); larger requests return AQTB200_EUNSUPPORTED with a
 *    message and launch nothing;
 *  - the first call on each device looks the array's address up
 *    (cudaGetSymbolAddress, with that device current) and caches it; make that
 *    first call before starting any stream capture on the device;
 *  - every call on a device shares the one array, which still holds the
 *    previous call's values when the next one starts (the kernel sequence
 *    zeroes the cells it accumulates into). Two calls whose kernels can run at
 *    the same time -- different streams, no ordering between them -- race on
 *    it; order them, or use aqtb200_quantize with separate workspaces;
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine.
 * Arguments and results are those of aqtb200_quantize minus the workspace.
 */
#define AQTB200_STATIC_MAX_SCALES 65536
int aqtb200_quantize_static(const aqtb200_view* x, const aqtb200_view* prescale,
                            const aqtb200_view* noise,
                            const aqtb200_quant_spec* spec, const void* scale_in,
                            void* q_out, void* scale_out, void* stream);

/* aqtb200_absmax_scale: the calibration half alone (scale_out only).
 * Replaces Quantizer.calibrate (aqt_quantizer.py:79-157). */
int aqtb200_absmax_scale(const aqtb200_view* x, const aqtb200_view* prescale,
                         const aqtb200_quant_spec* spec, void* scale_out,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * The two halves of aqtb200_absmax_scale, for callers that combine maxima
 * before turning them into scales -- several ranks holding shards of one
 * tensor (max-all-reduce in between), or one tensor that is quantized more
 * than once with different prescales, as the cotangent is in the backward
 * pass (aqt_dot_general.py:1206-1217).
 *   aqtb200_absmax_raw     : amax_out[i] = max |x| over the contraction index
 *                            (or the whole tensor), f32, 0 for an all-zero unit;
 *   aqtb200_scale_from_amax: scale = where(a==0,1,a)[*clipping]/quant_bound with
 *                            a = |round_T(amax * round_T(prescale[0]))|. Because
 *                            rounding is monotone this equals the maximum of the
 *                            prescaled elements whenever ONE prescale value
 *                            covers the reduced range (per-tensor forward scale).
 */
int aqtb200_absmax_raw(const aqtb200_view* x, int32_t per_tensor, float* amax_out,
                       void* stream);
int aqtb200_scale_from_amax(const float* amax, int64_t n, const void* prescale,
                            int32_t prescale_dtype, const aqtb200_quant_spec* spec,
                            void* scale_out, void* stream);

/*
 * One pass over an operand for the two layouts a training step needs it in.
 * The reference quantizes every operand twice: lhs for the forward dot and,
 * from the stored forward values, again for drhs; rhs likewise for dlhs
 * (_maybe_use_fwd_quant, aqt_dot_general.py:675-729); the cotangent once per
 * gradient dot (:1206-1217). The two contractions of one operand run along
 * different axes, so the two quantized copies are transposes of each other in
 * memory. aqtb200_quantize_pair reads the bf16 operand once and writes both:
 *   q_t [b0][b1][rows][cols]  the strided index of x contiguous (as the
 *                             transposing mode of aqtb200_quantize writes it);
 *   q_s [b0][b1][cols][rows]  x's own orientation.
 * x: row_stride == 1, col_stride != 1, rows and cols multiples of 16, every
 * stride a multiple of 8 elements. Each output has its own spec (fp8 or int8,
 * per_tensor, bf16 compute and scale dtype), its own one-element bf16 scale
 * and an optional one-element prescale. With amax == NULL the scales are
 * INPUTS. With amax given (one f32, the operand's raw maximum from
 * aqtb200_absmax_raw, max-reduced across ranks if the operand is sharded) they
 * are OUTPUTS: the kernel derives them as aqtb200_scale_from_amax and, for the
 * chained output, aqtb200_requant_amax would, so an operand costs two
 * launches in all.
 * chain = 0: both outputs quantize x (the cotangent);
 * chain = 1: q_s quantizes the values of q_t (x -> q_t -> q_s: q_t is the
 *            forward copy, q_s the backward re-quantization of it);
 * chain = 2: q_t quantizes the values of q_s.
 * amax_out, when non-NULL, receives max |x| (one f32, set by this call): with
 * scales that do not depend on this step's maximum (delayed scaling,
 * flax/delayed_scaling_calibration.py) the operand is then read ONCE in all --
 * quantized with the history's scales while its maximum for the next steps'
 * history is taken from the same read.
 * Results are bit-identical to two aqtb200_quantize calls. Other dtypes,
 * per-channel scales or noise: -2 (AQTB200_EUNSUPPORTED); call
 * aqtb200_quantize twice.
 *
 * aqtb200_requant_amax supplies the calibration of the chained output without
 * a pass over the data: quantization is monotone and odd, so the largest
 * magnitude among the quantized values is amax_q[i] = |value(Q(amax[i]))|, from
 * which aqtb200_scale_from_amax gives the second scale. `spec`, `scale` and
 * `prescale` are those of the FIRST quantization.
 */
int aqtb200_quantize_pair(const aqtb200_view* x,
                          const aqtb200_quant_spec* spec_t, void* scale_t,
                          const void* prescale_t, int32_t prescale_t_dtype, void* q_t,
                          const aqtb200_quant_spec* spec_s, void* scale_s,
                          const void* prescale_s, int32_t prescale_s_dtype, void* q_s,
                          int32_t chain, const float* amax, float* amax_out, void* stream);
int aqtb200_requant_amax(const float* amax, int64_t n, const void* prescale,
                         int32_t prescale_dtype, const aqtb200_quant_spec* spec,
                         const void* scale, float* amax_q_out, void* stream);

/*
 * aqtb200_quantize_dual: the cotangent's TWO calibrations and quantizations
 * (one per gradient dot, aqt_dot_general.py:1206-1217, each with the other
 * operand's forward scale folded in first, :714-720, and each with its own
 * stochastic-rounding noise, numerics/int_numerics.py:88-110) in two passes
 * over it instead of four, for per-row ("per token" / "per channel") scales:
 * the batched counterpart of aqtb200_quantize_pair.
 *
 * x is viewed as [b0][b1][cols][rows] with rows contiguous (row_stride 1).
 *   output S [b][cols][rows], x's orientation, contraction index = rows:
 *     v = round(x * prescale_s[b][row]); scale_s[b][col] = max_row |v| / bound;
 *     q_s = int8(round_half_even(clip(round(v / scale_s) + noise_s)))
 *   output T [b][rows][cols], transposed, contraction index = cols:
 *     v = round(x * prescale_t[b][col]); scale_t[b][row] = max_col |v| / bound;
 *     q_t likewise with noise_t.
 * For the cotangent g[..., t, s] of an einsum: rows = s, cols = t; S feeds dlhs
 * (contracts s), T feeds drhs (contracts t).
 * Requirements: x bf16; both specs int8, per-row scales, bf16 compute and scale
 * dtype; rows and cols multiples of 16; prescales bf16 (ptr NULL = none),
 * prescale_t indexed through its b0/b1/col strides, prescale_s through its
 * b0/b1/row strides; noise f32 in x's own layout, for both outputs or neither.
 * Results are bit-identical to two aqtb200_quantize calls. Anything else: -2.
 */
typedef struct aqtb200_dual_desc {
  aqtb200_view x;
  aqtb200_quant_spec spec_t, spec_s;
  aqtb200_view prescale_t, prescale_s;
  aqtb200_view noise_t, noise_s;
  void* q_t;      /* [b0][b1][rows][cols] int8 */
  void* scale_t;  /* [b0][b1][rows] bf16 */
  void* q_s;      /* [b0][b1][cols][rows] int8 */
  void* scale_s;  /* [b0][b1][cols] bf16 */
} aqtb200_dual_desc;

size_t aqtb200_quantize_dual_workspace_bytes(const aqtb200_dual_desc* desc);
int aqtb200_quantize_dual(const aqtb200_dual_desc* desc, void* workspace, size_t workspace_bytes,
                          void* stream);

int64_t aqtb200_round_up(int64_t v, int64_t multiple);

/*
 * One batched GEMM  acc[b,m,n] = sum_k A[b,m,k] * B[b,n,k]  on tcgen05 tensor
 * cores (kind::i8 -> int32, kind::f8f6f4 -> f32) with the dequantizing
 * epilogue fused. Replaces lax.dot_general at aqt_dot_general.py:921-927
 * together with QTensor.dequant (aqt_tensor.py:161-200) and the output
 * transpose of the backward pass (aqt_dot_general.py:1201).
 *
 *   r = cast_D(acc); r *= first scale; r *= second scale; out = cast_out(r)
 * where each multiply rounds to promote(current dtype, scale dtype), exactly
 * as the chain of jnp multiplies does; "first" is A's scale unless
 * b_scale_first.
 */
typedef struct aqtb200_gemm_desc {
  int64_t b0, b1, m, n, k;
  /* operands: 1-byte elements, k contiguous, row strides multiples of 16 */
  const void* a;
  int64_t a_b0_stride, a_b1_stride, lda;
  const void* b;
  int64_t b_b0_stride, b_b1_stride, ldb;
  int32_t a_dtype, b_dtype; /* S8/S8, or any mix of E4M3/E5M2 */
  /* scales: NULL = operand not quantized (factor 1). A stride of 0 on every
     index = per-tensor scalar. */
  const void* a_scale;
  int64_t a_scale_b0_stride, a_scale_b1_stride, a_scale_m_stride;
  const void* b_scale;
  int64_t b_scale_b0_stride, b_scale_b1_stride, b_scale_n_stride;
  int32_t a_scale_dtype, b_scale_dtype; /* F32|BF16 */
  int32_t b_scale_first;                /* multiply by B's scale before A's */
  int32_t dequant_dtype;                /* D: F32|BF16 (promote(lhs.dtype, rhs.dtype)) */
  void* out;
  int32_t out_dtype; /* F32|BF16 */
  int32_t reserved;
  int64_t out_b0_stride, out_b1_stride, out_m_stride, out_n_stride;
  /* optional raw accumulators, contiguous [b0][b1][m][n], int32 or f32: for
     parity checks of the tensor-core result, and -- with out == NULL -- for a
     contraction sharded over several GPUs, whose partial sums are added
     across ranks before the one dequantization (aqtb200_dot_general_raw_dequant). */
  void* acc_out;
  /* optional: one f32 cell, zeroed by the caller, that receives max |out| over
     everything this call writes (of the values as stored, i.e. after the last
     rounding), by atomic max on the bit pattern. A consumer that quantizes this
     output with a per-tensor scale -- the next layer, or a delayed-scaling
     calibrator (flax/delayed_scaling_calibration.py:119-124) -- then needs no
     pass of its own over it. NULL = not wanted. */
  float* amax_out;
  /* optional scratch, 256-byte aligned, aqtb200_gemm_workspace_bytes() bytes:
     with it a skinny problem (at most 64 columns against many row tiles, the
     decode-time serving GEMM) has its contraction split into parts that fill
     the SMs evenly, the part that finishes a tile last summing the others'
     accumulators and dequantizing. Without it (NULL) every tile is one unit of
     work. Results are identical for int8; fp8 sums its parts in part order. */
  void* workspace;
  size_t workspace_bytes;
} aqtb200_gemm_desc;

/* status: device int32[4], zeroed by the caller before first use; a kernel
 * whose bounded wait ran out writes a non-zero code there instead of hanging.
 * May be NULL. */
int aqtb200_gemm_dequant(const aqtb200_gemm_desc* desc, int32_t* status,
                         void* stream);
/* scratch that lets aqtb200_gemm_dequant split the contraction (0 when the
 * problem would not be split) */
size_t aqtb200_gemm_workspace_bytes(const aqtb200_gemm_desc* desc);

/*
 * aqtb200_dot_general_raw: one whole DotGeneralRaw.__call__
 * (aqt_dot_general.py:757-840) = quantize lhs, quantize rhs, contraction,
 * dequantize, for operands already normalised to views. The forward pass, the
 * dlhs pass and the drhs pass of dg_core_vjp_fwd / dg_core_vjp_bwd
 * (aqt_dot_general.py:1098-1221) are three calls of it with different views,
 * specs and prescales.
 *
 * lhs_q_in / rhs_q_in: when non-NULL the operand arrives already quantized
 * (serving, aqt_dot_general.py:623-635): the view's dtype is the container
 * type with contraction contiguous and its scale is passed in *_scale_in.
 */
typedef struct aqtb200_dg_raw_desc {
  aqtb200_view lhs, rhs;                    /* rows = M resp. N, cols = K */
  aqtb200_view lhs_prescale, rhs_prescale;  /* ptr NULL when absent */
  aqtb200_view lhs_noise, rhs_noise;        /* ptr NULL when absent */
  aqtb200_quant_spec lhs_spec, rhs_spec;
  const void* lhs_scale_in;                 /* optional caller-supplied scales */
  const void* rhs_scale_in;
  int32_t lhs_is_quantized, rhs_is_quantized;
  /* outputs of the quantization step (residuals of the forward pass) */
  void* lhs_q;      /* [b0][b1][M][ldk] */
  void* lhs_scale;  /* [b0][b1][M] or [1] */
  void* rhs_q;      /* [b0][b1][N][ldk] */
  void* rhs_scale;  /* [b0][b1][N] or [1] */
  /* output of the dot */
  int32_t swap_ab;  /* run the GEMM as (rhs rows) x (lhs rows): out tile rows = N */
  int32_t dequant_dtype;
  void* out;
  int32_t out_dtype;
  int32_t reserved;
  int64_t out_b0_stride, out_b1_stride, out_m_stride, out_n_stride;
  void* acc_out;
  float* amax_out;  /* as aqtb200_gemm_desc.amax_out */
  /* optional NUL-terminated name ("aqt_fwd", "aqt_dlhs", "aqt_drhs": the
     reference's DotGeneralRaw.jax_scope_name, entered as jax.named_scope at
     aqt_dot_general.py:767). The call's kernels are enclosed in an NVTX range
     of that name, so a profiler timeline shows the three passes. */
  const char* scope_name;
} aqtb200_dg_raw_desc;

size_t aqtb200_dot_general_raw_workspace_bytes(const aqtb200_dg_raw_desc* desc);

/* When desc->out is NULL and desc->acc_out is set, aqtb200_dot_general_raw
 * stops after the contraction and leaves the raw accumulators in acc_out
 * ([b0][b1][M][N], or [b0][b1][N][M] with swap_ab). A caller that shards the
 * contraction index over several GPUs sums those accumulators across ranks
 * and then calls aqtb200_dot_general_raw_dequant with the SAME descriptor
 * (out now set) to apply the dequantizing epilogue once, to the total. */

int aqtb200_dot_general_raw(const aqtb200_dg_raw_desc* desc, void* workspace,
                            size_t workspace_bytes, int32_t* status,
                            void* stream);

int aqtb200_dot_general_raw_dequant(const aqtb200_dg_raw_desc* desc,
                                    void* stream);

/* The sum across ranks, the dequantization and the distribution of the result
 * in one kernel over peer memory (one process per GPU on NVLink). With the
 * SAME descriptor, narrowed to a band of accumulator rows as for
 * aqtb200_dot_general_raw_dequant: acc[r] is rank r's accumulator band
 * ([rows][N], 4-byte, 16-byte aligned; the other ranks' through mappings made
 * with aqtb200_ipc_open), out[r] the band's place in rank r's output. The
 * calling rank reads every acc[r], adds them in rank order (so the f32 total
 * does not depend on who computes a band), dequantizes once and writes the
 * band to every out[r]. desc->out and desc->acc_out are ignored. The caller
 * orders this call after every rank's contraction of the band (a barrier or a
 * small collective on the same stream) and orders its readers of `out` after
 * every rank's call. world: 2, 4 or 8. max_sms > 0 caps the SMs the kernel
 * occupies (it runs beside a GEMM whose own cap is aqtb200_set_gemm_sm_budget).
 * The accumulators travel through the TMA unit (bulk copies, 192 KB in flight
 * per SM); status as for aqtb200_dot_general_raw (4 / 5: a bounded wait of the
 * exchange ran out).
 * Replaces: nothing in the reference (which has no collective on this path);
 * it is what ncclReduceScatter + dequantize + ncclAllGather would do. */
#define AQTB200_MAX_RANKS 8
typedef struct aqtb200_exchange_desc {
  int32_t world, rank;
  const void* acc[AQTB200_MAX_RANKS];
  void* out[AQTB200_MAX_RANKS];
  int32_t max_sms;
} aqtb200_exchange_desc;
int aqtb200_dot_general_raw_exchange(const aqtb200_dg_raw_desc* desc,
                                     const aqtb200_exchange_desc* exchange,
                                     int32_t* status, void* stream);

/* Elementwise helpers for the piecewise API (QTensor.quant / QTensor.dequant
 * used outside the fused path, aqt_tensor.py:125-200):
 *   dequantize: out = cast_D(q) * scale   (one scale, broadcast by strides) */
int aqtb200_dequantize(const aqtb200_view* q, const aqtb200_view* scale,
                       int32_t dequant_dtype, void* out, void* stream);

/*
 * Device memory and copies for hosts that bring no allocator of their own (a
 * ctypes harness, a test written in C). No counterpart in the reference: XLA
 * owns all buffers there. The copies are asynchronous on `stream`;
 * aqtb200_sync waits for it. Compute entry points never call these.
 */
int aqtb200_set_device(int device);
int aqtb200_dev_alloc(void** out, size_t bytes);
int aqtb200_dev_free(void* ptr);
int aqtb200_dev_memset(void* ptr, int value, size_t bytes, void* stream);
int aqtb200_h2d(void* dst, const void* src, size_t bytes, void* stream);
int aqtb200_d2h(void* dst, const void* src, size_t bytes, void* stream);
int aqtb200_sync(void* stream);
/* Peer memory for the fused exchange: a 64-byte handle of a device allocation
 * (ptr: its base address, e.g. from aqtb200_dev_alloc) that another process on
 * the same node opens as a pointer valid on ITS current device (peer access is
 * enabled on first use). Close every opened pointer before the owner frees. */
int aqtb200_ipc_export(const void* ptr, void* handle64);
int aqtb200_ipc_open(const void* handle64, void** out);
int aqtb200_ipc_close(void* ptr);

/*
 * Collectives of the row-sharded path (one process per GPU; the rows of lhs
 * and of the cotangent split over the ranks). The reference has no collective
 * on this path (flax/aqt_flax_calibration.py:161-164 refuses cross-replica
 * statistics); these are what a sharded host needs to keep the result equal
 * to one device's: a max-all-reduce of the absolute maxima behind per-tensor
 * scales, and the sum of drhs's raw accumulators before the one dequantization
 * (all-reduce, or reduce-scatter + all-gather of the finished bands).
 * NCCL (libnccl.so.2) is opened on first use. Rank 0 makes a 128-byte id with
 * aqtb200_comm_unique_id and hands it to every rank by whatever channel the
 * host has; all ranks then call aqtb200_comm_init. dtype: AQTB200_F32, _S32 or
 * _BF16; the calls are asynchronous on `stream`.
 */
int aqtb200_comm_unique_id(void* id128);
int aqtb200_comm_init(int nranks, int rank, const void* id128, void** comm_out);
int aqtb200_comm_destroy(void* comm);
/* in place; op_max != 0: maximum, else sum */
int aqtb200_allreduce(void* comm, void* buf, int64_t count, int32_t dtype, int32_t op_max,
                      void* stream);
/* send holds nranks * recv_count elements; rank r receives the sum of block r */
int aqtb200_reduce_scatter_sum(void* comm, const void* send, void* recv, int64_t recv_count,
                               int32_t dtype, void* stream);
/* recv holds nranks * send_count elements (send may be recv + rank * send_count) */
int aqtb200_all_gather(void* comm, const void* send, void* recv, int64_t send_count, int32_t dtype,
                       void* stream);

/* library / device queries */
int aqtb200_version(void);
/* 1 when the library was built with jaxlib's xla/ffi/api/ffi.h available and so
 * also exports the XLA FFI handler AqtB200DgRaw (csrc/xla_ffi.cc), else 0. */
int aqtb200_has_xla_ffi(void);
const char* aqtb200_last_error(void);
int aqtb200_device_sm_count(int* out);
/* number of kernels this library has launched in this process (all threads);
 * lets a harness report how much of its timed region ran in these kernels. */
int64_t aqtb200_kernel_launch_count(void);
/* selects the contraction kernel: 0 = tcgen05, chosen by shape: CTA pairs
 * (cta_group::2) when M > 128 -- 256 x 512 tiles when also N > 256 and the
 * contraction is at least 2048 bytes long, 256 x 256 tiles otherwise -- and
 * single CTAs (128 x 256) for M <= 128 (default); 1 = plain CUDA-core
 * reference kernel kept for cross-checking the tensor-core path; 2 = always
 * single CTAs; 3 = always 256 x 256 CTA pairs; 4 = always 256 x 512 CTA
 * pairs. */
int aqtb200_set_gemm_impl(int impl);
/* Caps the number of SMs the persistent GEMM kernels occupy (0 = all of them).
 * A caller that runs a collective concurrently with a GEMM leaves it room
 * this way: a persistent grid that fills every SM would otherwise make the
 * collective's kernel (or the GEMM's last CTAs) wait for a free SM. */
int aqtb200_set_gemm_sm_budget(int max_sms);

/*
 * Delayed scaling (flax/delayed_scaling_calibration.py:28-124, per-tensor): the
 * scale of a step comes from the maxima of earlier steps, so quantization does
 * not wait for a reduction over its own operand.
 *   aqtb200_delayed_scaling_scale: get_bound() + get_scale_and_bias_and_sparsity():
 *     new_bound = max(history) when that is > 0 and finite, else bound[0]
 *     (compute_bound, :107-111); bound[0] = new_bound when update_bound (TRAIN /
 *     CALIBRATE modes, :93-95); scale_out[0] = cast(new_bound / quant_bound),
 *     rounded to a power of two first when spec->po2_scale. f32 arithmetic, as
 *     the reference's f32 state arrays give.
 *   aqtb200_delayed_scaling_push: compute_history (:113-118):
 *     history = roll(history, -1), then history[0] = amax[0] (the operand's
 *     max |x|, e.g. from aqtb200_absmax_raw or a producer's amax_out).
 * history: f32[len], 1 <= len <= 4096; bound, amax: f32[1]. Call _scale before
 * _push within a step (the new bound reads the old history).
 */
int aqtb200_delayed_scaling_scale(const float* history, int64_t len, float* bound,
                                  int32_t update_bound, const aqtb200_quant_spec* spec,
                                  void* scale_out, void* stream);
int aqtb200_delayed_scaling_push(float* history, int64_t len, const float* amax, void* stream);
/* out[i] = |round_T(amax[i] * round_T(prescale[0]))|: the maximum of a tensor
 * once ONE prescale value has been folded into it, as the cotangent's is by
 * _maybe_use_fwd_quant (aqt_dot_general.py:714-720); T = compute_dtype. */
int aqtb200_prescale_amax(const float* amax, int64_t n, const void* prescale, int32_t prescale_dtype,
                          int32_t compute_dtype, float* out, void* stream);

/*
 * aqtb200_jax_noise: the stochastic-rounding noise tensor, generated on the
 * device. Replaces stochastic_rounding.JaxUniform (stochastic_rounding.py:
 * 35-46: jax.random.uniform(key, shape) - 0.5; kind 0 with shift 0.5) and
 * RandomCenteredUniform (:49-78: 16 random bits in an f32 mantissa, minus
 * 1.5 - 2^-17; kind 1, shift ignored). (key0, key1) is the raw threefry key;
 * `partitionable` picks jax's counter layout (jax_threefry_partitionable);
 * out receives n floats in row-major order of the noise tensor's shape.
 * jax's generator is restated from its published algorithm; it could not be
 * compared with a jax installation.
 */
int aqtb200_jax_noise(uint32_t key0, uint32_t key1, int64_t n, int32_t kind,
                      int32_t partitionable, float shift, float* out, void* stream);

/*
 * aqtb200_mma_peak: measurement helper, no counterpart in the reference.
 * Launches one CTA per SM that issues `mmas_per_sm` (rounded up to a multiple
 * of 16) tcgen05 MMAs of 128 x 256 x 32 -- kind::i8 when is_int, else
 * kind::f8f6f4 on e4m3 -- from operands that stay in shared memory, with no
 * loads from global memory and no epilogue. Timed with events around it, it
 * gives the 8-bit tensor-pipe ceiling of the device it runs on:
 *   ops = SMs * launched MMAs per SM * 2 * 128 * 256 * 32.
 * status as for aqtb200_gemm_dequant.
 */
int aqtb200_mma_peak(int32_t is_int, int64_t mmas_per_sm, int32_t* status, void* stream);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* AQT_B200_H_ */
