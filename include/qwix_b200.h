/*
 * qwix_b200 -- C ABI of the B200 (sm_100a) backend for qwix's quantized-inference path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, returns an
 * int32 status (0 = ok) and never allocates device memory: outputs and scratch are the
 * caller's.  Calls are re-entrant; the library keeps no mutable state besides a cache of
 * immutable driver entry points.  Paths cited below are inside the google/qwix tree.
 *
 * Array views.  A quantizer call sees its operand as a contiguous row-major [P, R, C]
 * array cut into tiles of (tp, tr, tc) elements; every tile owns one scale (and one
 * zero point), stored row-major as [P/tp, R/tr, C/tc].  This is the rank-collapsed form
 * of qwix's (channelwise_axes, tiled_axes): a channelwise axis has tile 1, a reduced axis
 * has tile = extent, a sub-channel axis has its tile size (qarray.py:332-349).
 *
 * int4.  QWX_S4 buffers are packed two codes per byte along C, low nibble = even index.
 * QWX_S4U holds one sign-extended code per byte (the logical layout of a QArray).
 */
#ifndef QWIX_B200_H_
#define QWIX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* qwx_stream_t; /* a cudaStream_t */

enum qwx_status {
  QWX_OK = 0,
  QWX_ERR_NULL = 1,        /* required pointer is NULL                       */
  QWX_ERR_SHAPE = 2,       /* extents / tiles inconsistent (ValueError)      */
  QWX_ERR_ALIGN = 3,       /* pointer or pitch misaligned for the kernel     */
  QWX_ERR_DTYPE = 4,       /* dtype combination not implemented (ValueError) */
  QWX_ERR_UNSUPPORTED = 5, /* valid in qwix, not built here                  */
  QWX_ERR_WORKSPACE = 6,   /* workspace missing or too small                 */
  QWX_ERR_LAUNCH = 7,      /* CUDA reported a launch / driver error          */
  QWX_ERR_DEVICE_WAIT = 8, /* a bounded device-side wait ran out             */
  QWX_ERR_NO_DEVICE = 9    /* no sm_100 device / driver entry point missing  */
};

enum qwx_dtype {
  QWX_F32 = 0, QWX_BF16 = 1, QWX_F16 = 2,
  QWX_S8 = 3, QWX_S4 = 4, QWX_E4M3 = 5, QWX_S32 = 6, QWX_S4U = 7,
  /* e4m3 codes whose scale is a power of two ("mxfp8": one scale per 32 values along the
   * contracted axis; qwix/_src/core/qarray.py:306-325, 566-579).  A quantizer qtype only: the
   * stored codes are QWX_E4M3 bytes for every other entry point. */
  QWX_MXFP8 = 8,
  QWX_MXFP4 = 9,     /* e2m1 codes, one per byte (low nibble), power-of-two scale per 32 values */
  QWX_NVFP4 = 10     /* e2m1 codes, one per byte (low nibble), e4m3-valued scale per 16 values */
};

enum qwx_calibration { QWX_ABSMAX = 0, QWX_MINMAX = 1, QWX_RMS = 2 };

/* How intermediates of x / scale (+ zero_point) round before round-half-even:
 * STRICT rounds every primitive to the array dtype (JAX eager semantics),
 * FUSED keeps them in float32 (XLA under jit).  Identical for float32 arrays. */
enum qwx_rounding { QWX_STRICT = 0, QWX_FUSED = 1 };

/* B-operand memory order of the GEMMs.  QWX_B_KN: the weight as qwix holds it, [K, N]
 * row-major (N contiguous).  QWX_B_NK: a pre-transposed copy, [N, K] row-major. */
enum qwx_b_layout { QWX_B_KN = 0, QWX_B_NK = 1 };

/* Epilogue rounding of the quantized GEMMs.  QWX_EPI_F32: float(acc) * sa * sb computed
 * in float32, rounded once to the output dtype.  QWX_EPI_REFERENCE: every step rounds to
 * the output dtype in the reference's order R(R(R(acc) * sa) * sb) (dot_general.py:255-261). */
enum qwx_epilogue { QWX_EPI_F32 = 0, QWX_EPI_REFERENCE = 1 };

int qwx_version(void);
const char* qwx_status_string(int status);

/* Process-wide option: launch the short kernels of a decode step (qwx_gemm_q8_decode, the
 * fused decoder stages below, the one-pass row quantizers) with CUDA's programmatic stream
 * serialization, so that a kernel's set-up and its weight fetches overlap the tail of the
 * kernel before it on the same stream.  Each of these kernels waits (griddepcontrol.wait) for
 * its predecessor before it reads an activation or writes anything, so results do not change.
 * Off by default; safe to set at any time, affects launches made afterwards (stream capture
 * included).  The reference has no counterpart (XLA schedules its own kernels). */
void qwx_set_programmatic_launch(int enabled);
int qwx_get_programmatic_launch(void);

/* Bytes of scratch the quantizer calls below need for this view (zero is possible). */
size_t qwx_quantize_workspace_bytes(int64_t P, int64_t R, int64_t C,
                                    int64_t tp, int64_t tr, int64_t tc);

/* qarray.calibrate (qarray.py:470-534): per-tile absmax, (min, max) or rms*arg.
 * out_a = absmax (or min), out_b = max for QWX_MINMAX else NULL; both in x_dtype.
 * has_arg selects the optional multiplier of absmax/minmax (required for rms). */
int qwx_calibrate(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C,
                  int64_t tp, int64_t tr, int64_t tc, int method, int has_arg,
                  double arg, void* out_a, void* out_b, void* workspace,
                  size_t workspace_bytes, qwx_stream_t stream);

/* qarray.compute_scale_zero_point (qarray.py:537-584) for int8/int4/e4m3 codes.
 * calib_b == NULL: symmetric, scale = calib_a / bound.  Otherwise asymmetric with
 * (min, max) = (calib_a, calib_b); zero_point is written as int8 codes. */
int qwx_compute_scale_zero_point(const void* calib_a, const void* calib_b, int dtype,
                                 int64_t n, int qtype, void* scale, void* zero_point,
                                 qwx_stream_t stream);

/* qarray.quantize_with_scale_zero_point (qarray.py:594-635): true division by the scale
 * (already in x_dtype), optional zero point (int8 codes), round-half-even + saturate
 * (ints) or clip + RN-even (e4m3) (numerics.py:139-196). */
int qwx_quantize_with_scale(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C,
                            int64_t tp, int64_t tr, int64_t tc, const void* scale,
                            const void* zero_point, int qtype, int rounding, void* q,
                            qwx_stream_t stream);

/* qarray.quantize (qarray.py:638-644): the three steps above in as few passes over x as
 * the view allows (one pass when tiles are row segments or fit in shared memory).
 * scale is written in x_dtype; zero_point (int8 codes) only for QWX_MINMAX. */
int qwx_quantize(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C,
                 int64_t tp, int64_t tr, int64_t tc, int method, int has_arg, double arg,
                 int qtype, int rounding, void* q, void* scale, void* zero_point,
                 void* workspace, size_t workspace_bytes, qwx_stream_t stream);

/* qwx_quantize for callers that have no way to provide scratch memory.  It has no
 * counterpart in the reference (XLA plans scratch for its own fusions); it exists for users of
 * this library such as a custom-call handler inside a framework that fixed all of its buffers
 * before the step started, or a serving process that must not call cudaMalloc once it is
 * warm (the call synchronises the device and may fail when memory is tight).
 *
 * Same arguments and results as qwx_quantize, without the workspace pair: the scratch is a
 * 1 MiB array in device global memory that is part of the library (every GPU that loads the
 * library holds it until the process ends; qwx_quantize_builtin_scratch_bytes() reports its
 * size).  Limit: the view may have at most 65,520 tiles (16 bytes of statistics per tile plus
 * 256); larger views return QWX_ERR_WORKSPACE and nothing is launched.  Views whose tiles are
 * row segments need no scratch and are never refused.
 *
 * The first call on each device looks up the array's device address (one
 * cudaGetSymbolAddress, made with that device current, result cached); make that first call
 * before starting any stream capture.  The call itself never allocates: no cudaMalloc,
 * cudaFree or allocating library routine.  All calls on a device share the one array and it
 * keeps whatever the previous call left, so each call clears the part it accumulates into;
 * two calls whose kernels overlap on the GPU (different streams, no ordering between them)
 * race on it and must be serialised by the caller. */
size_t qwx_quantize_builtin_scratch_bytes(void);
int qwx_quantize_noalloc(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C,
                         int64_t tp, int64_t tr, int64_t tc, int method, int has_arg, double arg,
                         int qtype, int rounding, void* q, void* scale, void* zero_point,
                         qwx_stream_t stream);

/* qarray.dequantize (qarray.py:692-708): (q - zero_point) * scale in scale_dtype. */
int qwx_dequantize(const void* q, int qtype, int64_t P, int64_t R, int64_t C,
                   int64_t tp, int64_t tr, int64_t tc, const void* scale, int scale_dtype,
                   const void* zero_point, void* out, qwx_stream_t stream);

/* Repack the logical [K, N] codes of a weight into the other GEMM operand order:
 * [K, N] -> [N, K] for 8-bit codes (elem_bytes = 1). */
int qwx_transpose_codes(const void* src, int64_t rows, int64_t cols, void* dst,
                        qwx_stream_t stream);

/* dot_general._fast_dot_general (dot_general.py:135-261) for 2-D operands whose codes
 * are int8 (acc int32, tcgen05 kind::i8) or e4m3 (acc float32, kind::f8f6f4):
 *   out[m, n] = sum_t ( sum_{k in tile t} a[m,k] * b[k,n] ) * sa[m, t] * sb[t, n]
 * a: [M, K] row-major.  b: [K, N] (QWX_B_KN) or [N, K] (QWX_B_NK).
 * k_tile = 0: one scale per row of a / column of b (sa: [M], sb: [N]); otherwise K is cut
 * in tiles of k_tile (a multiple of 128) and sa: [M, K/k_tile], sb: [K/k_tile, N]; a side
 * with sa_tiled/sb_tiled = 0 still has a single scale along K.  sa or sb may be NULL
 * (operand not a QArray).  out_dtype QWX_BF16 / QWX_F32 / QWX_F16, or QWX_S32 with both
 * scales NULL for the raw int32 accumulator.
 * error_flag: optional device int32 that receives a nonzero code if a bounded wait inside
 * the kernel ran out. */
int qwx_gemm_q8(const void* a, const void* b, int code_dtype, int b_layout,
                int64_t M, int64_t N, int64_t K, int64_t k_tile,
                const void* sa, int sa_tiled, const void* sb, int sb_tiled,
                int scale_dtype, void* out, int out_dtype, int epilogue, int32_t* error_flag,
                qwx_stream_t stream);

/* The same product with a caller-provided workspace, for decode-shaped problems (a few rows
 * of activations against a large weight) whose output tiles are fewer than the SMs: K is cut
 * into ranges so that every SM streams a share of the weight, each range writes its partial
 * sums to a slab of the workspace, and once all ranges of a tile are there its CTAs (a
 * cooperative launch: all resident) each add the slabs of a share of the tile's columns in
 * range order, scale and store.  Results are bit-identical to qwx_gemm_q8 for int8 codes and
 * repeatable for e4m3 codes (float32 partial sums are added in a fixed order).
 * qwx_gemm_q8_workspace_bytes returns 0 when the shape would not be cut (the call then
 * behaves exactly like qwx_gemm_q8 and workspace may be NULL).  The workspace opens with
 * two int32 counters per output tile; these must be zero on entry (workspace_is_zero = 0
 * makes the call clear them first) and are left zero on return, so one buffer cleared once
 * serves every call on a stream.  Up to 128 rows against an [N, K] weight with K <= 5120 and
 * enough columns to give at least half of the SMs a 32..256-wide column tile are not cut along
 * K at all (every CTA streams whole weight rows and finishes its own tile): such calls, through
 * either entry point, leave a workspace that was passed untouched.  The reference has no
 * counterpart: XLA picks its own split of the contraction (dot_general.py:253-258 hands it one
 * lax.dot_general). */
size_t qwx_gemm_q8_workspace_bytes(int64_t M, int64_t N, int64_t K);
int qwx_gemm_q8_ws(const void* a, const void* b, int code_dtype, int b_layout,
                   int64_t M, int64_t N, int64_t K, int64_t k_tile,
                   const void* sa, int sa_tiled, const void* sb, int sb_tiled,
                   int scale_dtype, void* out, int out_dtype, int epilogue,
                   void* workspace, size_t workspace_bytes, int workspace_is_zero,
                   int32_t* error_flag, qwx_stream_t stream);

/* An activation quantized on the fly and contracted with a quantized weight: what
 * BoxedParamProvider.dot_general does for a rule with act_qtype set (boxed_param.py:109-171:
 * quantize_act :416-455 with per-token absmax scales, then dot_general.py:135-261), as one
 * call.  a: bf16 [M, K]; wq: int8 or e4m3 codes ([K, N] or [N, K]) with scales sw: bf16 [N];
 * code_dtype is the qtype of both operands.  The codes and scales of a are written to the
 * workspace (scales: bf16 [M] at offset 0; codes: [M, K] at the next multiple of 256 bytes)
 * and are bit-identical to qwx_quantize with one tile per row; the product is bit-identical
 * to qwx_gemm_q8 on them.  workspace: qwx_quant_gemm_q8_workspace_bytes(M, K) bytes,
 * 256-byte aligned. */
size_t qwx_quant_gemm_q8_workspace_bytes(int64_t M, int64_t K);
int qwx_quant_gemm_q8(const void* a, int64_t M, int64_t K, const void* wq, const void* sw,
                      int64_t N, int code_dtype, int b_layout, int rounding, void* out,
                      int out_dtype, int epilogue, void* workspace, size_t workspace_bytes,
                      int32_t* error_flag, qwx_stream_t stream);

/* The same product for at most 32 rows of int8 activations against an int8 weight held
 * [N, K] (the decode step of a served model): a warp-level kernel that streams the weight
 * once with no per-tile set-up.  K a multiple of 256, N of 16.  out_dtype as qwx_gemm_q8
 * (QWX_S32 with both scales NULL for the raw accumulator); int32 partial sums are exact, so
 * the result is bit-identical to qwx_gemm_q8.  workspace: qwx_gemm_q8_skinny_workspace_bytes
 * bytes, zero on entry (workspace_is_zero = 0 clears it first), left zero.  The reference
 * has no counterpart: XLA picks its own kernel for the shape. */
size_t qwx_gemm_q8_skinny_workspace_bytes(int64_t M, int64_t N);
int qwx_gemm_q8_skinny(const void* a, const void* w, int64_t M, int64_t N, int64_t K,
                       const void* sa, const void* sb, int scale_dtype, void* out, int out_dtype,
                       int epilogue, void* workspace, size_t workspace_bytes,
                       int workspace_is_zero, qwx_stream_t stream);

/* The same product for the decode step of a served model: at most 128 rows of int8 activations
 * against an int8 weight held [N, K], on the tensor cores with the operands swapped (128 output
 * channels are the tcgen05.mma's M, the tokens its N), the (channel tile, K stage) units dealt
 * to the SMs in equal contiguous runs so that every SM streams the same share of the weight.
 * Tiles shared by several CTAs are summed with exact int32 atomics in the workspace; the CTA
 * that adds last scales, stores and clears, and nobody waits for another CTA.  K a multiple of
 * 16.  out_dtype as qwx_gemm_q8 (QWX_S32 with both scales NULL for the raw accumulator); the
 * result is bit-identical to qwx_gemm_q8.  workspace: qwx_gemm_q8_decode_workspace_bytes bytes,
 * 16-byte aligned, zero on entry (workspace_is_zero = 0 clears it first), left zero.  The
 * reference has no counterpart: XLA picks its own kernel for the shape
 * (dot_general.py:253-258 hands it one lax.dot_general). */
size_t qwx_gemm_q8_decode_workspace_bytes(int64_t M, int64_t N);
int qwx_gemm_q8_decode(const void* a, const void* w, int64_t M, int64_t N, int64_t K,
                       const void* sa, const void* sb, int scale_dtype, void* out, int out_dtype,
                       int epilogue, void* workspace, size_t workspace_bytes,
                       int workspace_is_zero, int32_t* error_flag, qwx_stream_t stream);

/* The general dequantize-on-output contraction of dot_general._fast_dot_general
 * (dot_general.py:135-261): scales that change along K (sub-channel quantization, the tiled
 * contracting axis of :187-203 and the tile sum of :259) and the zero-point correction of an
 * asymmetric operand (:228-253), all inside one kernel:
 *   out[m, n] = sum_t ( acc_t[m, n] - corr_row[m, t] * corr_col[t, n] ) * sa[m, t] * sb[t, n]
 * with acc_t the integer (or float32, for e4m3 codes) dot over K tile t.  T = K / k_tile tiles;
 * k_tile is a multiple of 128, or 0 / K for a single tile.  sa: [M, T] if sa_tiled else [M];
 * sb: [T, N] if sb_tiled else [N]; either may be NULL.  corr_row [M, T] and corr_col [T, N]
 * are int32 and given together or not at all (int8 codes only):
 *   asymmetric a (zero point za[m, t]):  corr_row = za,           corr_col = column sums of b
 *   asymmetric b (zero point zb[t, n]):  corr_row = row sums of a, corr_col = zb
 * the sums taken over each K tile (qwx_code_sums).  out_dtype QWX_BF16 / QWX_F32 / QWX_F16.
 * qwx_gemm_q8 forwards here when k_tile cuts K. */
int qwx_gemm_q8_tiled(const void* a, const void* b, int code_dtype, int b_layout,
                      int64_t M, int64_t N, int64_t K, int64_t k_tile,
                      const void* sa, int sa_tiled, const void* sb, int sb_tiled,
                      int scale_dtype, const int32_t* corr_row, const int32_t* corr_col,
                      void* out, int out_dtype, int epilogue, int32_t* error_flag,
                      qwx_stream_t stream);

/* Sums of int8 codes over each K tile, the integer dot of the other operand with a broadcast
 * zero point (dot_general.py:233, :246) reduced to what it is: a row or column sum.
 * k_axis = 1: codes [rows, cols = K]; k_axis = 0: codes [rows = K, cols].  k_tile = 0 means K.
 * out is int32 [T, other] if t_major else [other, T], other being the non-K extent. */
int qwx_code_sums(const void* codes, int64_t rows, int64_t cols, int k_axis, int64_t k_tile,
                  int t_major, int32_t* out, qwx_stream_t stream);

/* MXFP8 block-scaled GEMM: what dot_general computes when both operands are "mxfp8" QArrays
 * (qwix/_src/core/mxfp_dot.py:24-79, jax.nn.scaled_matmul in the reference):
 *   out[m, n] = sum_j ( sum_{k in 32-wide block j} a[m, k] * b[k, n] ) * sa[m, j] * sb[j, n]
 * a [M, K] and b ([K, N] for QWX_B_KN, [N, K] for QWX_B_NK) hold e4m3 codes, the scales are
 * powers of two, accumulation is float32 inside tcgen05.mma.kind::mxf8f6f4.block_scale.
 * K must be a multiple of 128 (QWX_ERR_UNSUPPORTED otherwise: dequantize instead).
 *
 * The kernel reads the scales as E8M0 bytes in its own staging order; qwx_mx_pack_scales
 * produces that from a QArray's scale array (operand 0 = a: scale [rows = M, K / 32];
 * operand 1 = b: scale [rows = N, K / 32], or [K / 32, N] with k_major = 1), once per weight
 * and once per activation.  qwx_mx_scales_packed_bytes gives the size of `out` (0 for
 * arguments the GEMM would refuse). */
size_t qwx_mx_scales_packed_bytes(int operand, int64_t rows, int64_t K);
int qwx_mx_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows, int64_t K,
                       int k_major, void* out, size_t out_bytes, qwx_stream_t stream);
int qwx_gemm_mx8(const void* a, const void* b, int b_layout, int64_t M, int64_t N, int64_t K,
                 const void* sfa_packed, const void* sfb_packed, void* out, int out_dtype,
                 int32_t* error_flag, qwx_stream_t stream);

/* MXFP4 block-scaled GEMM: the same contraction for two "mxfp4" QArrays (e2m1 codes: sign,
 * two exponent bits, one significand bit; values 0, 0.5, 1, 1.5, 2, 3, 4, 6), through
 * tcgen05.mma.kind::mxf4.block_scale.  The kernel takes both operands K-major with two codes
 * per byte, the even K index in the low nibble: a_packed [M, K / 2], b_packed [N, K / 2].
 * qwx_mx4_pack_codes makes that from a QArray's codes (one per byte, low nibble): rows x K, or
 * K x rows with k_major = 1 (a [K, N] weight).  K must be a multiple of 256
 * (QWX_ERR_UNSUPPORTED otherwise).  Scales as for MXFP8, packed by qwx_mx4_pack_scales. */
size_t qwx_mx4_scales_packed_bytes(int operand, int64_t rows, int64_t K);
int qwx_mx4_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows, int64_t K,
                        int k_major, void* out, size_t out_bytes, qwx_stream_t stream);
int qwx_mx4_pack_codes(const void* codes, int64_t rows, int64_t K, int k_major, void* out,
                       qwx_stream_t stream);
int qwx_gemm_mx4(const void* a_packed, const void* b_packed, int64_t M, int64_t N, int64_t K,
                 const void* sfa_packed, const void* sfb_packed, void* out, int out_dtype,
                 int32_t* error_flag, qwx_stream_t stream);

/* NVFP4 block-scaled GEMM: two "nvfp4" QArrays (e2m1 codes, one scale per 16 contracted
 * elements whose value is an e4m3 number: qarray.py:580-581), through
 * tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X.  Codes packed as for MXFP4
 * (qwx_mx4_pack_codes); the scales (scale [rows, K / 16], or [K / 16, rows] with k_major = 1)
 * are laid out as e4m3 bytes by qwx_nvfp4_pack_scales.  K a multiple of 256. */
size_t qwx_nvfp4_scales_packed_bytes(int operand, int64_t rows, int64_t K);
int qwx_nvfp4_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows, int64_t K,
                          int k_major, void* out, size_t out_bytes, qwx_stream_t stream);
int qwx_gemm_nvfp4(const void* a_packed, const void* b_packed, int64_t M, int64_t N, int64_t K,
                   const void* sfa_packed, const void* sfb_packed, void* out, int out_dtype,
                   int32_t* error_flag, qwx_stream_t stream);

/* Element-wise stages of a Llama-style decoder layer fused with the per-token int8
 * quantization of the next projection's activation.  The quantization half is
 * qarray.quantize with per-token absmax scales (qarray.py:638-644; the activation side of
 * boxed_param.py:416-455): scale[row] = bf16(absmax / 127.5) (1 below 2^-63), codes by the
 * strict recipe.  The element-wise halves (RMSNorm, SwiGLU, rotary embedding, KV-cache
 * write) are model code and have no counterpart in qwix; every rounding of their unfused
 * bf16/float32 composition is kept.  All tensors bf16, row-major; q int8; scale bf16 [rows].
 *
 * qwx_add_rmsnorm_quantize: x' = bf16(x + delta) (delta may be NULL: x' = x), written to x_out
 *   when delta is given; y = bf16((f32(x') * rsqrt(mean(x'^2) + eps)) * f32(weight)); y_out
 *   and/or (q, scale) receive the result.  d a multiple of 8, at most 8192.
 * qwx_silu_mul_quantize: gu is [rows, 2 f] = [gate | up]; y = bf16(bf16(silu(gate)) * up).
 * qwx_rope_cache: qkv [B, T, (hq + 2 hkv) * hd]; heads are rotated with the float32 tables
 *   cos/sin [positions, hd / 2] at position pos + t (pos_dev, a device int64, replaces pos
 *   when not NULL: the form a CUDA graph can replay); q goes to q_out [B, T, hq, hd], k and v
 *   to cache_k / cache_v [B, hkv, S, hd] views with the given batch and head strides
 *   (elements) at sequence index pos + t. */
int qwx_add_rmsnorm_quantize(const void* x, const void* delta, const void* weight, double eps,
                             int64_t rows, int64_t d, void* x_out, void* y_out, void* q,
                             void* scale, qwx_stream_t stream);
/* qwx_add_rmsnorm_quantize with the all-reduce of a row-parallel projection folded in: delta
 * is the sum over `world` ranks of bf16 partial outputs that every rank keeps in a buffer the
 * other ranks have mapped (partials[r], flags[r]: rank r's buffers as mapped in this process,
 * e.g. through CUDA IPC / symmetric memory over NVLink).  The kernel reads the partials with
 * peer loads, adds them in rank order in float32 and rounds once to bf16 (what an all-reduce
 * delivers), then proceeds as above.  flags[r]: int32 [max_ctas][world], zero before the first
 * call on every rank; launches: this rank's int32 [max_ctas], zero before the first call.
 * Every rank must make the same sequence of calls with the same rows, and a partial buffer
 * may be rewritten only after one further call of this function (callers alternate two
 * buffers).  The grid is min(rows, max_ctas, CTAs the device keeps resident), so that every
 * hand-shaking CTA is running while it waits; ranks must sit on identical GPUs.  The hand-shake
 * is bounded by wait_cycles SM clocks (<= 0: the default of 4e9, about two seconds): ranks must
 * enter the call within that budget of each other.  If a peer never arrives the call reports
 * QWX_ERR_DEVICE_WAIT through error_flag and writes none of its outputs.  No counterpart in the
 * reference (GSPMD inserts the all-reduce there, flax_util.py:354-357). */
int qwx_add_rmsnorm_quantize_peer(const void* x, const void* const* partials, void* const* flags,
                                  int world, int rank, int* launches, int max_ctas,
                                  const void* weight, double eps, int64_t rows, int64_t d,
                                  void* x_out, void* y_out, void* q, void* scale,
                                  int32_t* error_flag, int64_t wait_cycles, qwx_stream_t stream);
/* The all-reduce of such partials on its own, in place, for many rows (a prefill chunk): rank
 * r sums its share of the rows over all ranks' buffers (float32, rank order, one rounding to
 * bf16) and writes the sums into the same rows of every rank's buffer with plain peer stores,
 * so (world - 1) / world of the tensor crosses NVLink in each direction instead of
 * (world - 1) x the tensor inbound.  When the call has completed on a rank, that rank's buffer
 * [rows, d] holds the reduced tensor (what an all-reduce delivers), for an ordinary local
 * consumer such as qwx_add_rmsnorm_quantize.  partials[r] / flags[r]: rank r's buffers as
 * mapped in this process; flags[r]: int32 [(max_ctas + 1) * world], launches: int32
 * [max_ctas + 2], all zero before the first call; every rank makes the same sequence of calls
 * with the same rows.  Waits are bounded by wait_cycles (<= 0: about two seconds); if a peer
 * never arrives the call reports QWX_ERR_DEVICE_WAIT through error_flag.  No counterpart in the
 * reference (GSPMD inserts the all-reduce there, flax_util.py:354-357). */
int qwx_peer_allreduce(void* const* partials, void* const* flags, int world, int rank,
                       int* launches, int max_ctas, int64_t rows, int64_t d, int32_t* error_flag,
                       int64_t wait_cycles, qwx_stream_t stream);
int qwx_silu_mul_quantize(const void* gu, int64_t rows, int64_t f, void* y_out, void* q,
                          void* scale, qwx_stream_t stream);
/* Greedy sampling over the logits a (column-parallel) lm_head projection produced: for every
 * row of x (bf16 [rows, cols]) the largest value (best_value, float32 [rows], may be NULL) and
 * index_offset + its lowest index (best_index, int64 [rows]); a positive NaN counts as the
 * largest value.  index_offset is the first vocabulary entry of this rank's shard.  Model code
 * like the stages above (no counterpart in qwix).  workspace: qwx_argmax_rows_workspace_bytes
 * bytes, 16-byte aligned, its first rows * 4 bytes zero on entry and left zero. */
size_t qwx_argmax_rows_workspace_bytes(int64_t rows, int64_t cols);
int qwx_argmax_rows(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t index_offset,
                    float* best_value, int64_t* best_index, void* workspace,
                    size_t workspace_bytes, qwx_stream_t stream);
int qwx_rope_cache(const void* qkv, int64_t B, int64_t T, int hq, int hkv, int hd,
                   const float* cos_t, const float* sin_t, int64_t pos, const int64_t* pos_dev,
                   void* q_out, void* cache_k, void* cache_v, int64_t cache_batch_stride,
                   int64_t cache_head_stride, qwx_stream_t stream);

/* Weight-only int4 GEMM, the fused form of dot_general._slow_dot_general
 * (dot_general.py:264-275, chosen at :444-452 when the activation is not quantized):
 *   out[m, n] = sum_k a[m, k] * ( q[k, n] * scale[k / k_tile, n] )
 * with the code products summed exactly per 128 K and the scale applied in float32.  For
 * float32 scales this is the reference's dequantized weight (q * s is exact in float32); for
 * bf16 scales the reference rounds q * s to bf16, which is not reproduced (the result is
 * closer to the unquantized product, inside the output tolerance).
 * a: bf16 [M, K], M <= 128 (the weight is streamed once per 32 tokens).  The weight is given
 * in the kernel's streaming layout, made once by qwx_pack_w4 from the logical codes q[K, N]
 * (QWX_S4U, one code per byte): 1 KB chunks of 16 channels x 128 K, ordered [N / 16][K / 128],
 * each lane's 2 x 16 bytes holding its tensor-core fragment values.  scale: [K / k_tile, N]
 * in f32 or bf16, k_tile a multiple of 128.  K must be a multiple of 128, N of 16.
 * out: bf16 or f32 [M, N].
 * workspace: qwx_gemm_a16w4_workspace_bytes(M, N) bytes that must be zero when the kernel
 * starts; the kernel leaves them zero.  workspace_is_zero = 0 makes the call clear it first.
 * error_flag is accepted for symmetry with the other GEMMs; this kernel has no device-side
 * waits and never writes it. */
size_t qwx_w4_packed_bytes(int64_t K, int64_t N);
int qwx_pack_w4(const void* q, int64_t K, int64_t N, void* packed, qwx_stream_t stream);
size_t qwx_gemm_a16w4_workspace_bytes(int64_t M, int64_t N);
int qwx_gemm_a16w4(const void* a, const void* w_packed, const void* scale, int scale_dtype,
                   int64_t M, int64_t N, int64_t K, int64_t k_tile, void* out, int out_dtype,
                   void* workspace, size_t workspace_bytes, int workspace_is_zero,
                   int32_t* error_flag, qwx_stream_t stream);

/* The same contraction on the tcgen05 tensor cores, for batches the warp-level kernel above
 * would stream the weight several times for (33 tokens and more; M <= 128 per call):
 *   out[m, n] = sum_k a[m, k] * bf16( q[k, n] * scale[k / k_tile, n] )
 * The codes are unpacked and scaled into shared memory as bfloat16 and contracted with the
 * activation in one float32 accumulation over all of K.  With bf16 scales that is the
 * reference's arithmetic (dequantize to the scale dtype, qarray.py:692-708, then a bf16 dot with
 * float32 accumulation, dot_general.py:264-275); with float32 scales the reference keeps q * s in
 * float32 and this kernel rounds it once to bfloat16.
 * w_tiles: the weight in this kernel's layout, made once by qwx_pack_w4_tiles from the logical
 * codes q[K, N] (QWX_S4U): [N / 128][K / 128][4 quarters of 32 K][128 channels][16 bytes].  K a multiple of 128;
 * scale [K / k_tile, N] in f32 or bf16, k_tile a multiple of 128; out bf16 or f32 [M, N].
 * workspace: qwx_gemm_a16w4_mma_workspace_bytes(M, N) bytes, zero on entry, left zero (partial
 * sums of channel tiles that several CTAs share, added with float32 atomics: the order of those
 * additions, and with it the last bits of such tiles, can differ between runs).
 * error_flag receives QWX_ERR_DEVICE_WAIT if a bounded device-side wait runs out. */
size_t qwx_w4_tiles_packed_bytes(int64_t K, int64_t N);
int qwx_pack_w4_tiles(const void* q, int64_t K, int64_t N, void* packed, qwx_stream_t stream);
size_t qwx_gemm_a16w4_mma_workspace_bytes(int64_t M, int64_t N);
int qwx_gemm_a16w4_mma(const void* a, const void* w_tiles, const void* scale, int scale_dtype,
                       int64_t M, int64_t N, int64_t K, int64_t k_tile, void* out, int out_dtype,
                       void* workspace, size_t workspace_bytes, int workspace_is_zero,
                       int32_t* error_flag, qwx_stream_t stream);

/* Blockwise Hadamard rotation, the arithmetic of qwix/contrib/hadamard_rot.py:35-117 with the
 * Sylvester matrix H of size `block` (= 128) and optional +/-1 sign vectors (int8, one entry
 * per index of the rotated axis; `signs_in` is applied before H, `signs_out` after it, as in
 * contrib/kernels/fused_hadamard_quantized_matmul.py:150-160).  x: bf16 [R, C].
 *   axis = 1: out = x . H per `block` columns               (_apply_hadamard_lhs, :99-106)
 *   axis = 0: out = H . x / block per `block` rows          (_apply_hadamard_rhs, :109-117;
 *             contrib/kernels/fused_hadamard_quantized_matmul.py:443-478) */
int qwx_hadamard_rotate(const void* x, int x_dtype, int64_t R, int64_t C, int axis, int block,
                        const int8_t* signs_in, const int8_t* signs_out, void* out,
                        qwx_stream_t stream);

/* Rotate (axis = 1) and quantize in one pass over x: bf16 [rows, K] -> codes [rows, K] (QWX_S8
 * or QWX_E4M3) with one absmax scale per row (bf16 [rows]); the fused form of
 * contrib/kernels/fused_hadamard_quantize.py:43-119 and of `quantize_a_tile`
 * (fused_hadamard_quantized_matmul.py:50-56) for whole-row tiles.  K <= 8192. */
int qwx_hadamard_quantize(const void* x, int x_dtype, int64_t rows, int64_t K, int block,
                          const int8_t* signs_in, const int8_t* signs_out, int qtype,
                          int rounding, void* q, void* scale, qwx_stream_t stream);

/* The Hadamard-quantized matmul (`hadamard_quantize_multiply`,
 * fused_hadamard_quantized_matmul.py:349-414): a bf16 [M, K] is rotated and quantized per row,
 * then contracted with the already rotated and quantized weight wq ([K, N] or [N, K] codes of
 * code_dtype, scales sw [N] bf16) on the tensor cores, scales applied in the epilogue.
 * workspace: qwx_hadamard_gemm_workspace_bytes(M, K) bytes, 256-byte aligned. */
size_t qwx_hadamard_gemm_workspace_bytes(int64_t M, int64_t K);
int qwx_hadamard_gemm(const void* a, int64_t M, int64_t K, const int8_t* signs_in,
                      const int8_t* signs_out, const void* wq, const void* sw, int64_t N,
                      int code_dtype, int b_layout, int rounding, void* out, int out_dtype,
                      int epilogue, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                      qwx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QWIX_B200_H_ */
