/*
 * fpq_b200 -- C ABI of the B200 (sm_100a) MR-GPTQ hot-path library.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream
 * (cudaStream_t passed as void*), launches on that stream without synchronising,
 * allocates nothing (the caller owns inputs, outputs and workspaces) and returns
 * FPQ_OK or a negative status; fpq_last_error() gives the text of the calling
 * thread's last failure.  Citations name the file and lines of IST-DASLab/FP-Quant
 * whose behaviour the entry point replaces.
 */
#ifndef FPQ_B200_H_
#define FPQ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define FPQ_OK 0
#define FPQ_ERR_INVALID_ARGUMENT (-1)
#define FPQ_ERR_CUDA (-2)
#define FPQ_ERR_UNSUPPORTED_DEVICE (-3)
#define FPQ_ERR_DEVICE_TIMEOUT (-4)
#define FPQ_ERR_NOT_POSITIVE_DEFINITE (-5)

/* element formats */
#define FPQ_FMT_MXFP4 0 /* E2M1 codes, one E8M0 scale per 32 elements */
#define FPQ_FMT_NVFP4 1 /* E2M1 codes, one E4M3 scale per 16 elements + fp32 tensor scale */
#define FPQ_FMT_MXFP8 3 /* E4M3 bytes, one E8M0 scale per 32 elements: operands of fpq_gemm_mxf8 only */

/* tensor dtypes */
#define FPQ_DT_BF16 0
#define FPQ_DT_F32 1

/* layouts of the scale bytes */
#define FPQ_SCALES_ROWMAJOR 0 /* [rows, cols/g] */
#define FPQ_SCALES_SWIZZLED 1 /* 128x4 tiles, padded to [ceil(rows/128)*128, ceil(cols/g/4)*4] */

/* what fpq_apply_scales writes */
#define FPQ_OUT_CODES 0      /* packed E2M1 codes, uint8 [rows, cols/2] */
#define FPQ_OUT_GRID 1       /* E2M1 grid values in the dtype of x */
#define FPQ_OUT_DEQUANT 2    /* grid value * scale in the dtype of x */
#define FPQ_OUT_DEQUANT_STE 3 /* fl(x + fl(grid*scale - x)), the value `Quantizer.__call__` returns */

typedef void* fpq_stream_t;

int fpq_version(void);
const char* fpq_last_error(void);

/* FPQ_OK when `device` is a compute-capability 10.0 GPU. */
int fpq_check_device(int device);

/*
 * Block-Hadamard rotation of every contiguous `group` (16/32/64/128) elements of
 * the last dim: fp32 butterfly, pair distances 1,2,..,group/2, then * fl32(1/sqrt(group)).
 * Replaces HadamardTransform.forward (src/transforms/transforms.py:81-84) and its
 * external `fast_hadamard_transform` kernel.  x, y: [rows, cols]; y may alias x
 * when the dtypes match.
 */
int fpq_rotate_hadamard(const void* x, int dtype_in, void* y, int dtype_out, int64_t rows,
                        int64_t cols, int group, fpq_stream_t stream);

/*
 * y = x.view(-1, g) @ matrix for an arbitrary g x g rotation (g in 16/32/64/128),
 * fp32 sequential accumulation over k.  Covers the identity / GSR / user matrices
 * that `forward_quantize` accepts (inference_lib/src/fp_quant/module/linear_fns.py:27-50,
 * linear.py:37-41).  matrix: fp32 [g, g] row-major.
 */
int fpq_rotate_dense(const void* x, int dtype_in, void* y, int dtype_out, int64_t rows,
                     int64_t cols, int group, const float* matrix, fpq_stream_t stream);

/*
 * Tensor-wide max |rotate(x)| folded into *absmax_bits with an unsigned atomic max on
 * the fp32 bit pattern (the caller zeroes it first).  First half of the NVFP4 global
 * scale (src/quantization/quantizer.py:146).  hadamard_group 0 = no rotation.
 */
int fpq_absmax(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
               uint32_t* absmax_bits, fpq_stream_t stream);

/*
 * *global_scale = min(*global_scale, fl(2688 * fl(1 / absmax))) -- the running-min
 * update of Quantizer.global_scale (src/quantization/quantizer.py:10-16, :145-150).
 * A zero absmax leaves the scale unchanged and sets *status to 1.
 */
int fpq_global_scale_update(const uint32_t* absmax_bits, float* global_scale, int32_t* status,
                            fpq_stream_t stream);

/*
 * Fused rotate + micro-scaled FP4 quantise: the one memory-bound pass that replaces
 * Quantizer.get_quantization_params + quantize + pack_fp4_to_uint8 + cast_scales_to_eXmY
 * (src/quantization/quantizer.py:87-182, quant_ops.py:31-40, :57-71, :82-94, :111-118),
 * qutlass.fusedQuantizeMx / fusedQuantizeNv and the `to_blocked` re-layout
 * (inference_lib/src/fp_quant/module/qutlass_ops.py:36-105, :122-123, :334-335).
 *   x            [rows, cols] bf16 or fp32, cols % 32 == 0 and cols % hadamard_group == 0
 *   hadamard_group 0 (none), 16, 32, 64 or 128
 *   global_scale device fp32[1], NVFP4 only (NULL for MXFP4)
 *   codes        uint8 [rows, cols/2] or NULL
 *   scale_bytes  uint8 in `scale_layout` or NULL; in the swizzled layout the kernel also zeroes the
 *                bytes of the pad rows (rows .. next multiple of 128); the caller zero-fills the
 *                buffer only when (cols/g) % 4 != 0 (pad columns)
 *   scales_f32   fp32 [rows, cols/g] (the divisor actually used) or NULL
 */
int fpq_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                 int format, const float* global_scale, uint8_t* codes, uint8_t* scale_bytes,
                 int scale_layout, float* scales_f32, fpq_stream_t stream);

/*
 * fpq_quantize of the tensor `silu(gate) * up` without materialising it: the input of an MLP's down-projection,
 * which the reference computes, rotates and quantises in separate passes over memory
 * (src/utils/llama_utils.py:62-70: `x = self.act_fn(gate) * up`, `down_in_transform(x)`, then the activation
 * quantiser of `down_proj`; in the inference library the same tensor reaches FPQuantLinear.forward of the
 * down-projection, inference_lib/src/fp_quant/module/linear.py:250-368).  The reference's rounding points are
 * kept: silu evaluated in fp32 as x / (1 + exp(-x)) and rounded to bf16, the product rounded to bf16, then
 * rotation and quantisation in fp32 as in fpq_quantize.  gate, up: bf16 [rows, cols]; other arguments and
 * constraints as for fpq_quantize (codes and scale_bytes are both required).
 */
int fpq_quantize_silu_mul(const void* gate_bf16, const void* up_bf16, int64_t rows, int64_t cols, int hadamard_group,
                          int format, const float* global_scale, uint8_t* codes, uint8_t* scale_bytes,
                          int scale_layout, fpq_stream_t stream);

/*
 * Fused rotate + quantise + dequantise ("pseudo-quantisation"): y = grid(code) * scale
 * (or the straight-through form when ste != 0), same dtype as x.  Replaces the Triton
 * kernels mxfp4_forward_kernel / nvfp4_forward_kernel
 * (inference_lib/src/fp_quant/module/triton/mxfp4.py:19-119, nvfp4.py:19-106) with the
 * rounding rule of Quantizer.__call__ (src/quantization/quantizer.py:190-197).
 */
int fpq_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                      int format, const float* global_scale, void* y, int ste,
                      fpq_stream_t stream);

/*
 * The forward_method = "quest" variant of the MXFP4 quantise (the default method of FPQuantConfig,
 * inference_lib/src/fp_quant/utils/config.py:20; qutlass.fusedQuantizeMx(method="quest"),
 * inference_lib/src/fp_quant/module/qutlass_ops.py:36-71; its only in-tree statement is the Triton kernel
 * inference_lib/src/fp_quant/module/triton/mxfp4.py:51-59, :105-110).  Per group of 32 rotated values:
 * std = sqrt(mean(x^2) - mean(x)^2), scale = (2.92247856 / 6) * std + 1e-8, divisor 2^floor(log2(scale)),
 * stored E8M0 byte = that exponent + 127 (the tensor scale of this method is 1, linear.py:190-196); codes are
 * E2M1 round-to-nearest-even of x / divisor, saturating at +-6.  clip_mask (optional): uint8 [rows, cols/8],
 * bit i of byte b set when element 8 b + i was inside the grid's range (|x / divisor| < 6), the packing
 * `_unpack_mask` reads (linear_fns.py:66-76).  Other arguments as for fpq_quantize.
 */
int fpq_quantize_quest(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group, uint8_t* codes,
                       uint8_t* scale_bytes, int scale_layout, uint8_t* clip_mask, fpq_stream_t stream);

/*
 * Pseudo-quantisation with the QuEST scale rule: y = grid(code) * divisor in the dtype of x, clip_mask
 * (optional) one byte per element, 1 = inside the range.  Replaces mxfp4_forward_kernel with quest=True
 * (inference_lib/src/fp_quant/module/triton/mxfp4.py:19-119; pseudoquant_linear_fns.py:19-34) up to its
 * rounding of exact ties (the Triton kernel rounds them toward zero, this rounds to even).
 */
int fpq_fake_quantize_quest(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group, void* y,
                            uint8_t* clip_mask, fpq_stream_t stream);

/*
 * Quantise with scales given by the caller: Quantizer.quantize / dequantize / __call__
 * (src/quantization/quantizer.py:175-197).  scales: fp32 [rows, cols/group]; `group` any
 * divisor of cols (1 = one scale per element); cols % 8 == 0; out_kind one of FPQ_OUT_*.
 */
int fpq_apply_scales(const void* x, int dtype, int64_t rows, int64_t cols, const float* scales,
                     int group, int out_kind, void* out, fpq_stream_t stream);

/*
 * The MSE observer of Quantizer.get_quantization_params (src/quantization/quantizer.py:117-134): per
 * group, `iters` candidate scales fl(f_i * s0), f_i = 1 - i * max_shrink / iters, s0 = fl(fl(2 absmax)/12);
 * the one with the smallest sum |x - dequant(quant(x, s))| ^ error_norm (first strictly smaller wins) goes
 * through the scale-precision chain (E4M3 with the tensor scale, or E8M0).  x [rows, cols] bf16 or fp32
 * (already rotated), cols % 32 == 0; scales_f32 [rows, cols/g] receives the divisors.  The reference's
 * defaults are iters 100, max_shrink 0.8, error_norm 2.4.  global_scale: device fp32[1], NVFP4 only.
 */
int fpq_mse_scales(const void* x, int dtype, int64_t rows, int64_t cols, int format,
                   const float* global_scale, int iters, double max_shrink, float error_norm,
                   float* scales_f32, fpq_stream_t stream);

/*
 * pack_fp4_to_uint8 (src/quantization/quant_ops.py:31-40): tensor of E2M1 grid values ->
 * two 4-bit codes per byte, even element in the low nibble, zeros as 0x8.
 */
int fpq_pack_grid(const void* q, int dtype, int64_t rows, int64_t cols, uint8_t* packed,
                  fpq_stream_t stream);

/*
 * Row-major scale bytes [rows, sf_cols] -> zero-padded 128x4-tile layout.  Replaces
 * qutlass.utils.to_blocked (inference_lib/src/fp_quant/module/qutlass_ops.py:334-335).
 */
int fpq_swizzle_scales(const uint8_t* rowmajor, int64_t rows, int64_t sf_cols, uint8_t* swizzled,
                       fpq_stream_t stream);

/*
 * Y[M,N] (bf16) = alpha * dq(A)[M,K] * dq(B)[N,K]^T (+ bias[N]) on the tcgen05 tensor cores,
 * A and B as packed E2M1 codes [rows, K/2] (K-major), scales in the swizzled layout.
 * Replaces matmul_mxf4_bf16_tn_op / matmul_nvf4_bf16_tn_op and the per-call `to_blocked`
 * (inference_lib/src/fp_quant/module/qutlass_ops.py:111-168) and `forward_gemm`
 * (inference_lib/src/fp_quant/module/linear_fns.py:53-64).  alpha: device fp32[1];
 * bias: device bf16[N] or NULL; K % 64 == 0, N % 8 == 0.
 * error_flag: device int32 the caller zeroes; set to 1 if a bounded in-kernel wait ran out
 * (the output is then invalid; the context stays usable).
 */
int fpq_gemm_fp4(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* a_scales_swizzled,
                 const uint8_t* b_scales_swizzled, const float* alpha, const void* bias_bf16,
                 void* out_bf16, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                 fpq_stream_t stream);

/*
 * Y[M,N] (bf16) = alpha * dq(A)[M,K] * dq(B)[N,K]^T on the tcgen05 tensor cores (kind::mxf8f6f4, CTA pairs),
 * A and B as E4M3 bytes [rows, K] (K-major), one E8M0 scale per 32 elements along K in the swizzled
 * layout (as fpq_swizzle_scales writes it).  Replaces matmul_mxf8_bf16_tn_op and its per-call `to_blocked`
 * (inference_lib/src/fp_quant/module/qutlass_ops.py:171-189), the GEMM of the MXFP8 backward pass
 * (linear_fns.py:311-318).  alpha: device fp32[1]; K % 32 == 0, K % 16 == 0 bytes, N % 8 == 0.
 * error_flag as in fpq_gemm_fp4.
 */
int fpq_gemm_mxf8(const uint8_t* a_e4m3, const uint8_t* b_e4m3, const uint8_t* a_scales_swizzled,
                  const uint8_t* b_scales_swizzled, const float* alpha, void* out_bf16, int64_t M, int64_t N,
                  int64_t K, int32_t* error_flag, fpq_stream_t stream);

/*
 * bf16 [rows, cols] -> MXFP8 with one E8M0 scale per 32 x 32 square, so that the same E4M3 bytes serve a GEMM
 * that contracts over the columns (row_scales [rows_pad, cols/32]) and one that contracts over the rows
 * (col_scales [cols, rows_pad/32]); rows_pad = rows rounded up to 128, the padding rows are written as
 * zeros.  Stands for backward_bf16_square_double_mxfp8 (qutlass_ops.py:277-304; QuTLASS itself is not
 * available, so the arithmetic is this library's: scale 2^(floor(log2(max|x|)) - 8), byte 0 for an all-zero
 * square, x / scale clamped to +-448 and rounded to nearest even).  out_e4m3: [rows_pad, cols] bytes;
 * out_t_e4m3 (optional, may be NULL): the same bytes transposed, [cols, rows_pad], for the GEMM that
 * contracts over the rows.  scale_layout: FPQ_SCALES_ROWMAJOR, or FPQ_SCALES_SWIZZLED to write both scale
 * tensors in the layout the GEMM reads (buffers of the padded size; bytes of the padding are not written:
 * zero them once).  cols % 32 == 0.
 */
int fpq_quantize_mxfp8_square(const void* x_bf16, int64_t rows, int64_t cols, uint8_t* out_e4m3,
                              uint8_t* out_t_e4m3, uint8_t* row_scales, uint8_t* col_scales, int scale_layout,
                              fpq_stream_t stream);

/*
 * MXFP4 [rows, cols] (packed codes [rows, cols/2], row-major E8M0 bytes [rows, cols/32]) -> its transpose
 * as MXFP8: out_e4m3 [cols, rows_pad] bytes, out_scales [cols, rows_pad/32] E8M0 bytes, rows_pad = rows
 * rounded up to 128 (padding zero).  Stands for mxfp4_transpose_mxfp8 (qutlass_ops.py:307-330; arithmetic
 * defined here): a 32 x 32 square takes 2^(emax - 6), emax the largest of its 32 source exponents, and an
 * element becomes fp4 * 2^(e_row - emax + 6), exact unless its row lies more than 2^-14 below the largest
 * (then rounded to nearest even on the E4M3 grid).  scale_layout as for fpq_quantize_mxfp8_square (it
 * applies to out_scales; the input scales are always row-major).  cols % 32 == 0.
 */
int fpq_mxfp4_transpose_mxfp8(const uint8_t* codes, const uint8_t* scales_rowmajor, int64_t rows, int64_t cols,
                              uint8_t* out_e4m3, uint8_t* out_scales, int scale_layout, fpq_stream_t stream);

/*
 * MXFP4 [rows, cols] (packed codes, row-major E8M0 bytes [rows, cols/32]) -> bf16 [cols, rows]: the transpose
 * of the dequantised tensor, every element divided by *alpha (device fp32[1]: the tensor scale the operand
 * was quantised under) and rounded once to bf16.  First half of backward_qt_bf16 (qutlass_ops.py:248-274:
 * dequantise, transpose, rotate, quantise again); the second half is fpq_quantize on the result.
 * out_ld: row stride of the output in elements (>= rows; columns [rows, out_ld) are not written, so a caller
 * that needs the contraction axis padded passes a zeroed buffer).  cols % 32 == 0.
 */
int fpq_mxfp4_transpose_dequant(const uint8_t* codes, const uint8_t* scales_rowmajor, int64_t rows, int64_t cols,
                                const float* alpha, void* out_bf16, int64_t out_ld, fpq_stream_t stream);

/*
 * MXFP4 of the TRANSPOSE of a bf16 matrix without materialising it: x [t_rows, n] row-major -> codes
 * [n, t_pad/2] and E8M0 scale bytes of x^T, rotated (Hadamard group 0, 16 or 32) and scaled along the t axis;
 * rows of x beyond t_rows count as zero (t_pad >= t_rows, a multiple of 32).  Same arithmetic as
 * fpq_quantize on the transposed copy.  Stands for backward_t_bf16 (qutlass_ops.py:218-245): the upstream
 * gradient as the operand of the weight-gradient GEMM, which contracts over the tokens.  n % 8 == 0.
 */
int fpq_quantize_transposed(const void* x_bf16, int64_t t_rows, int64_t n, int64_t t_pad, int hadamard_group,
                            uint8_t* codes, uint8_t* scale_bytes, int scale_layout, fpq_stream_t stream);

/*
 * Column-parallel form of fpq_gemm_fp4 for tensor parallelism over NVLink (no counterpart in the reference,
 * which is single-GPU, README.md:92): this rank holds N of the layer's ldc output features, starting at
 * col_offset.  Its [M, N] product is written into columns [col_offset, col_offset + N) of its own
 * [M, ldc] buffer `out_bf16` and, from the same epilogue, of the n_peers (<= 7) other ranks' buffers
 * `peer_outs[i]` (device pointers that are valid on this GPU: P2P / symmetric-memory mappings), with
 * ordinary stores, so the all-gather of the slices overlaps the GEMM.  When the kernel has finished its
 * stores are complete; the ranks then synchronise among themselves before reading their buffers.
 * M > 128, N >= 256 (the large-M kernel); other constraints as for fpq_gemm_fp4.
 */
int fpq_gemm_fp4_push(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* a_scales_swizzled,
                      const uint8_t* b_scales_swizzled, const float* alpha, const void* bias_bf16,
                      void* out_bf16, void* const* peer_outs, int n_peers, int64_t ldc, int64_t col_offset,
                      int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag, fpq_stream_t stream);

/*
 * C[M,N] = beta * C + alpha * A[M,K] * op(B) in true fp32 (no TF32), row-major with leading
 * dimensions; op(B) = B[K,N] or, when b_transposed, B[N,K]^T.  Stands in for the torch fp32
 * matmuls of the GPTQ path (src/quantization/gptq.py:29-30, :184-187; TF32 is switched off at
 * model_quant.py:27-29).
 */
int fpq_sgemm(const float* A, int64_t lda, const float* B, int64_t ldb, int b_transposed, float* C,
              int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta, fpq_stream_t stream);

/*
 * H[d,d] (fp32) = beta * H + alpha * Xa^T Xb on the tcgen05 tensor cores (bf16 operands, exact products,
 * fp32 accumulation).  With xb NULL or equal to xa only the lower-triangle tiles are computed and
 * mirrored, as accumulate_hessian does (src/quantization/accumulate_hessian.py:20-148); alpha and beta
 * carry the running-mean factors of GPTQ.update (src/quantization/gptq.py:94-102), so the input is
 * not rescaled.  xa, xb: bf16 [tokens, d] row-major, d % 8 == 0.  error_flag as in fpq_gemm_fp4.
 * Tokens are processed in slabs of 4096 (one launch each) because the tensor core's accumulator truncates:
 * 4.5e-6 relative Frobenius error against fp64 for any number of tokens.
 */
int fpq_hessian_accumulate(float* H, int64_t d, const void* xa_bf16, const void* xb_bf16, int64_t tokens,
                           float alpha, float beta, int32_t* error_flag, fpq_stream_t stream);

/*
 * In-place Hessian preparation of GPTQ._get_hessian_inverse (src/quantization/gptq.py:201-211):
 * rows/columns of H whose weight column W[:, j] is entirely zero are cleared and get a unit
 * diagonal, then rel_damp * mean(diag H) is added to the diagonal.  H [d,d], W [rows,d] fp32;
 * workspace: d bytes.
 */
int fpq_hessian_prepare(float* H, int64_t d, const float* W, int64_t rows, float rel_damp,
                        uint8_t* workspace, fpq_stream_t stream);

/*
 * fpq_hessian_prepare for callers that cannot hand over a workspace.  It has no counterpart in the
 * reference.  Some hosts may not allocate device memory at the point where they prepare a Hessian:
 * a serving or quantisation runtime that gives all of HBM to its own pool at start-up, a plugin that
 * runs under a framework which forbids driver allocations in its steady state, code between
 * cudaStreamBeginCapture and EndCapture (where cudaMalloc is illegal).  This variant keeps its one
 * scratch buffer -- a dead-column flag per input channel -- in a fixed array inside the library
 * (FPQ_PREPARE_NOALLOC_MAX_D bytes per GPU that loads the library, held until the process exits) and
 * calls no cudaMalloc, cudaFree or any allocating routine.
 *   - d must not exceed FPQ_PREPARE_NOALLOC_MAX_D; larger d is rejected with FPQ_ERR_INVALID_ARGUMENT.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before any stream capture begins.
 *   - The scratch used is the CURRENT device's copy of the array: make the GPU that owns H, W and the
 *     stream current before the call (a Hessian on another device is rejected).
 *   - All calls on one GPU share the array: calls whose kernels may overlap on the GPU (different
 *     streams without ordering between them) race on it.  Serialise them, or use fpq_hessian_prepare.
 *     The array keeps the last call's flags; every flag the next call reads is rewritten first, so no
 *     clearing is needed.
 * Same arithmetic and result as fpq_hessian_prepare.
 */
#define FPQ_PREPARE_NOALLOC_MAX_D 32768
int fpq_hessian_prepare_noalloc(float* H, int64_t d, const float* W, int64_t rows, float rel_damp,
                                fpq_stream_t stream);

/* Number of floats fpq_cholesky_inverse_upper needs as workspace for a d x d matrix (sizing helper; the
 * reference's torch.linalg calls allocate their own, src/utils/linalg_utils.py:8-12). */
int64_t fpq_cholesky_workspace_floats(int64_t d);

/*
 * U = upper-triangular factor with U^T U = H^-1: what `torch.linalg.cholesky(inv_sym(H), upper=True)`
 * returns (src/quantization/gptq.py:212-215, src/utils/linalg_utils.py:8-12), computed as one
 * Cholesky factorisation of the index-reversed H and one triangular inverse, all in fp32.
 * *status (device int32) becomes 1 when a pivot is not positive -- the reference then falls back to
 * the identity (gptq.py:216-217); the caller decides.  H is not modified; U must not alias H.
 * The large trailing updates and triangular-inverse products run on the tensor cores as three-term
 * bf16 splits (fp32-level accuracy); error_flag as for fpq_gemm_fp4.
 */
int fpq_cholesky_inverse_upper(const float* H, float* U, int64_t d, float* workspace, int32_t* status,
                               int32_t* error_flag, fpq_stream_t stream);

/*
 * The column loop of GPTQ.step (src/quantization/gptq.py:159-187), default column order:
 * W [rows, cols] fp32 (rotated weights) is overwritten with the dequantised result; `scales`
 * fp32 [rows, cols/group] are the static group scales computed beforehand from the unmodified
 * W (gptq.py:142); U from fpq_cholesky_inverse_upper; codes (optional) receives the packed E2M1
 * codes [rows, cols/2] (what pack_fp4_to_uint8(qweight) yields, gptq.py:429).
 * cols % 128 == 0; group 16 or 32.  The update of the columns right of each 128-column block
 * (gptq.py:186-187, an fp32 addmm in the reference) runs on the tensor cores as a three-term bf16
 * split of both factors (fp32-level accuracy); workspace: fpq_gptq_workspace_bytes(rows, cols) bytes,
 * 256-byte aligned; error_flag as for fpq_gemm_fp4.
 */
int fpq_gptq_quantize(float* W, int64_t rows, int64_t cols, const float* scales, int group,
                      const float* U, uint8_t* codes, void* workspace, int32_t* error_flag, fpq_stream_t stream);

/*
 * The same loop in activation order (quantization_order = "activation", gptq.py:146-155, 170-171): the
 * caller has permuted the columns of W (and the Hessian behind U) by falling diag(H); group_index
 * (device int32 [cols]) names, for every permuted column, which of the cols/group static scale groups
 * of the unpermuted W it belongs to.  W and codes come back in the permuted order (gptq.py:190-192
 * undoes it).  group_index == NULL is fpq_gptq_quantize.
 */
int fpq_gptq_quantize_ordered(float* W, int64_t rows, int64_t cols, const float* scales, int group,
                              const int32_t* group_index, const float* U, uint8_t* codes, void* workspace,
                              int32_t* error_flag, fpq_stream_t stream);

/* Bytes of workspace fpq_gptq_quantize needs for a [rows, cols] weight (sizing helper for the call above;
 * the reference allocates its temporaries implicitly, gptq.py:159-187). */
int64_t fpq_gptq_workspace_bytes(int64_t rows, int64_t cols);

/*
 * get_relative_mse_error (src/quantization/gptq.py:28-30):
 * out[0] = mean(((Wq - W) H) * (Wq - W)) / (mean((W H) * W) + 1e-6).  Wq, W [rows, d], H [d, d] fp32;
 * diff_workspace: rows * d floats; acc_workspace: FPQ_RELATIVE_MSE_ACC_DOUBLES doubles (one slot per CTA:
 * partial sums are written, never added atomically, and summed in a fixed order, so the result is the same
 * bit pattern on every run); out: device fp32[1].
 */
#define FPQ_RELATIVE_MSE_ACC_DOUBLES 32768
int fpq_relative_mse(const float* Wq, const float* W, const float* H, int64_t rows, int64_t d,
                     float* diff_workspace, double* acc_workspace, float* out, fpq_stream_t stream);

/*
 * The same metric (src/quantization/gptq.py:28-30) on the tensor cores: sum((A H) .* A) = <H, A^T A>, with
 * A^T A computed like a Hessian from a two-term bf16 split of A (~1e-5 relative accuracy).
 * bf16_workspace: 2 * rows * d bf16; gram_workspace: d * d floats; acc_workspace:
 * FPQ_RELATIVE_MSE_ACC_DOUBLES doubles (deterministic reduction as above); d % 8 == 0.
 */
int fpq_relative_mse_tc(const float* Wq, const float* W, const float* H, int64_t rows, int64_t d,
                        void* bf16_workspace, float* gram_workspace, double* acc_workspace, float* out,
                        int32_t* error_flag, fpq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FPQ_B200_H_ */
