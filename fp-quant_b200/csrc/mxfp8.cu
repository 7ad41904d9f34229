// MXFP8 operands for the quantised backward pass (sm_100a): the two re-quantisation steps that feed
// fpq_gemm_mxf8.  Both work on 32 x 32 squares, so that one E8M0 scale serves a square read along its rows
// or along its columns, and both are plain HBM-bound passes: a block of 256 threads owns 32 rows x 256
// columns of the input (eight squares), a thread one row of one square (32 elements: 64 bytes of bf16 or
// 16 bytes of FP4 codes), so eight neighbouring threads read 512 (or 128) contiguous bytes of a row.
//
// The external kernels these stand for (QuTLASS' backward_bf16_square_double_mxfp8 and
// mxfp4_transpose_mxfp8, bound at inference_lib/src/fp_quant/module/qutlass_ops.py:277-330) are not
// available; the arithmetic below is this library's definition, restated bit for bit by oracle/mxfp8.py.

#include "common.cuh"

namespace fpq {
namespace {

constexpr int SQ = 32;                 // side of a square
constexpr int SQ_PER_BLOCK = 8;        // squares (of one row band) per thread block
constexpr int THREADS = SQ * SQ_PER_BLOCK;

// Byte offset of scale (row, column) in the 128-row x 4-column tile layout the GEMM reads (tiles row-block-major).
__device__ __forceinline__ size_t sf_offset(int64_t row, int64_t sfc, int64_t sf_cols, int layout) {
  if (layout != FPQ_SCALES_SWIZZLED) return (size_t)(row * sf_cols + sfc);
  const int64_t tiles_per_row_block = (sf_cols + 3) / 4;
  return (size_t)(((row >> 7) * tiles_per_row_block + (sfc >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (sfc & 3));
}

// Shared-memory tiles of the transposing kernels: [square][source column][source row], rows padded to a
// multiple of 16 bytes and squares skewed by one more 16-byte unit so that the eight squares a warp writes at
// once start in different banks.
constexpr int T8_ROW = SQ + 4, T8_SQ = SQ * T8_ROW + 16;         // bytes
constexpr int T16_ROW = SQ + 8, T16_SQ = SQ * T16_ROW + 8;       // bf16 elements

// v * 2^k, exact: one multiply while 2^k is a normal number, the library routine at the extremes.
__device__ __forceinline__ float scale_pow2(float v, int k) {
  if (k >= -126 && k <= 127) return v * __int_as_float((k + 127) << 23);
  return scalbnf(v, k);
}

__device__ __forceinline__ uint16_t e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// Maximum over the 32 rows of every square of the band: thread (r, c) contributes v, all get the result.
__device__ __forceinline__ float square_max(float v, int r, int c, float (*sm)[SQ + 1]) {
  sm[c][r] = v;
  __syncthreads();
  float m = sm[c][0];
#pragma unroll
  for (int i = 1; i < SQ; ++i) m = fmaxf(m, sm[c][i]);
  __syncthreads();
  return m;
}

// ---------------------------------------------------------------------------------------------------------
// bf16 [rows, cols] -> E4M3 [rows_pad, cols] + one E8M0 byte per 32 x 32 square, written twice: as
// row_scales [rows_pad, cols/32] (the scale of element (i, j) at [i, j/32]) and as col_scales
// [cols, rows_pad/32] (at [j, i/32]).  Square scale: 2^(floor(log2(amax)) - 8) (8 = exponent of the largest
// E4M3 binade), byte 0 for an all-zero square; elements are divided by it exactly, clamped to +-448 and
// rounded to nearest even.  Rows in [rows, rows_pad) are zero.
__global__ void __launch_bounds__(THREADS) square_quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows,
                                                                  int64_t cols, int64_t rows_pad, uint8_t* __restrict__ out,
                                                                  uint8_t* __restrict__ out_t, uint8_t* __restrict__ row_scales,
                                                                  uint8_t* __restrict__ col_scales, int layout) {
  __shared__ float sm[SQ_PER_BLOCK][SQ + 1];
  __shared__ __align__(16) uint8_t tile[SQ_PER_BLOCK * T8_SQ];
  const int r = threadIdx.x / SQ_PER_BLOCK, c = threadIdx.x % SQ_PER_BLOCK;
  const int64_t row = (int64_t)blockIdx.y * SQ + r;
  const int64_t sq_col = (int64_t)blockIdx.x * SQ_PER_BLOCK + c;          // square index along the columns
  const int64_t col0 = sq_col * SQ;
  const bool in_cols = col0 < cols, live = in_cols && row < rows;
  float v[SQ];
  float amax = 0.0f;
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + row * cols + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 w = src[q];
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * q + 2 * j] = __uint_as_float(ws[j] << 16);
        v[8 * q + 2 * j + 1] = __uint_as_float(ws[j] & 0xffff0000u);
      }
    }
#pragma unroll
    for (int i = 0; i < SQ; ++i) amax = fmaxf(amax, fabsf(v[i]));
  } else {
#pragma unroll
    for (int i = 0; i < SQ; ++i) v[i] = 0.0f;
  }
  amax = square_max(amax, r, c, sm);
  uint32_t byte = 0;
  int shift = 0;                                      // elements are multiplied by 2^shift
  if (amax > 0.0f && amax < __int_as_float(0x7f800000)) {
    int e = ilogbf(amax) - 8;                         // floor(log2(amax)) - 8; bf16 subnormals included
    e = max(-127, min(127, e));
    byte = (uint32_t)(e + 127);
    shift = -e;
  }
  uint32_t o[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    float s[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j] = fminf(fmaxf(scale_pow2(v[4 * q + j], shift), -448.0f), 448.0f);
    o[q] = (uint32_t)e4m3x2(s[0], s[1]) | ((uint32_t)e4m3x2(s[2], s[3]) << 16);
  }
  if (out_t != nullptr) {      // the same bytes the other way round: [column][row] through shared memory
#pragma unroll
    for (int q = 0; q < 8; ++q) {
#pragma unroll
      for (int j = 0; j < 4; ++j) tile[c * T8_SQ + (4 * q + j) * T8_ROW + r] = (uint8_t)(o[q] >> (8 * j));
    }
    __syncthreads();
  }
  if (!in_cols) return;
  uint4* dst = reinterpret_cast<uint4*>(out + row * cols + col0);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  row_scales[sf_offset(row, sq_col, cols / SQ, layout)] = (uint8_t)byte;
  // the same byte for the 32 columns of the square, seen from the transposed side: thread r takes column r
  col_scales[sf_offset(col0 + r, blockIdx.y, rows_pad / SQ, layout)] = (uint8_t)byte;
  if (out_t != nullptr) {
    const uint32_t* t32 = reinterpret_cast<const uint32_t*>(&tile[c * T8_SQ + r * T8_ROW]);
    uint4* dt = reinterpret_cast<uint4*>(out_t + (col0 + r) * rows_pad + (int64_t)blockIdx.y * SQ);
    dt[0] = make_uint4(t32[0], t32[1], t32[2], t32[3]);
    dt[1] = make_uint4(t32[4], t32[5], t32[6], t32[7]);
  }
}

// ---------------------------------------------------------------------------------------------------------
// MXFP4 [rows, cols] (packed E2M1 codes [rows, cols/2], E8M0 bytes [rows, cols/32]) -> its transpose as
// MXFP8: E4M3 [cols, rows_pad] with E8M0 bytes [cols, rows_pad/32].  The 32 rows of a square carry 32
// different source exponents e_i; the square gets 2^(emax - 6) (6 = the head room between the largest FP4
// magnitude 6 and 448, so that rows up to 2^-14 below the largest are kept exactly) and element (i, j)
// becomes fp4 * 2^(e_i - emax + 6), rounded to nearest even where it falls below the E4M3 grid.  Source
// rows in [rows, rows_pad) count as zero; a square without source rows has byte 0.
__global__ void __launch_bounds__(THREADS) fp4_transpose_fp8_kernel(const uint8_t* __restrict__ codes,
                                                                    const uint8_t* __restrict__ scales, int64_t rows,
                                                                    int64_t cols, int64_t rows_pad, uint8_t* __restrict__ out,
                                                                    uint8_t* __restrict__ out_scales, int layout) {
  __shared__ float sm[SQ_PER_BLOCK][SQ + 1];
  __shared__ __align__(16) uint8_t tile[SQ_PER_BLOCK * T8_SQ];
  const int r = threadIdx.x / SQ_PER_BLOCK, c = threadIdx.x % SQ_PER_BLOCK;
  const int64_t row = (int64_t)blockIdx.y * SQ + r;
  const int64_t sq_col = (int64_t)blockIdx.x * SQ_PER_BLOCK + c;
  const int64_t col0 = sq_col * SQ;
  const bool in_cols = col0 < cols, live = in_cols && row < rows;
  uint4 w = make_uint4(0, 0, 0, 0);
  int e_row = -1000;                                   // below every real exponent
  if (live) {
    w = *reinterpret_cast<const uint4*>(codes + row * (cols / 2) + col0 / 2);
    e_row = (int)scales[row * (cols / SQ) + sq_col] - 127;
  }
  const int emax = (int)square_max((float)e_row, r, c, sm);
  uint32_t byte = 0;
  int shift = 0;
  if (emax > -1000) {
    const int e_sq = max(-127, emax - 6);
    byte = (uint32_t)(e_sq + 127);
    shift = e_row - e_sq;                              // <= 6 for live rows; very negative rows round to zero
  }
  // Every code of the row is scaled by the same power of two, so the 32 conversions are table look-ups: the
  // E4M3 bytes of the eight FP4 magnitudes times 2^shift, once as they are and once with the sign bit (the
  // zero stays +0 in both, as the code's "-0" must come out), selected four at a time with byte permutes.
  uint32_t pa = 0, pb = 0, na = 0, nb = 0;
  if (live) {
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = scale_pow2(e2m1_magnitude(i), shift);
    pa = (uint32_t)e4m3x2(m[0], m[1]) | ((uint32_t)e4m3x2(m[2], m[3]) << 16);
    pb = (uint32_t)e4m3x2(m[4], m[5]) | ((uint32_t)e4m3x2(m[6], m[7]) << 16);
    na = (pa | 0x80808080u) & 0xffffff00u;
    nb = pb | 0x80808080u;
  }
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t x = half ? ws[q] >> 16 : ws[q];                   // four codes in the low 16 bits
      const uint32_t sel = x & 0x7777u;                                // their magnitudes as byte selectors
      const uint32_t pos = __byte_perm(pa, pb, sel), neg = __byte_perm(na, nb, sel);
      const uint32_t o4 = __byte_perm(pos, neg, ((x & 0x8888u) >> 1) | 0x3210u);   // byte i from neg where code i is negative
#pragma unroll
      for (int i = 0; i < 4; ++i)
        tile[c * T8_SQ + (8 * q + 4 * half + i) * T8_ROW + r] = (uint8_t)(o4 >> (8 * i));
    }
  }
  __syncthreads();
  // thread (r, c) now owns source column col0 + r: 32 contiguous output bytes
  if (!in_cols) return;
  const int64_t out_row = col0 + r;
  const uint32_t* t32 = reinterpret_cast<const uint32_t*>(&tile[c * T8_SQ + r * T8_ROW]);
  uint4* dst = reinterpret_cast<uint4*>(out + out_row * rows_pad + (int64_t)blockIdx.y * SQ);
  dst[0] = make_uint4(t32[0], t32[1], t32[2], t32[3]);
  dst[1] = make_uint4(t32[4], t32[5], t32[6], t32[7]);
  out_scales[sf_offset(out_row, blockIdx.y, rows_pad / SQ, layout)] = (uint8_t)byte;
}

// ---------------------------------------------------------------------------------------------------------
// MXFP4 [rows, cols] -> bf16 [cols, rows]: the transpose of the dequantised tensor divided by *alpha (the
// tensor scale the operand was quantised under), rounded once to bf16.  First half of backward_qt_bf16
// (qutlass_ops.py:248-274); the rotation and re-quantisation that follow are the forward quantise kernel.
__global__ void __launch_bounds__(THREADS) fp4_transpose_bf16_kernel(const uint8_t* __restrict__ codes,
                                                                     const uint8_t* __restrict__ scales, int64_t rows,
                                                                     int64_t cols, const float* __restrict__ alpha,
                                                                     __nv_bfloat16* __restrict__ out, int64_t out_ld) {
  __shared__ __align__(16) __nv_bfloat16 tile[SQ_PER_BLOCK * T16_SQ];      // [square][column of the source][row of the source]
  const int r = threadIdx.x / SQ_PER_BLOCK, c = threadIdx.x % SQ_PER_BLOCK;
  const int64_t row = (int64_t)blockIdx.y * SQ + r;
  const int64_t sq_col = (int64_t)blockIdx.x * SQ_PER_BLOCK + c;
  const int64_t col0 = sq_col * SQ;
  const bool in_cols = col0 < cols, live = in_cols && row < rows;
  const float a = *alpha;
  if (live) {
    const uint4 w = *reinterpret_cast<const uint4*>(codes + row * (cols / 2) + col0 / 2);
    const int e = (int)scales[row * (cols / SQ) + sq_col] - 127;
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    // fl((m 2^e) / a) = fl(m / a) 2^e while nothing leaves the normal range: seven divisions per row instead
    // of thirty-two, and the 32 conversions become table look-ups (low and high bytes of the eight bf16
    // quotients, the high bytes once more with the sign bit; the zero stays +0), four codes per byte permute.
    // The bound on e keeps every quotient normal for 2^-20 < a < 2^20.
    const bool table = e > -100 && e < 100 && a > 9.5367e-7f && a < 1.048576e6f;
    uint16_t* tile16 = reinterpret_cast<uint16_t*>(tile);
    if (table) {
      uint32_t lo_a = 0, lo_b = 0, hi_a = 0, hi_b = 0;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const __nv_bfloat16 h = __float2bfloat16_rn(scale_pow2(__fdiv_rn(e2m1_magnitude(m), a), e));
        const uint32_t bits = *reinterpret_cast<const uint16_t*>(&h);
        if (m < 4) {
          lo_a |= (bits & 0xffu) << (8 * m);
          hi_a |= (bits >> 8) << (8 * m);
        } else {
          lo_b |= (bits & 0xffu) << (8 * (m - 4));
          hi_b |= (bits >> 8) << (8 * (m - 4));
        }
      }
      const uint32_t nhi_a = (hi_a | 0x80808080u) & 0xffffff00u, nhi_b = hi_b | 0x80808080u;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t x = half ? ws[q] >> 16 : ws[q];                 // four codes in the low 16 bits
          const uint32_t sel = x & 0x7777u;
          const uint32_t lo4 = __byte_perm(lo_a, lo_b, sel);
          const uint32_t hi4 = __byte_perm(__byte_perm(hi_a, hi_b, sel), __byte_perm(nhi_a, nhi_b, sel),
                                           ((x & 0x8888u) >> 1) | 0x3210u);
          const uint32_t w01 = __byte_perm(lo4, hi4, 0x5140), w23 = __byte_perm(lo4, hi4, 0x7362);
          uint16_t* col = tile16 + c * T16_SQ + (8 * q + 4 * half) * T16_ROW + r;
          col[0] = (uint16_t)w01;
          col[T16_ROW] = (uint16_t)(w01 >> 16);
          col[2 * T16_ROW] = (uint16_t)w23;
          col[3 * T16_ROW] = (uint16_t)(w23 >> 16);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __fdiv_rn(scale_pow2(e2m1_value((ws[q] >> (4 * j)) & 15u), e), a);
          tile[c * T16_SQ + (8 * q + j) * T16_ROW + r] = __float2bfloat16_rn(v + 0.0f);
        }
      }
    }
  }
  __syncthreads();
  if (!in_cols) return;
  // thread (r, c) owns source column col0 + r: up to 32 contiguous bf16 of the output row
  const int64_t out_row = col0 + r;
  const int64_t m0 = (int64_t)blockIdx.y * SQ;
  __nv_bfloat16* dst = out + out_row * out_ld + m0;
  if (m0 + SQ <= rows && (out_ld % 8) == 0) {
    const uint4* t = reinterpret_cast<const uint4*>(&tile[c * T16_SQ + r * T16_ROW]);
#pragma unroll
    for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(dst)[q] = t[q];
  } else {
    for (int i = 0; i < SQ && m0 + i < rows; ++i) dst[i] = tile[c * T16_SQ + r * T16_ROW + i];
  }
}

}  // namespace
}  // namespace fpq

using namespace fpq;

extern "C" int fpq_mxfp4_transpose_dequant(const uint8_t* codes, const uint8_t* scales_rowmajor, int64_t rows, int64_t cols,
                                           const float* alpha, void* out_bf16, int64_t out_ld, fpq_stream_t stream) {
  FPQ_CHECK_ARG(codes && scales_rowmajor && alpha && out_bf16, "NULL pointer");
  FPQ_CHECK_ARG(out_ld >= rows, "out_ld (%lld) must not be below rows (%lld)", (long long)out_ld, (long long)rows);
  FPQ_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "cols (%lld) must be a positive multiple of 32", (long long)cols);
  FPQ_CHECK_ARG(rows < (1ll << 31) && cols < (1ll << 31), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)codes & 15) == 0 && ((uintptr_t)out_bf16 & 15) == 0, "codes and out must be 16-byte aligned");
  const dim3 grid((unsigned)((cols / SQ + SQ_PER_BLOCK - 1) / SQ_PER_BLOCK), (unsigned)((rows + SQ - 1) / SQ));
  FPQ_CHECK_ARG(grid.y < 65536, "too many rows for one launch");
  fp4_transpose_bf16_kernel<<<grid, THREADS, 0, (cudaStream_t)stream>>>(codes, scales_rowmajor, rows, cols, alpha,
                                                                        reinterpret_cast<__nv_bfloat16*>(out_bf16), out_ld);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_quantize_mxfp8_square(const void* x_bf16, int64_t rows, int64_t cols, uint8_t* out_e4m3,
                                         uint8_t* out_t_e4m3, uint8_t* row_scales, uint8_t* col_scales,
                                         int scale_layout, fpq_stream_t stream) {
  FPQ_CHECK_ARG(x_bf16 && out_e4m3 && row_scales && col_scales, "NULL pointer");
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale layout");
  FPQ_CHECK_ARG(out_t_e4m3 == nullptr || ((uintptr_t)out_t_e4m3 & 15) == 0, "out_t must be 16-byte aligned");
  FPQ_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "cols (%lld) must be a positive multiple of 32", (long long)cols);
  FPQ_CHECK_ARG(rows < (1ll << 31) && cols < (1ll << 31), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)x_bf16 & 15) == 0 && ((uintptr_t)out_e4m3 & 15) == 0, "x and out must be 16-byte aligned");
  const int64_t rows_pad = (rows + 127) / 128 * 128;
  const dim3 grid((unsigned)((cols / SQ + SQ_PER_BLOCK - 1) / SQ_PER_BLOCK), (unsigned)(rows_pad / SQ));
  FPQ_CHECK_ARG(grid.y < 65536, "too many rows for one launch");
  square_quantize_kernel<<<grid, THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(x_bf16), rows,
                                                                     cols, rows_pad, out_e4m3, out_t_e4m3, row_scales,
                                                                     col_scales, scale_layout);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_mxfp4_transpose_mxfp8(const uint8_t* codes, const uint8_t* scales_rowmajor, int64_t rows, int64_t cols,
                                         uint8_t* out_e4m3, uint8_t* out_scales, int scale_layout, fpq_stream_t stream) {
  FPQ_CHECK_ARG(codes && scales_rowmajor && out_e4m3 && out_scales, "NULL pointer");
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale layout");
  FPQ_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "cols (%lld) must be a positive multiple of 32", (long long)cols);
  FPQ_CHECK_ARG(rows < (1ll << 31) && cols < (1ll << 31), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)codes & 15) == 0 && ((uintptr_t)out_e4m3 & 15) == 0, "codes and out must be 16-byte aligned");
  const int64_t rows_pad = (rows + 127) / 128 * 128;
  const dim3 grid((unsigned)((cols / SQ + SQ_PER_BLOCK - 1) / SQ_PER_BLOCK), (unsigned)(rows_pad / SQ));
  FPQ_CHECK_ARG(grid.y < 65536, "too many rows for one launch");
  fp4_transpose_fp8_kernel<<<grid, THREADS, 0, (cudaStream_t)stream>>>(codes, scales_rowmajor, rows, cols, rows_pad, out_e4m3,
                                                                       out_scales, scale_layout);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}
