// Fused block-Hadamard rotation + micro-scaled FP4 quantisation (MXFP4 / NVFP4) for sm_100a.
//
// One thread owns 32 contiguous elements of a row (64 B of bf16 = two 128-bit loads, one
// 256-bit load on sm_100).  Butterfly stages with pair distance <= 16 run in registers, the
// stages for distance 32 and 64 exchange registers with the neighbouring lanes by warp
// shuffle.  All rotation arithmetic is IEEE fp32 add/sub/mul in a fixed order (distances
// 1,2,4,..,g/2, then one multiply by fl32(1/sqrt(g))) so that a CPU can reproduce it bit
// for bit.  The scale chain and the division that precedes E2M1 rounding reproduce the
// fp32 operation sequence of the reference Quantizer (src/quantization/quantizer.py:107-168,
// src/quantization/quant_ops.py:57-94 of IST-DASLab/FP-Quant).
//
// The kernel is HBM-bound: 2 B read + 0.5 B codes + 1/g B scale per element.

#include "common.cuh"

namespace fpq {
namespace {

enum Mode { MODE_CODES = 0, MODE_DEQUANT = 1, MODE_ROTATE = 2, MODE_ABSMAX = 3 };

struct QuantParams {
  const void* x;
  int64_t n_chunks;     // rows * cols / 32
  uint32_t chunks_per_row;
  uint64_t row_magic;   // ceil(2^64 / chunks_per_row) (0 when chunks_per_row == 1): chunk -> row by one multiply
  uint8_t* codes;       // [rows, cols/2]
  uint8_t* sbytes;      // scale bytes
  float* sf32;          // fp32 scales, row-major
  void* y;              // dequantised / rotated output
  const float* gs;      // NVFP4 tensor scale
  uint32_t* absmax_bits;
  uint8_t* mask;        // QuEST clip mask: one bit per element (codes) or one byte per element (dequantised output)
  uint32_t sf_tiles_per_row_block;  // ceil((cols/g)/4)
  uint32_t rows, pad_rows;          // swizzled scale layout: rows of the tensor and rows up to the next multiple of 128
  int layout;
  int out_bf16;
  int ste;
};

typedef unsigned long long u64;

__device__ __forceinline__ u64 pack2(float lo, float hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(u64 p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
  u64 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
  u64 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
  u64 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
  u64 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// 32 contiguous elements of a row as they lie in memory: sixteen 32-bit words of bf16 pairs, or
// sixteen 64-bit words of fp32 pairs (element 2j in the low half of word j).
template <bool IN_BF16> struct RawChunk;
template <> struct RawChunk<true> { uint32_t w[16]; };
template <> struct RawChunk<false> { u64 w[16]; };

__device__ __forceinline__ void load_raw(const void* base, int64_t chunk, bool active, RawChunk<true>& r) {
  if (active) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(base) + chunk * 16;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]),
                   "=r"(r.w[6]), "=r"(r.w[7])
                 : "l"(p));
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[8]), "=r"(r.w[9]), "=r"(r.w[10]), "=r"(r.w[11]), "=r"(r.w[12]), "=r"(r.w[13]),
                   "=r"(r.w[14]), "=r"(r.w[15])
                 : "l"(p + 8));
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) r.w[j] = 0;
  }
}
__device__ __forceinline__ void load_raw(const void* base, int64_t chunk, bool active, RawChunk<false>& r) {
  if (active) {
    const u64* p = reinterpret_cast<const u64*>(base) + chunk * 16;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      asm volatile("ld.global.nc.L1::no_allocate.v4.b64 {%0,%1,%2,%3}, [%4];"
                   : "=l"(r.w[4 * q]), "=l"(r.w[4 * q + 1]), "=l"(r.w[4 * q + 2]), "=l"(r.w[4 * q + 3])
                   : "l"(p + 4 * q));
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) r.w[j] = 0ull;
  }
}

#ifndef FPQ_Q_UNPACK
#define FPQ_Q_UNPACK 0      // 1: bf16 -> fp32 with cvt instead of shift / mask (measured: see the profile notes)
#endif
#ifndef FPQ_Q_MAX3
#define FPQ_Q_MAX3 1
#endif

// Raw words -> fp32 pairs.  With STAGE1 the first butterfly stage (distance 1: the two elements
// of a pair become their sum and difference) is applied on the way.
template <bool STAGE1>
__device__ __forceinline__ void unpack_chunk(const RawChunk<true>& r, u64 (&P)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
#if FPQ_Q_UNPACK == 1
    uint16_t l16, h16;
    float a, b;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(l16), "=h"(h16) : "r"(r.w[j]));
    asm("cvt.f32.bf16 %0, %1;" : "=f"(a) : "h"(l16));
    asm("cvt.f32.bf16 %0, %1;" : "=f"(b) : "h"(h16));
#else
    const float a = __uint_as_float(r.w[j] << 16), b = __uint_as_float(r.w[j] & 0xffff0000u);
#endif
    P[j] = STAGE1 ? pack2(__fadd_rn(a, b), __fsub_rn(a, b)) : pack2(a, b);
  }
}
template <bool STAGE1>
__device__ __forceinline__ void unpack_chunk(const RawChunk<false>& r, u64 (&P)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (STAGE1) {
      float a, b;
      unpack2(r.w[j], a, b);
      P[j] = pack2(__fadd_rn(a, b), __fsub_rn(a, b));
    } else {
      P[j] = r.w[j];
    }
  }
}

// Butterfly stages with pair distance 1..min(GH,32)/2 inside the thread, then the
// cross-lane stages for distance 32 (GH >= 64) and 64 (GH == 128), then * 1/sqrt(GH).
template <int GH>
__device__ __forceinline__ constexpr float hadamard_scale() {
  return GH == 16 ? 0.25f : GH == 32 ? 0.17677669529663687f : GH == 64 ? 0.125f : GH == 128 ? 0.08838834764831845f : 1.0f;
}

template <int GH, bool SCALE = true>
__device__ __forceinline__ void rotate_chunk(u64 (&P)[16], int lane) {
  // distance 1 (inside each packed pair) was applied by unpack_chunk<true>
  // distances 2, 4, 8, 16 <-> pair index distance 1, 2, 4, 8
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    if (GH != 0 && 2 * d < (GH < 32 ? GH : 32)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if ((j & d) == 0) {
          u64 a = P[j], b = P[j + d];
          P[j] = add2(a, b);
          P[j + d] = sub2(a, b);
        }
      }
    }
  }
  if (GH >= 64) {
#pragma unroll
    for (int bit = 1; bit < GH / 32; bit <<= 1) {
      const float sgn = (lane & bit) ? -1.0f : 1.0f;
      const u64 S = pack2(sgn, sgn);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        u64 other = __shfl_xor_sync(0xffffffffu, P[j], bit);
        P[j] = fma2(S, P[j], other);  // bit clear: own + other, bit set: other - own
      }
    }
  }
  if (SCALE && GH != 0) {
    const float c = hadamard_scale<GH>();
    const u64 C = pack2(c, c);
#pragma unroll
    for (int j = 0; j < 16; ++j) P[j] = mul2(P[j], C);
  }
}

__device__ __forceinline__ u64 mul2_rz(u64 a, u64 b) {
  u64 r;
  asm("mul.rz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// MXFP4 shortcut.  With s = fl(4/3) * 2^(e-2) the E2M1 code of fl(fl(t*c) / s) -- t the unscaled
// butterfly output, c = 1/sqrt(g) -- equals the code of ONE rounded product t * (m * 2^(2-e)):
//   c a power of two (g = 16, 64, or no rotation): m = 0.75 * c, product rounded toward zero;
//   g = 32, 128:                                   m = fl(c / fl(4/3)), product rounded to nearest.
// Both were checked against the two-step form on every fp32 input within 20000 ulps of each of the
// seven rounding boundaries (and on random inputs); away from the boundaries the two values differ
// by a few ulps at most, which cannot change the code.
template <int GH>
__device__ __forceinline__ u64 mx_code_multiplier(int e) {
  constexpr bool POW2 = GH == 0 || GH == 16 || GH == 64;
  constexpr uint32_t mbits = GH == 0 ? 0x3f400000u : GH == 16 ? 0x3e400000u : GH == 64 ? 0x3dc00000u
                           : GH == 32 ? 0x3e07c3b6u : 0x3d87c3b6u;
  (void)POW2;
  const float m = __uint_as_float(mbits + ((uint32_t)(2 - e) << 23));   // exact scaling by 2^(2-e)
  return pack2(m, m);
}

__device__ __forceinline__ float absmax_pairs(const u64* P, int n) {
  float m = 0.0f;
#pragma unroll
  for (int j = 0; j < n; ++j) {
    float a, b;
    unpack2(P[j], a, b);
#if FPQ_Q_MAX3
    asm("max.f32 %0, %0, %1, %2;" : "+f"(m) : "f"(fabsf(a)), "f"(fabsf(b)));
#else
    m = fmaxf(m, fmaxf(fabsf(a), fabsf(b)));
#endif
  }
  return m;
}

// floor(fl32(log2(m))) as torch's fp32 log2 yields it: the exponent field, plus one when m is
// so close below a power of two that the correctly rounded fp32 logarithm is that integer.
__device__ __forceinline__ int mx_exponent(float m /* >= 2^-126, finite */) {
  uint32_t b = __float_as_uint(m);
  int e = (int)(b >> 23) - 127;
  if ((b & 0x7fffffu) >= 0x7fff00u) {
    float l = (float)log2((double)m);
    e = (int)floorf(l);
  }
  return max(-127, min(127, e));
}

// MXFP4 scale of one 32-element group: returns the divisor s and the stored byte.
// The reference computes e = floor(log2(m)) with m = fl(6 * fl(fl(2a) / 12)), which lies within
// two ulps of a.  When a's mantissa is at least four ulps away from both ends of its binade (and
// from the 0x7fff00 threshold of the logarithm's rounding artefact) m has a's exponent, so the
// division chain is only evaluated for the rare group maxima near a power of two.
__device__ __forceinline__ float mx_scale(float a, uint32_t& byte, int& e) {
  const uint32_t bits = __float_as_uint(a);
  const uint32_t mant = bits & 0x7fffffu, ex = bits >> 23;   // a >= 0
  if (mant - 4u <= 0x7ffef7u && ex - 8u <= 239u) {           // mant in [4, 0x7ffefb], ex in [8, 247]
    e = (int)ex - 127;
    byte = ex;
    return __uint_as_float(((ex - 2u) << 23) | 0x2aaaabu);
  }
  float s0 = __fdiv_rn(__fmul_rn(2.0f, a), 12.0f);
  float m = fmaxf(__fmul_rn(6.0f, s0), 1.17549435e-38f);
  e = mx_exponent(m);
  byte = (uint32_t)(e + 127);
  float s;
  if (e >= -124) {
    // fl(2^(e-2) / 0.75) = 2^(e-2) * fl(4/3): exponent field e-2+127, mantissa of fl(4/3)
    s = __uint_as_float(((uint32_t)(e + 125) << 23) | 0x2aaaabu);
  } else {
    s = __fdiv_rn(ldexpf(1.0f, e - 2), 0.75f);  // subnormal power of two
    if (s == 0.0f) s = 1.0f;
  }
  return s;
}

// Third value of the FMT template parameter (not part of the C ABI's format numbers): MXFP4 codes and
// E8M0 scale bytes with the QuEST scale rule instead of the group maximum.
constexpr int FMT_MXQUEST = 2;

// QuEST scale of one 32-element group (inference_lib/src/fp_quant/module/triton/mxfp4.py:51-59):
// std = sqrt(mean(x^2) - mean(x)^2), scale = fl(fl(c * std) + 1e-8) with c = fl32(2.92247856 / 6)
// (pseudoquant_linear_fns.py:20), divisor 2^floor(log2(scale)), stored byte = that exponent + 127.
// The sums run over the sixteen register pairs in order, even and odd elements separately (one packed
// add per pair), then even + odd; squares are rounded products (no fused multiply-add), so a CPU
// reproduces every bit.  A variance that rounds below zero counts as zero.  scale >= 1e-8 is a normal
// number, so the exponent field is floor(log2(scale)) exactly.
__device__ __forceinline__ float quest_scale(const u64* P, uint32_t& byte) {
  u64 acc = P[0], acc2 = mul2(P[0], P[0]);
#pragma unroll
  for (int j = 1; j < 16; ++j) {
    acc = add2(acc, P[j]);
    acc2 = add2(acc2, mul2(P[j], P[j]));
  }
  float a0, a1, q0, q1;
  unpack2(acc, a0, a1);
  unpack2(acc2, q0, q1);
  const float mean = __fmul_rn(__fadd_rn(a0, a1), 0.03125f);
  const float mean_sq = __fmul_rn(__fadd_rn(q0, q1), 0.03125f);
  const float var = fmaxf(__fsub_rn(mean_sq, __fmul_rn(mean, mean)), 0.0f);
  const float scale = __fadd_rn(__fmul_rn(0.48707976f, __fsqrt_rn(var)), 1e-8f);
  byte = (__float_as_uint(scale) >> 23) & 0xffu;
  return __uint_as_float(byte << 23);
}

// NVFP4 scale of one 16-element group.
__device__ __forceinline__ float nv_scale(float a, float gs, float rgs, uint32_t& byte) {
  // s0 = fl(fl(2a) / 12) = fl(a / 3) / 2.  With r = fl(1/3), q = fl(a r), e = a - 3 q (exact, fused) the
  // value fl(q + e r) is the correctly rounded a / 3 for every fp32 mantissa (checked exhaustively on the
  // CPU); halving is exact while nothing underflows, so the general division is kept for the extremes.
  float s0;
  if (a > 7.8886e-31f /* 2^-100 */ && a < 1.3292e36f /* 2^120 */) {
    const float r = 0.333333343f;             // 0x3eaaaaab
    float q = __fmul_rn(a, r);
    const float e = __fmaf_rn(-3.0f, q, a);
    q = __fmaf_rn(e, r, q);
    s0 = 0.5f * q;
  } else {
    s0 = __fdiv_rn(__fmul_rn(2.0f, a), 12.0f);
  }
  float t = fminf(fmaxf(__fmul_rn(s0, gs), -448.0f), 448.0f);
  uint16_t u2;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(u2) : "f"(0.0f), "f"(t));
  uint32_t u = u2 & 0xffu;
  // decode the (non-negative) E4M3 byte exactly: (8+m) * 2^(e-10), or m * 2^-9 when e == 0
  uint32_t ex = u >> 3, ma = u & 7u;
  float uf = ex == 0 ? (float)ma * 0.001953125f : __uint_as_float(((ex + 120u) << 23) | (ma << 20));
  float s = __fmul_rn(uf, rgs);
  byte = u;
  return s == 0.0f ? 1.0f : s;
}

// Correctly rounded y / s for the pairs P[0..n): reciprocal once per group, then the classic
// multiply + two fused residual corrections, two elements per instruction.  Falls back to
// per-element IEEE division when s is so small or large that the reciprocal or a residual
// could leave the normal range.
__device__ __forceinline__ void divide_pairs(u64* P, int n, float s) {
  const float as = fabsf(s);
  if (as > 7.8886e-31f /* 2^-100 */ && as < 1.2676e30f /* 2^100 */) {
    const float r = __frcp_rn(s);
    const u64 R = pack2(r, r), NS = pack2(-s, -s);
#pragma unroll
    for (int j = 0; j < n; ++j) {
      u64 y = P[j];
      u64 q = mul2(y, R);
      u64 e = fma2(q, NS, y);
      q = fma2(e, R, q);
      e = fma2(q, NS, y);
      P[j] = fma2(e, R, q);
    }
  } else {
#pragma unroll
    for (int j = 0; j < n; ++j) {
      float a, b;
      unpack2(P[j], a, b);
      P[j] = pack2(__fdiv_rn(a, s), __fdiv_rn(b, s));
    }
  }
}

// Eight quotients (4 pairs) -> one word of eight 4-bit codes, element 0 in the lowest nibble.
#ifndef FPQ_Q_PACKMOV
#define FPQ_Q_PACKMOV 1
#endif
__device__ __forceinline__ uint32_t codes_word(const u64* P) {
  uint32_t w = 0;
#if FPQ_Q_PACKMOV
  float a0, b0, a1, b1, a2, b2, a3, b3;
  unpack2(P[0], a0, b0);
  unpack2(P[1], a1, b1);
  unpack2(P[2], a2, b2);
  unpack2(P[3], a3, b3);
  asm("{ .reg .b8 t0, t1, t2, t3;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
      "  mov.b32 %0, {t0, t1, t2, t3}; }"
      : "=r"(w)
      : "f"(a0), "f"(b0), "f"(a1), "f"(b1), "f"(a2), "f"(b2), "f"(a3), "f"(b3));
#else
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float a, b;
    unpack2(P[j], a, b);
    uint32_t byte;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }"
        : "=r"(byte)
        : "f"(b), "f"(a));
    w |= byte << (8 * j);
  }
#endif
  return patch_zero_codes(w);
}

__device__ __forceinline__ size_t swizzled_offset(uint32_t row, uint32_t sfc, uint32_t tiles_per_row_block) {
  return ((size_t)(row >> 7) * tiles_per_row_block + (sfc >> 2)) * 512u + (row & 31u) * 16u +
         ((row >> 5) & 3u) * 4u + (sfc & 3u);
}

// chunk index -> (row, chunk in row).  One 64 x 64 -> high 64 multiply: with M = ceil(2^64 / d)
// the quotient floor(c * M / 2^64) is exact whenever c * (M d - 2^64) < 2^64, which holds for
// c, d < 2^32.  Larger chunk counts take the division.
__device__ __forceinline__ void chunk_row(const QuantParams& p, int64_t c, uint32_t& row, uint32_t& cir) {
  if (p.chunks_per_row == 1) {
    row = (uint32_t)c;
    cir = 0;
  } else if (p.row_magic) {
    row = (uint32_t)__umul64hi((u64)c, p.row_magic);
    cir = (uint32_t)c - row * p.chunks_per_row;
  } else {
    row = (uint32_t)(c / p.chunks_per_row);
    cir = (uint32_t)(c - (int64_t)row * p.chunks_per_row);
  }
}

// Everything that happens to one chunk of 32 elements after its load.
template <int GH, int FMT, bool IN_BF16, int MODE>
__device__ __forceinline__ void process_chunk(const QuantParams& p, const RawChunk<IN_BF16>& raw, int64_t c,
                                              bool active, int lane, float gs, float rgs, float& running_max) {
    u64 P[16];
    unpack_chunk<GH != 0>(raw, P);
    // MXFP4 codes take the unscaled butterfly output (the 1/sqrt(g) factor is folded into the
    // code multiplier); every other mode works on the scaled rotation.
    constexpr bool MX_FAST = MODE == MODE_CODES && FMT == FPQ_FMT_MXFP4;
    // NVFP4 codes with a rotation whose 1/sqrt(g) is a power of two (g = 16, 64): the factor c goes into the
    // divisor instead, t / (s / c) = (t c) / s exactly, which saves the sixteen scaling multiplies.
    constexpr bool NV_FOLD = MODE == MODE_CODES && FMT == FPQ_FMT_NVFP4 && (GH == 16 || GH == 64);
    rotate_chunk<GH, !(MX_FAST || NV_FOLD)>(P, lane);

    if (MODE == MODE_ABSMAX) {
      running_max = fmaxf(running_max, absmax_pairs(P, 16));
      return;
    }
    if (MODE == MODE_ROTATE) {
      if (active) {
        if (p.out_bf16) {
          uint4* o = reinterpret_cast<uint4*>(p.y) + c * 4;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float a, b;
              unpack2(P[4 * q + j], a, b);
              __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            o[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          ulonglong2* o = reinterpret_cast<ulonglong2*>(p.y) + c * 8;
#pragma unroll
          for (int q = 0; q < 8; ++q) o[q] = make_ulonglong2(P[2 * q], P[2 * q + 1]);
        }
      }
      return;
    }

    // ---- scales
    constexpr int NG = FMT == FPQ_FMT_NVFP4 ? 2 : 1;  // groups per thread
    constexpr int PG = 16 / NG;                       // pairs per group
    float s[NG];
    float amax_g[NG];
    uint32_t sb[NG];
    int mx_e = 0;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if (FMT == FMT_MXQUEST) break;
      float a = absmax_pairs(P + g * PG, PG);
      if ((MX_FAST || NV_FOLD) && GH != 0) a = __fmul_rn(a, hadamard_scale<GH>());   // max |t*c| = fl(c * max |t|)
      if (NV_FOLD) amax_g[g] = a;
      s[g] = FMT == FPQ_FMT_NVFP4 ? nv_scale(a, gs, rgs, sb[g]) : mx_scale(a, sb[g], mx_e);
    }
    if (FMT == FMT_MXQUEST) s[0] = quest_scale(P, sb[0]);
    if (MODE == MODE_CODES && active) {
      if (p.sbytes) {
        size_t off = (size_t)c * NG;
        if (p.layout == FPQ_SCALES_SWIZZLED) {
          uint32_t row, cir;
          chunk_row(p, c, row, cir);
          off = swizzled_offset(row, cir * NG, p.sf_tiles_per_row_block);
        }
        if (NG == 2)
          *reinterpret_cast<uint16_t*>(p.sbytes + off) = (uint16_t)(sb[0] | (sb[NG - 1] << 8));
        else
          p.sbytes[off] = (uint8_t)sb[0];
      }
      if (p.sf32) {
        if (NG == 2)
          *reinterpret_cast<float2*>(p.sf32 + c * 2) = make_float2(s[0], s[NG - 1]);
        else
          p.sf32[c] = s[0];
      }
    }
    if (MODE == MODE_CODES && p.codes == nullptr) return;

    // ---- keep the rotated values when the straight-through form needs them
    u64 Y[MODE == MODE_DEQUANT ? 16 : 1];
    if (MODE == MODE_DEQUANT) {
#pragma unroll
      for (int j = 0; j < 16; ++j) Y[j] = P[j];
    }

    if (MX_FAST) {
      if (mx_e >= -120 && mx_e <= 120) {
        const u64 MK = mx_code_multiplier<GH>(mx_e);
        constexpr bool RZ = GH == 0 || GH == 16 || GH == 64;
#pragma unroll
        for (int j = 0; j < 16; ++j) P[j] = RZ ? mul2_rz(P[j], MK) : mul2(P[j], MK);
      } else {   // extreme exponents: scale, then divide exactly
        if (GH != 0) {
          const float cc = hadamard_scale<GH>();
          const u64 C = pack2(cc, cc);
#pragma unroll
          for (int j = 0; j < 16; ++j) P[j] = mul2(P[j], C);
        }
        divide_pairs(P, 16, s[0]);
      }
    } else if (NV_FOLD) {
      constexpr float c = GH == 16 ? 0.25f : 0.125f;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const float sf = s[g] * (1.0f / c);
        // Exact while nothing leaves the normal range: then t c is exact for every element that can get a
        // non-zero code (an element whose t c is subnormal is > 2^20 below the group's scale).
        if (amax_g[g] > 7.8886e-31f /* 2^-100 */ && sf < 1.2676e30f /* 2^100 */) {
          divide_pairs(P + g * PG, PG, sf);
        } else {
          const u64 C = pack2(c, c);
#pragma unroll
          for (int j = 0; j < PG; ++j) P[g * PG + j] = mul2(P[g * PG + j], C);
          divide_pairs(P + g * PG, PG, s[g]);
        }
      }
    } else {
#pragma unroll
      for (int g = 0; g < NG; ++g) divide_pairs(P + g * PG, PG, s[g]);
    }

    if (FMT == FMT_MXQUEST && p.mask != nullptr) {
      // bit i set = element i lies inside the grid's range (|x / 2^e| < 6, triton/mxfp4.py:105-110)
      uint32_t inside = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float a, b;
        unpack2(P[j], a, b);
        inside |= (fabsf(a) < 6.0f ? 1u : 0u) << (2 * j);
        inside |= (fabsf(b) < 6.0f ? 1u : 0u) << (2 * j + 1);
      }
      if (active) {
        if (MODE == MODE_CODES) {
          reinterpret_cast<uint32_t*>(p.mask)[c] = inside;            // bit i of byte b = element 8 b + i
        } else {
          uint4* o = reinterpret_cast<uint4*>(p.mask) + c * 2;        // one bool byte per element
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t nib = (inside >> (16 * h + 4 * q)) & 15u;
              w[q] = (nib & 1u) | ((nib & 2u) << 7) | ((nib & 4u) << 14) | ((nib & 8u) << 21);
            }
            o[h] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }

    uint32_t cw[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) cw[q] = codes_word(P + 4 * q);

    if (MODE == MODE_CODES) {
      if (active) reinterpret_cast<uint4*>(p.codes)[c] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    } else {  // MODE_DEQUANT
      float out[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float sc = s[(i * NG) / 32];
        float v = __fmul_rn(e2m1_value((cw[i / 8] >> (4 * (i % 8))) & 15u), sc);
        if (p.ste) {
          float a, b;
          unpack2(Y[i / 2], a, b);
          const float x = (i & 1) ? b : a;
          v = __fadd_rn(x, __fsub_rn(v, x));
        }
        out[i] = v;
      }
      if (active) {
        if (p.out_bf16) {
          uint4* o = reinterpret_cast<uint4*>(p.y) + c * 4;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h = __floats2bfloat162_rn(out[8 * q + 2 * j], out[8 * q + 2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            o[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          float4* o = reinterpret_cast<float4*>(p.y) + c * 8;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            o[q] = make_float4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
        }
      }
    }
}

#ifndef FPQ_Q_PREFETCH
#define FPQ_Q_PREFETCH 1
#endif
#ifndef FPQ_Q_MINBLOCKS
#define FPQ_Q_MINBLOCKS 3
#endif

// A warp walks the chunks 32 at a time with a grid-wide stride.  For bf16 input the next chunk's
// sixteen words are loaded into a second register set before the current chunk is processed, so
// every thread keeps two 64-byte requests in flight.
template <bool IN_BF16, int MODE>
struct Prefetches { static constexpr bool value = FPQ_Q_PREFETCH && IN_BF16 && MODE != MODE_DEQUANT; };

template <int GH, int FMT, bool IN_BF16, int MODE>
__global__ void __launch_bounds__(256, Prefetches<IN_BF16, MODE>::value ? FPQ_Q_MINBLOCKS : 1) quant_kernel(const QuantParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t stride = (((int64_t)gridDim.x * blockDim.x) >> 5) * 32;
  launch_dependents();         // the next kernel may set itself up while this one runs
  grid_dependency_wait();      // the input (and the global scale) may come from the previous kernel
  float gs = 0.0f, rgs = 0.0f;
  if (FMT == FPQ_FMT_NVFP4 && (MODE == MODE_CODES || MODE == MODE_DEQUANT)) {
    gs = *p.gs;
    rgs = gs == 0.0f ? 0.0f : __frcp_rn(gs);
  }
  float running_max = 0.0f;

  int64_t cb = warp * 32;
  if (Prefetches<IN_BF16, MODE>::value) {
    RawChunk<IN_BF16> r0, r1;
    if (cb < p.n_chunks) load_raw(p.x, cb + lane, cb + lane < p.n_chunks, r0);
    while (cb < p.n_chunks) {
      int64_t nx = cb + stride + lane;
      load_raw(p.x, nx, nx < p.n_chunks, r1);
      process_chunk<GH, FMT, IN_BF16, MODE>(p, r0, cb + lane, cb + lane < p.n_chunks, lane, gs, rgs, running_max);
      cb += stride;
      if (cb >= p.n_chunks) break;
      nx = cb + stride + lane;
      load_raw(p.x, nx, nx < p.n_chunks, r0);
      process_chunk<GH, FMT, IN_BF16, MODE>(p, r1, cb + lane, cb + lane < p.n_chunks, lane, gs, rgs, running_max);
      cb += stride;
    }
  } else {
    for (; cb < p.n_chunks; cb += stride) {
      const int64_t c = cb + lane;
      RawChunk<IN_BF16> r;
      load_raw(p.x, c, c < p.n_chunks, r);
      process_chunk<GH, FMT, IN_BF16, MODE>(p, r, c, c < p.n_chunks, lane, gs, rgs, running_max);
    }
  }

  if (MODE == MODE_CODES && p.pad_rows != 0) {
    // swizzled scale bytes of the rows between the tensor's last row and the end of its 128-row block: zero
    // (the GEMM's TMA loads whole 512-byte tiles, and a defined value keeps its pad rows finite)
    const int64_t n_words = (int64_t)p.pad_rows * p.sf_tiles_per_row_block;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += (int64_t)gridDim.x * blockDim.x) {
      const uint32_t r = p.rows + (uint32_t)(w / p.sf_tiles_per_row_block);
      const uint32_t kb = (uint32_t)(w % p.sf_tiles_per_row_block);
      *reinterpret_cast<uint32_t*>(p.sbytes + swizzled_offset(r, kb * 4u, p.sf_tiles_per_row_block)) = 0u;
    }
  }

  if (MODE == MODE_ABSMAX) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      running_max = fmaxf(running_max, __shfl_xor_sync(0xffffffffu, running_max, o));
    if (lane == 0) atomicMax(p.absmax_bits, __float_as_uint(running_max));
  }
}

// ---------------------------------------------------------------------------------------------------
// SiLU(gate) * up fused in front of the rotate + quantise pass: the input of an MLP's down-projection
// (src/utils/llama_utils.py:62-70 of IST-DASLab/FP-Quant computes `act_fn(gate) * up`, rotates it and
// quantises it in three passes over memory).  The activation keeps the reference's rounding points: it is
// what torch computes for bf16 tensors, silu in fp32 rounded to bf16, then the product rounded to bf16;
// from there on the chunk goes through process_chunk like any bf16 input.
__device__ __forceinline__ uint32_t silu_mul_word(uint32_t g2, uint32_t u2) {
  const float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xffff0000u);
  const float u0 = __uint_as_float(u2 << 16), u1 = __uint_as_float(u2 & 0xffff0000u);
  // x / (1 + exp(-x)) with the library exponential and an IEEE division, as torch evaluates silu
  const float s0 = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(g0, __fadd_rn(1.0f, expf(-g0)))));
  const float s1 = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(g1, __fadd_rn(1.0f, expf(-g1)))));
  const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(s0, u0), __fmul_rn(s1, u1));
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int GH, int FMT>
__global__ void __launch_bounds__(256, 2) quant_silu_mul_kernel(const QuantParams p, const void* up) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t stride = (((int64_t)gridDim.x * blockDim.x) >> 5) * 32;
  launch_dependents();
  grid_dependency_wait();
  float gs = 0.0f, rgs = 0.0f;
  if (FMT == FPQ_FMT_NVFP4) {
    gs = *p.gs;
    rgs = gs == 0.0f ? 0.0f : __frcp_rn(gs);
  }
  float unused_max = 0.0f;
  int64_t cb = warp * 32;
  RawChunk<true> g, u;
  if (cb < p.n_chunks) {
    load_raw(p.x, cb + lane, cb + lane < p.n_chunks, g);
    load_raw(up, cb + lane, cb + lane < p.n_chunks, u);
  }
  while (cb < p.n_chunks) {
    RawChunk<true> h;
#pragma unroll
    for (int j = 0; j < 16; ++j) h.w[j] = silu_mul_word(g.w[j], u.w[j]);
    const int64_t nx = cb + stride + lane;          // the next chunk's loads fly while this one is quantised
    load_raw(p.x, nx, nx < p.n_chunks, g);
    load_raw(up, nx, nx < p.n_chunks, u);
    process_chunk<GH, FMT, true, MODE_CODES>(p, h, cb + lane, cb + lane < p.n_chunks, lane, gs, rgs, unused_max);
    cb += stride;
  }
  if (p.pad_rows != 0) {
    const int64_t n_words = (int64_t)p.pad_rows * p.sf_tiles_per_row_block;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += (int64_t)gridDim.x * blockDim.x) {
      const uint32_t r = p.rows + (uint32_t)(w / p.sf_tiles_per_row_block);
      const uint32_t kb = (uint32_t)(w % p.sf_tiles_per_row_block);
      *reinterpret_cast<uint32_t*>(p.sbytes + swizzled_offset(r, kb * 4u, p.sf_tiles_per_row_block)) = 0u;
    }
  }
}

template <int GH, int FMT>
int launch_silu_mul(const QuantParams& params, const void* up, cudaStream_t stream) {
  QuantParams p = params;
  p.row_magic = (p.chunks_per_row >= 2 && p.n_chunks < (1ll << 32)) ? ~0ull / p.chunks_per_row + 1 : 0;
  const int64_t blocks_needed = ceil_div64(ceil_div64(p.n_chunks, 32), 8);
  int64_t blocks = (int64_t)sm_count() * 2;          // persistent: the two resident blocks per SM
  if (blocks > blocks_needed) blocks = blocks_needed;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_dependent_launch() ? 1 : 0;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, quant_silu_mul_kernel<GH, FMT>, p, up));
  return FPQ_OK;
}

// ---------------------------------------------------------------------------------------------------
// Quantise the TRANSPOSE of a bf16 matrix: x [t_rows, n] row-major -> MXFP4 of x^T [n, t_pad], rotated and
// scaled along the t axis (groups of 32 consecutive rows of x), without materialising x^T.  This is what
// the weight-gradient GEMM of the quantised backward pass needs of the upstream gradient
// (backward_t_bf16, inference_lib/src/fp_quant/module/qutlass_ops.py:218-245 of IST-DASLab/FP-Quant).
// A warp takes a 32 x 32 tile of x (32 rows of 64 bytes), turns it round through shared memory, and every
// lane then owns one output chunk: 32 consecutive t of one column of x, i.e. exactly the chunk
// process_chunk expects.  Rows of x beyond t_rows read as zero (t_pad may exceed t_rows).  The rotation must
// stay inside a chunk: group 0, 16 or 32.
constexpr int TQ_ROW_BYTES = 64 + 16;      // a tile row in shared memory, padded against bank conflicts

template <int GH, int FMT>
__global__ void __launch_bounds__(256, 2) quant_transposed_kernel(const QuantParams p, int64_t t_rows, int64_t n) {
  static_assert(GH == 0 || GH == 16 || GH == 32, "the rotation group must fit one 32-element chunk");
  __shared__ __align__(16) uint8_t tiles[8][32 * TQ_ROW_BYTES];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  uint8_t* tile = tiles[wib];
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  launch_dependents();
  grid_dependency_wait();
  const int64_t col_tiles = (n + 31) / 32, t_tiles = p.chunks_per_row;      // tiles along x's columns / rows
  float unused_max = 0.0f;
  // tile index = t_tile * col_tiles + col_tile: neighbouring warps read neighbouring 64-byte pieces of the same rows
  for (int64_t tix = warp; tix < col_tiles * t_tiles; tix += n_warps) {
    const int64_t tt = tix / col_tiles, ct = tix - tt * col_tiles;
    const int64_t t0 = tt * 32, j0 = ct * 32;
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = q * 8 + (lane >> 2), piece = lane & 3;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t0 + row < t_rows && j0 + piece * 8 < n)
        v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x) + (t0 + row) * n + j0 + piece * 8);
      *reinterpret_cast<uint4*>(tile + row * TQ_ROW_BYTES + piece * 16) = v;
    }
    __syncwarp();
    RawChunk<true> raw;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t lo = *reinterpret_cast<const uint16_t*>(tile + (2 * k) * TQ_ROW_BYTES + lane * 2);
      const uint32_t hi = *reinterpret_cast<const uint16_t*>(tile + (2 * k + 1) * TQ_ROW_BYTES + lane * 2);
      raw.w[k] = lo | (hi << 16);
    }
    const int64_t out_row = j0 + lane;
    const bool active = out_row < n;
    process_chunk<GH, FMT, true, MODE_CODES>(p, raw, active ? out_row * p.chunks_per_row + tt : 0, active, lane, 0.0f, 0.0f,
                                             unused_max);
  }
  if (p.pad_rows != 0) {
    const int64_t n_words = (int64_t)p.pad_rows * p.sf_tiles_per_row_block;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += (int64_t)gridDim.x * blockDim.x) {
      const uint32_t r = p.rows + (uint32_t)(w / p.sf_tiles_per_row_block);
      const uint32_t kb = (uint32_t)(w % p.sf_tiles_per_row_block);
      *reinterpret_cast<uint32_t*>(p.sbytes + swizzled_offset(r, kb * 4u, p.sf_tiles_per_row_block)) = 0u;
    }
  }
}

template <int GH>
int launch_transposed(const QuantParams& params, int64_t t_rows, int64_t n, cudaStream_t stream) {
  QuantParams p = params;
  p.row_magic = (p.chunks_per_row >= 2 && p.n_chunks < (1ll << 32)) ? ~0ull / p.chunks_per_row + 1 : 0;
  const int64_t tiles = ((n + 31) / 32) * (int64_t)p.chunks_per_row;
  int64_t blocks = (int64_t)sm_count() * 2;          // persistent: two resident blocks of eight warps per SM
  if (blocks > ceil_div64(tiles, 8)) blocks = ceil_div64(tiles, 8);
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_dependent_launch() ? 1 : 0;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, quant_transposed_kernel<GH, FPQ_FMT_MXFP4>, p, t_rows, n));
  return FPQ_OK;
}

template <int FMT>
int launch_silu_mul_gh(int gh, const QuantParams& p, const void* up, cudaStream_t stream) {
  switch (gh) {
    case 0: return launch_silu_mul<0, FMT>(p, up, stream);
    case 16: return launch_silu_mul<16, FMT>(p, up, stream);
    case 32: return launch_silu_mul<32, FMT>(p, up, stream);
    case 64: return launch_silu_mul<64, FMT>(p, up, stream);
    case 128: return launch_silu_mul<128, FMT>(p, up, stream);
  }
  set_error("hadamard_group must be 0, 16, 32, 64 or 128 (got %d)", gh);
  return FPQ_ERR_INVALID_ARGUMENT;
}

template <int GH, int FMT, bool IN_BF16, int MODE>
int launch_one(const QuantParams& params, cudaStream_t stream) {
  QuantParams p = params;
  p.row_magic = (p.chunks_per_row >= 2 && p.n_chunks < (1ll << 32)) ? ~0ull / p.chunks_per_row + 1 : 0;
  // persistent grid: exactly the number of blocks that are resident at once
  static int resident[64] = {};
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  int per_sm = dev < 64 ? resident[dev] : 0;
  if (per_sm == 0) {
    FPQ_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_kernel<GH, FMT, IN_BF16, MODE>, 256, 0));
    if (per_sm < 1) per_sm = 1;
    if (dev < 64) resident[dev] = per_sm;
  }
  const int64_t warps_needed = ceil_div64(p.n_chunks, 32);
  const int64_t blocks_needed = ceil_div64(warps_needed, 8);
  int64_t blocks = (int64_t)sm_count() * per_sm;
  if (blocks > blocks_needed) blocks = blocks_needed;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_dependent_launch() ? 1 : 0;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, quant_kernel<GH, FMT, IN_BF16, MODE>, p));
  return FPQ_OK;
}

template <int FMT, bool IN_BF16, int MODE>
int launch_gh(int gh, const QuantParams& p, cudaStream_t stream) {
  switch (gh) {
    case 0: return launch_one<0, FMT, IN_BF16, MODE>(p, stream);
    case 16: return launch_one<16, FMT, IN_BF16, MODE>(p, stream);
    case 32: return launch_one<32, FMT, IN_BF16, MODE>(p, stream);
    case 64: return launch_one<64, FMT, IN_BF16, MODE>(p, stream);
    case 128: return launch_one<128, FMT, IN_BF16, MODE>(p, stream);
  }
  set_error("hadamard_group must be 0, 16, 32, 64 or 128 (got %d)", gh);
  return FPQ_ERR_INVALID_ARGUMENT;
}

template <int MODE>
int launch_mode(int gh, int fmt, int dtype, const QuantParams& p, cudaStream_t stream) {
  if constexpr (MODE == MODE_ROTATE || MODE == MODE_ABSMAX) {
    return dtype == FPQ_DT_BF16 ? launch_gh<FPQ_FMT_MXFP4, true, MODE>(gh, p, stream)
                                : launch_gh<FPQ_FMT_MXFP4, false, MODE>(gh, p, stream);
  } else {
    if (fmt == FMT_MXQUEST)
      return dtype == FPQ_DT_BF16 ? launch_gh<FMT_MXQUEST, true, MODE>(gh, p, stream)
                                  : launch_gh<FMT_MXQUEST, false, MODE>(gh, p, stream);
    if (fmt == FPQ_FMT_MXFP4)
      return dtype == FPQ_DT_BF16 ? launch_gh<FPQ_FMT_MXFP4, true, MODE>(gh, p, stream)
                                  : launch_gh<FPQ_FMT_MXFP4, false, MODE>(gh, p, stream);
    return dtype == FPQ_DT_BF16 ? launch_gh<FPQ_FMT_NVFP4, true, MODE>(gh, p, stream)
                                : launch_gh<FPQ_FMT_NVFP4, false, MODE>(gh, p, stream);
  }
}

int check_common(const void* x, int dtype, int64_t rows, int64_t cols, int gh) {
  FPQ_CHECK_ARG(x != nullptr, "x is NULL");
  FPQ_CHECK_ARG(dtype == FPQ_DT_BF16 || dtype == FPQ_DT_F32, "dtype must be FPQ_DT_BF16 or FPQ_DT_F32");
  FPQ_CHECK_ARG(rows >= 0 && cols > 0, "bad shape [%lld, %lld]", (long long)rows, (long long)cols);
  FPQ_CHECK_ARG(cols % 32 == 0, "cols (%lld) must be a multiple of 32", (long long)cols);
  FPQ_CHECK_ARG(gh == 0 || gh == 16 || gh == 32 || gh == 64 || gh == 128,
                "hadamard_group must be 0, 16, 32, 64 or 128 (got %d)", gh);
  FPQ_CHECK_ARG(gh == 0 || cols % gh == 0, "cols (%lld) must be a multiple of the hadamard group %d",
                (long long)cols, gh);
  FPQ_CHECK_ARG(((uintptr_t)x & 31) == 0, "x must be 32-byte aligned");
  FPQ_CHECK_ARG(rows * cols / 32 < (int64_t)1 << 40, "tensor too large");
  return FPQ_OK;
}

// ------------------------------------------------------------------ auxiliary kernels
__global__ void global_scale_update_kernel(const uint32_t* absmax_bits, float* gs, int32_t* status) {
  float a = __uint_as_float(*absmax_bits);
  if (a == 0.0f) {
    if (status) *status = 1;
    return;
  }
  float cur = __fmul_rn(2688.0f, __fdiv_rn(1.0f, a));
  *gs = fminf(*gs, cur);
  if (status) *status = 0;
}

template <bool IN_BF16>
__global__ void __launch_bounds__(256) apply_scales_kernel(const void* x, int64_t n_words, uint32_t cols,
                                                           const float* scales, uint32_t group, int out_kind,
                                                           void* out) {
  // one thread per 8 consecutive elements (one word of codes)
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words;
       w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e0 = w * 8;
    const int64_t row = e0 / cols;
    const uint32_t col = (uint32_t)(e0 - row * cols);
    const float* srow = scales + row * (cols / group);
    const bool one_scale = (group & 7u) == 0;   // the 8 elements share a scale
    const float s0 = srow[col / group];
    float v[8];
    if (IN_BF16) {
      uint4 raw = reinterpret_cast<const uint4*>(x)[w];
      const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(r[j] << 16);
        v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
      }
    } else {
      float4 a = reinterpret_cast<const float4*>(x)[2 * w], b = reinterpret_cast<const float4*>(x)[2 * w + 1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    uint32_t word = 0;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = one_scale ? s0 : srow[(col + j) / group];
      const uint32_t code = e2m1_code(__fdiv_rn(v[j], s));
      word |= code << (4 * j);
      float g = e2m1_value(code);
      if (out_kind == FPQ_OUT_GRID) o[j] = g;
      else {
        float d = __fmul_rn(g, s);
        o[j] = out_kind == FPQ_OUT_DEQUANT_STE ? __fadd_rn(v[j], __fsub_rn(d, v[j])) : d;
      }
    }
    if (out_kind == FPQ_OUT_CODES) {
      reinterpret_cast<uint32_t*>(out)[w] = word;
    } else if (IN_BF16) {
      uint32_t r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
        r[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(out)[w] = make_uint4(r[0], r[1], r[2], r[3]);
    } else {
      reinterpret_cast<float4*>(out)[2 * w] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(out)[2 * w + 1] = make_float4(o[4], o[5], o[6], o[7]);
    }
  }
}

template <bool IN_BF16>
__global__ void __launch_bounds__(256) pack_grid_kernel(const void* q, int64_t n_words, uint32_t* packed) {
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words;
       w += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    if (IN_BF16) {
      uint4 raw = reinterpret_cast<const uint4*>(q)[w];
      const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(r[j] << 16);
        v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
      }
    } else {
      float4 a = reinterpret_cast<const float4*>(q)[2 * w], b = reinterpret_cast<const float4*>(q)[2 * w + 1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) word |= e2m1_code(v[j]) << (4 * j);
    packed[w] = word;
  }
}

__global__ void __launch_bounds__(256) swizzle_scales_kernel(const uint8_t* __restrict__ src, uint32_t rows,
                                                             uint32_t sf_cols, uint32_t rows_pad,
                                                             uint32_t tiles_per_row_block,
                                                             uint32_t* __restrict__ dst) {
  // one thread per destination word (4 scale bytes of one row inside one tile)
  const int64_t n_words = (int64_t)rows_pad * tiles_per_row_block;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words;
       w += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t tile = (uint32_t)(w >> 7), in_tile = (uint32_t)(w & 127);
    const uint32_t rb = tile / tiles_per_row_block, kb = tile - rb * tiles_per_row_block;
    const uint32_t row = rb * 128 + (in_tile & 3u) * 32 + (in_tile >> 2);
    uint32_t word = 0;
    if (row < rows) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t c = kb * 4 + j;
        if (c < sf_cols) word |= (uint32_t)src[(size_t)row * sf_cols + c] << (8 * j);
      }
    }
    dst[w] = word;
  }
}

__global__ void __launch_bounds__(128) rotate_dense_kernel(const void* x, int in_bf16, void* y, int out_bf16,
                                                           int64_t n_groups, int g, const float* matrix) {
  // one warp per group; the g x g matrix lives in shared memory
  extern __shared__ float sm[];
  float* M = sm;                  // g * g
  float* xs = sm + g * g;         // 4 warps * g
  for (int i = threadIdx.x; i < g * g; i += blockDim.x) M[i] = matrix[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float* xw = xs + wid * g;
  for (int64_t grp = (int64_t)blockIdx.x * 4 + wid; grp < n_groups; grp += (int64_t)gridDim.x * 4) {
    for (int i = lane; i < g; i += 32)
      xw[i] = in_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[grp * g + i])
                      : reinterpret_cast<const float*>(x)[grp * g + i];
    __syncwarp();
    for (int j = lane; j < g; j += 32) {
      float acc = 0.0f;
      for (int k = 0; k < g; ++k) acc = __fadd_rn(acc, __fmul_rn(xw[k], M[k * g + j]));
      if (out_bf16) reinterpret_cast<__nv_bfloat16*>(y)[grp * g + j] = __float2bfloat16_rn(acc);
      else reinterpret_cast<float*>(y)[grp * g + j] = acc;
    }
    __syncwarp();
  }
}

int grid_for(int64_t work_items, int threads);

// ------------------------------------------------------------------ MSE observer
// One thread per scale group.  Candidates fl(f_i * s0), f_i = 1 - i * max_shrink / iters evaluated in double
// and rounded to fp32 as the reference's Python float is by the tensor multiply; error
// sum_j |x_j - grid(fl(x_j / s)) * s| ^ norm; the first strictly smaller error wins; the winner then goes
// through the scale-precision chain (src/quantization/quantizer.py:117-134, :143-165).  The candidates are
// not rounded to E4M3 / E8M0 during the search.
template <int G, bool NV, bool IN_BF16>
__global__ void __launch_bounds__(128) mse_scales_kernel(const void* __restrict__ x, int64_t n_groups,
                                                         const float* __restrict__ gs_ptr, int iters, double max_shrink,
                                                         float norm, float* __restrict__ scales_out) {
  float gs = 0.0f, rgs = 0.0f;
  if (NV) {
    gs = *gs_ptr;
    rgs = gs == 0.0f ? 0.0f : __fdiv_rn(1.0f, gs);
  }
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += (int64_t)gridDim.x * blockDim.x) {
    float v[G];
    if (IN_BF16) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + g * G);
#pragma unroll
      for (int q = 0; q < G / 8; ++q) {
        const uint4 raw = src[q];
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[8 * q + 2 * j] = __uint_as_float(r[j] << 16);
          v[8 * q + 2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
        }
      }
    } else {
      const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + g * G);
#pragma unroll
      for (int q = 0; q < G / 4; ++q) {
        const float4 t = src[q];
        v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
      }
    }
    float a = 0.0f;
#pragma unroll
    for (int j = 0; j < G; ++j) a = fmaxf(a, fabsf(v[j]));
    const float s0 = __fdiv_rn(__fmul_rn(2.0f, a), 12.0f);
    float best = s0, best_err = __int_as_float(0x7f800000);
    if (s0 != 0.0f) {                         // an all-zero group divides 0 by 0: no candidate is ever "better"
      for (int i = 0; i < iters; ++i) {
        const float f = (float)(1.0 - (double)i * max_shrink / (double)iters);
        const float s = __fmul_rn(f, s0);
        float err = 0.0f;
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const float gv = e2m1_value(e2m1_code(__fdiv_rn(v[j], s)));
          const float d = fabsf(__fsub_rn(v[j], __fmul_rn(gv, s)));
          err = __fadd_rn(err, powf(d, norm));
        }
        if (err < best_err) {
          best_err = err;
          best = s;
        }
      }
    }
    uint32_t byte;
    float out;
    if (NV) {
      float t = fminf(fmaxf(__fmul_rn(best, gs), -448.0f), 448.0f);
      uint16_t u2;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(u2) : "f"(0.0f), "f"(t));
      const uint32_t u = u2 & 0xffu, ex = u >> 3, ma = u & 7u;
      const float uf = ex == 0 ? (float)ma * 0.001953125f : __uint_as_float(((ex + 120u) << 23) | (ma << 20));
      out = __fmul_rn(uf, rgs);
      byte = u;
    } else {
      const float m = fmaxf(__fmul_rn(6.0f, best), 1.17549435e-38f);
      const int e = mx_exponent(m);
      out = e >= -124 ? __uint_as_float(((uint32_t)(e + 125) << 23) | 0x2aaaabu) : __fdiv_rn(ldexpf(1.0f, e - 2), 0.75f);
      byte = (uint32_t)(e + 127);
    }
    (void)byte;
    scales_out[g] = out == 0.0f ? 1.0f : out;
  }
}

template <int G, bool NV>
int launch_mse(const void* x, int dtype, int64_t n_groups, const float* gs, int iters, double max_shrink, float norm,
               float* out, cudaStream_t st) {
  const int grid = grid_for(n_groups, 128);
  if (dtype == FPQ_DT_BF16)
    mse_scales_kernel<G, NV, true><<<grid, 128, 0, st>>>(x, n_groups, gs, iters, max_shrink, norm, out);
  else
    mse_scales_kernel<G, NV, false><<<grid, 128, 0, st>>>(x, n_groups, gs, iters, max_shrink, norm, out);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

int grid_for(int64_t work_items, int threads) {
  int64_t b = ceil_div64(work_items, threads);
  int64_t cap = (int64_t)sm_count() * 16;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace
}  // namespace fpq

using namespace fpq;

extern "C" int fpq_rotate_hadamard(const void* x, int dtype_in, void* y, int dtype_out, int64_t rows,
                                   int64_t cols, int group, fpq_stream_t stream) {
  if (int rc = check_common(x, dtype_in, rows, cols, group)) return rc;
  FPQ_CHECK_ARG(group != 0, "group must be 16, 32, 64 or 128");
  FPQ_CHECK_ARG(y != nullptr && ((uintptr_t)y & 15) == 0, "y must be non-NULL and 16-byte aligned");
  FPQ_CHECK_ARG(dtype_out == FPQ_DT_BF16 || dtype_out == FPQ_DT_F32, "bad dtype_out");
  FPQ_CHECK_ARG(x != y || dtype_in == dtype_out, "in-place rotation needs equal dtypes");
  if (rows == 0) return FPQ_OK;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.y = y;
  p.out_bf16 = dtype_out == FPQ_DT_BF16;
  return launch_mode<MODE_ROTATE>(group, 0, dtype_in, p, (cudaStream_t)stream);
}

extern "C" int fpq_rotate_dense(const void* x, int dtype_in, void* y, int dtype_out, int64_t rows,
                                int64_t cols, int group, const float* matrix, fpq_stream_t stream) {
  FPQ_CHECK_ARG(x && y && matrix, "NULL pointer");
  FPQ_CHECK_ARG(group == 16 || group == 32 || group == 64 || group == 128, "group must be 16, 32, 64 or 128");
  FPQ_CHECK_ARG(rows >= 0 && cols > 0 && cols % group == 0, "cols must be a multiple of group");
  FPQ_CHECK_ARG(x != y, "fpq_rotate_dense cannot run in place");
  if (rows == 0) return FPQ_OK;
  const int64_t n_groups = rows * cols / group;
  const size_t smem = (size_t)(group * group + 4 * group) * sizeof(float);
  FPQ_CHECK_CUDA(cudaFuncSetAttribute(rotate_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  rotate_dense_kernel<<<grid_for(n_groups, 4), 128, smem, (cudaStream_t)stream>>>(
      x, dtype_in == FPQ_DT_BF16, y, dtype_out == FPQ_DT_BF16, n_groups, group, matrix);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_absmax(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                          uint32_t* absmax_bits, fpq_stream_t stream) {
  if (int rc = check_common(x, dtype, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(absmax_bits != nullptr, "absmax_bits is NULL");
  if (rows == 0) return FPQ_OK;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.absmax_bits = absmax_bits;
  return launch_mode<MODE_ABSMAX>(hadamard_group, 0, dtype, p, (cudaStream_t)stream);
}

extern "C" int fpq_global_scale_update(const uint32_t* absmax_bits, float* global_scale, int32_t* status,
                                       fpq_stream_t stream) {
  FPQ_CHECK_ARG(absmax_bits && global_scale, "NULL pointer");
  global_scale_update_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(absmax_bits, global_scale, status);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                            int format, const float* global_scale, uint8_t* codes, uint8_t* scale_bytes,
                            int scale_layout, float* scales_f32, fpq_stream_t stream) {
  if (int rc = check_common(x, dtype, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(format == FPQ_FMT_MXFP4 || format == FPQ_FMT_NVFP4, "format must be FPQ_FMT_MXFP4 or FPQ_FMT_NVFP4");
  FPQ_CHECK_ARG(format != FPQ_FMT_NVFP4 || global_scale != nullptr, "NVFP4 needs a global_scale pointer");
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale_layout");
  FPQ_CHECK_ARG(codes || scale_bytes || scales_f32, "no output requested");
  FPQ_CHECK_ARG(((uintptr_t)codes & 15) == 0 && ((uintptr_t)scale_bytes & 15) == 0 && ((uintptr_t)scales_f32 & 15) == 0,
                "outputs must be 16-byte aligned");
  if (rows == 0) return FPQ_OK;
  const int g = format == FPQ_FMT_NVFP4 ? 16 : 32;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.codes = codes;
  p.sbytes = scale_bytes;
  p.sf32 = scales_f32;
  p.gs = global_scale;
  p.sf_tiles_per_row_block = (uint32_t)ceil_div64(cols / g, 4);
  p.layout = scale_layout;
  if (scale_bytes && scale_layout == FPQ_SCALES_SWIZZLED) {
    FPQ_CHECK_ARG(rows < ((int64_t)1 << 31), "too many rows for the swizzled scale layout");
    p.rows = (uint32_t)rows;
    p.pad_rows = (uint32_t)(ceil_div64(rows, 128) * 128 - rows);
  }
  return launch_mode<MODE_CODES>(hadamard_group, format, dtype, p, (cudaStream_t)stream);
}

extern "C" int fpq_quantize_silu_mul(const void* gate_bf16, const void* up_bf16, int64_t rows, int64_t cols,
                                     int hadamard_group, int format, const float* global_scale, uint8_t* codes,
                                     uint8_t* scale_bytes, int scale_layout, fpq_stream_t stream) {
  if (int rc = check_common(gate_bf16, FPQ_DT_BF16, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(up_bf16 != nullptr && ((uintptr_t)up_bf16 & 31) == 0, "up must be non-NULL and 32-byte aligned");
  FPQ_CHECK_ARG(format == FPQ_FMT_MXFP4 || format == FPQ_FMT_NVFP4, "format must be FPQ_FMT_MXFP4 or FPQ_FMT_NVFP4");
  FPQ_CHECK_ARG(format != FPQ_FMT_NVFP4 || global_scale != nullptr, "NVFP4 needs a global_scale pointer");
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale_layout");
  FPQ_CHECK_ARG(codes != nullptr && scale_bytes != nullptr, "codes and scale_bytes are required");
  FPQ_CHECK_ARG(((uintptr_t)codes & 15) == 0 && ((uintptr_t)scale_bytes & 15) == 0, "outputs must be 16-byte aligned");
  if (rows == 0) return FPQ_OK;
  const int g = format == FPQ_FMT_NVFP4 ? 16 : 32;
  QuantParams p{};
  p.x = gate_bf16;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.codes = codes;
  p.sbytes = scale_bytes;
  p.gs = global_scale;
  p.sf_tiles_per_row_block = (uint32_t)ceil_div64(cols / g, 4);
  p.layout = scale_layout;
  if (scale_layout == FPQ_SCALES_SWIZZLED) {
    FPQ_CHECK_ARG(rows < ((int64_t)1 << 31), "too many rows for the swizzled scale layout");
    p.rows = (uint32_t)rows;
    p.pad_rows = (uint32_t)(ceil_div64(rows, 128) * 128 - rows);
  }
  return format == FPQ_FMT_NVFP4 ? launch_silu_mul_gh<FPQ_FMT_NVFP4>(hadamard_group, p, up_bf16, (cudaStream_t)stream)
                                 : launch_silu_mul_gh<FPQ_FMT_MXFP4>(hadamard_group, p, up_bf16, (cudaStream_t)stream);
}

extern "C" int fpq_quantize_transposed(const void* x_bf16, int64_t t_rows, int64_t n, int64_t t_pad, int hadamard_group,
                                       uint8_t* codes, uint8_t* scale_bytes, int scale_layout, fpq_stream_t stream) {
  FPQ_CHECK_ARG(x_bf16 && codes && scale_bytes, "NULL pointer");
  FPQ_CHECK_ARG(t_rows > 0 && n > 0 && n % 8 == 0, "n (%lld) must be a positive multiple of 8", (long long)n);
  FPQ_CHECK_ARG(t_pad >= t_rows && t_pad % 32 == 0, "t_pad (%lld) must be a multiple of 32 not below t_rows", (long long)t_pad);
  FPQ_CHECK_ARG(hadamard_group == 0 || hadamard_group == 16 || hadamard_group == 32,
                "the rotation group of the transposing quantiser must be 0, 16 or 32 (got %d)", hadamard_group);
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale_layout");
  FPQ_CHECK_ARG(((uintptr_t)x_bf16 & 15) == 0 && ((uintptr_t)codes & 15) == 0 && ((uintptr_t)scale_bytes & 15) == 0,
                "pointers must be 16-byte aligned");
  FPQ_CHECK_ARG(n < ((int64_t)1 << 31) && t_pad < ((int64_t)1 << 31), "shape too large");
  QuantParams p{};
  p.x = x_bf16;
  p.n_chunks = n * t_pad / 32;
  p.chunks_per_row = (uint32_t)(t_pad / 32);
  p.codes = codes;
  p.sbytes = scale_bytes;
  p.sf_tiles_per_row_block = (uint32_t)ceil_div64(t_pad / 32, 4);
  p.layout = scale_layout;
  if (scale_layout == FPQ_SCALES_SWIZZLED) {
    p.rows = (uint32_t)n;
    p.pad_rows = (uint32_t)(ceil_div64(n, 128) * 128 - n);
  }
  switch (hadamard_group) {
    case 0: return launch_transposed<0>(p, t_rows, n, (cudaStream_t)stream);
    case 16: return launch_transposed<16>(p, t_rows, n, (cudaStream_t)stream);
    default: return launch_transposed<32>(p, t_rows, n, (cudaStream_t)stream);
  }
}

extern "C" int fpq_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                                 int format, const float* global_scale, void* y, int ste, fpq_stream_t stream) {
  if (int rc = check_common(x, dtype, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(format == FPQ_FMT_MXFP4 || format == FPQ_FMT_NVFP4, "format must be FPQ_FMT_MXFP4 or FPQ_FMT_NVFP4");
  FPQ_CHECK_ARG(format != FPQ_FMT_NVFP4 || global_scale != nullptr, "NVFP4 needs a global_scale pointer");
  FPQ_CHECK_ARG(y != nullptr && ((uintptr_t)y & 15) == 0, "y must be non-NULL and 16-byte aligned");
  if (rows == 0) return FPQ_OK;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.y = y;
  p.gs = global_scale;
  p.out_bf16 = dtype == FPQ_DT_BF16;
  p.ste = ste;
  return launch_mode<MODE_DEQUANT>(hadamard_group, format, dtype, p, (cudaStream_t)stream);
}

extern "C" int fpq_quantize_quest(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                                  uint8_t* codes, uint8_t* scale_bytes, int scale_layout, uint8_t* clip_mask,
                                  fpq_stream_t stream) {
  if (int rc = check_common(x, dtype, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(scale_layout == FPQ_SCALES_ROWMAJOR || scale_layout == FPQ_SCALES_SWIZZLED, "bad scale_layout");
  FPQ_CHECK_ARG(codes != nullptr, "codes is NULL");
  FPQ_CHECK_ARG(((uintptr_t)codes & 15) == 0 && ((uintptr_t)scale_bytes & 15) == 0 && ((uintptr_t)clip_mask & 3) == 0,
                "codes and scale_bytes must be 16-byte aligned, clip_mask 4-byte aligned");
  if (rows == 0) return FPQ_OK;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.codes = codes;
  p.sbytes = scale_bytes;
  p.mask = clip_mask;
  p.sf_tiles_per_row_block = (uint32_t)ceil_div64(cols / 32, 4);
  p.layout = scale_layout;
  if (scale_bytes && scale_layout == FPQ_SCALES_SWIZZLED) {
    FPQ_CHECK_ARG(rows < ((int64_t)1 << 31), "too many rows for the swizzled scale layout");
    p.rows = (uint32_t)rows;
    p.pad_rows = (uint32_t)(ceil_div64(rows, 128) * 128 - rows);
  }
  return launch_mode<MODE_CODES>(hadamard_group, FMT_MXQUEST, dtype, p, (cudaStream_t)stream);
}

extern "C" int fpq_fake_quantize_quest(const void* x, int dtype, int64_t rows, int64_t cols, int hadamard_group,
                                       void* y, uint8_t* clip_mask, fpq_stream_t stream) {
  if (int rc = check_common(x, dtype, rows, cols, hadamard_group)) return rc;
  FPQ_CHECK_ARG(y != nullptr && ((uintptr_t)y & 15) == 0, "y must be non-NULL and 16-byte aligned");
  FPQ_CHECK_ARG(((uintptr_t)clip_mask & 15) == 0, "clip_mask must be 16-byte aligned");
  if (rows == 0) return FPQ_OK;
  QuantParams p{};
  p.x = x;
  p.n_chunks = rows * cols / 32;
  p.chunks_per_row = (uint32_t)(cols / 32);
  p.y = y;
  p.mask = clip_mask;
  p.out_bf16 = dtype == FPQ_DT_BF16;
  return launch_mode<MODE_DEQUANT>(hadamard_group, FMT_MXQUEST, dtype, p, (cudaStream_t)stream);
}

extern "C" int fpq_apply_scales(const void* x, int dtype, int64_t rows, int64_t cols, const float* scales,
                                int group, int out_kind, void* out, fpq_stream_t stream) {
  FPQ_CHECK_ARG(x && scales && out, "NULL pointer");
  FPQ_CHECK_ARG(dtype == FPQ_DT_BF16 || dtype == FPQ_DT_F32, "bad dtype");
  FPQ_CHECK_ARG(rows >= 0 && cols > 0 && group > 0 && cols % group == 0 && cols % 8 == 0,
                "group (%d) must divide cols (%lld) and cols must be a multiple of 8", group, (long long)cols);
  FPQ_CHECK_ARG(out_kind >= FPQ_OUT_CODES && out_kind <= FPQ_OUT_DEQUANT_STE, "bad out_kind");
  FPQ_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0, "x and out must be 16-byte aligned");
  FPQ_CHECK_ARG(cols < ((int64_t)1 << 31), "cols too large");
  if (rows == 0) return FPQ_OK;
  const int64_t n_words = rows * cols / 8;
  const int grid = grid_for(n_words, 256);
  if (dtype == FPQ_DT_BF16)
    apply_scales_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(x, n_words, (uint32_t)cols, scales, (uint32_t)group, out_kind, out);
  else
    apply_scales_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(x, n_words, (uint32_t)cols, scales, (uint32_t)group, out_kind, out);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_mse_scales(const void* x, int dtype, int64_t rows, int64_t cols, int format,
                              const float* global_scale, int iters, double max_shrink, float error_norm,
                              float* scales_f32, fpq_stream_t stream) {
  FPQ_CHECK_ARG(x && scales_f32, "NULL pointer");
  FPQ_CHECK_ARG(dtype == FPQ_DT_BF16 || dtype == FPQ_DT_F32, "bad dtype");
  FPQ_CHECK_ARG(format == FPQ_FMT_NVFP4 || format == FPQ_FMT_MXFP4, "bad format");
  FPQ_CHECK_ARG(format != FPQ_FMT_NVFP4 || global_scale != nullptr, "NVFP4 needs the tensor scale");
  FPQ_CHECK_ARG(rows >= 0 && cols > 0 && cols % 32 == 0, "cols must be a multiple of 32");
  FPQ_CHECK_ARG(iters > 0 && iters <= 100000 && max_shrink >= 0.0 && max_shrink < 1.0, "bad search parameters");
  FPQ_CHECK_ARG(((uintptr_t)x & 15) == 0, "x must be 16-byte aligned");
  if (rows == 0) return FPQ_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (format == FPQ_FMT_NVFP4)
    return launch_mse<16, true>(x, dtype, rows * cols / 16, global_scale, iters, max_shrink, error_norm, scales_f32, st);
  return launch_mse<32, false>(x, dtype, rows * cols / 32, nullptr, iters, max_shrink, error_norm, scales_f32, st);
}

extern "C" int fpq_pack_grid(const void* q, int dtype, int64_t rows, int64_t cols, uint8_t* packed,
                             fpq_stream_t stream) {
  FPQ_CHECK_ARG(q && packed, "NULL pointer");
  FPQ_CHECK_ARG(dtype == FPQ_DT_BF16 || dtype == FPQ_DT_F32, "bad dtype");
  FPQ_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0, "cols must be a multiple of 8");
  FPQ_CHECK_ARG(((uintptr_t)q & 15) == 0 && ((uintptr_t)packed & 3) == 0, "bad alignment");
  if (rows == 0) return FPQ_OK;
  const int64_t n_words = rows * cols / 8;
  const int grid = grid_for(n_words, 256);
  if (dtype == FPQ_DT_BF16)
    pack_grid_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(q, n_words, reinterpret_cast<uint32_t*>(packed));
  else
    pack_grid_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(q, n_words, reinterpret_cast<uint32_t*>(packed));
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_swizzle_scales(const uint8_t* rowmajor, int64_t rows, int64_t sf_cols, uint8_t* swizzled,
                                  fpq_stream_t stream) {
  FPQ_CHECK_ARG(rowmajor && swizzled, "NULL pointer");
  FPQ_CHECK_ARG(rows > 0 && sf_cols > 0 && rows < ((int64_t)1 << 31) && sf_cols < ((int64_t)1 << 31), "bad shape");
  FPQ_CHECK_ARG(((uintptr_t)swizzled & 3) == 0, "swizzled must be 4-byte aligned");
  const uint32_t rows_pad = (uint32_t)(ceil_div64(rows, 128) * 128);
  const uint32_t tprb = (uint32_t)ceil_div64(sf_cols, 4);
  const int64_t n_words = (int64_t)rows_pad * tprb;
  swizzle_scales_kernel<<<grid_for(n_words, 256), 256, 0, (cudaStream_t)stream>>>(
      rowmajor, (uint32_t)rows, (uint32_t)sf_cols, rows_pad, tprb, reinterpret_cast<uint32_t*>(swizzled));
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}
