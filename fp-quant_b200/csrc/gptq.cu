// On-device GPTQ core for sm_100a: Hessian preparation, U = chol(H^-1, upper), the column-block
// quantise / error-propagation loop and the relative-MSE metric.  Replaces GPTQ._get_hessian_inverse,
// GPTQ.step and get_relative_mse_error of src/quantization/gptq.py (IST-DASLab/FP-Quant), which run
// as ~50 small torch kernels per weight column plus cuSOLVER calls.
//
// All arithmetic is fp32 (the reference disables TF32).  The reference chain
// cholesky -> cholesky_inverse -> cholesky(upper) is replaced by the mathematically equal
//   P = J H J (rows and columns reversed),  P = L L^T,  U = J L^-1 J
// because H = (J L J)(J L J)^T with J L J upper triangular, hence H^-1 = U^T U with U = (J L J)^-1.
// One factorisation and one triangular inverse instead of two factorisations and a full inverse.

#include <cstdlib>
#include <vector>
#include "common.cuh"

#include <atomic>
#include "sgemm.cuh"

namespace fpq {
// defined in hessian.cu: out = beta * out + alpha * A^T B on the tensor cores (bf16 operands, fp32 accumulation)
int gemm_atb_bf16(float* out, int64_t ldc, int64_t d1, int64_t d2, const void* A, int64_t lda, int64_t a_rows,
                  int64_t a_x0, const void* B, int64_t ldb, int64_t b_rows, int64_t b_x0, bool symmetric, bool mirror,
                  int n_seg, int64_t seg_rows, const int* a_seg_y, const int* b_seg_y, float alpha, float beta,
                  int32_t* error_flag, cudaStream_t stream, int tri = 0);
}  // namespace fpq

namespace fpq {
namespace {

constexpr int NB = 128;   // block size of the factorisation and of the GPTQ column blocks

// ------------------------------------------------------------------ Hessian preparation
__global__ void dead_columns_kernel(const float* __restrict__ W, int64_t rows, int64_t d, uint8_t* dead) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= d) return;
  bool all_zero = true;
  for (int64_t i = 0; i < rows && all_zero; ++i) all_zero = (W[i * d + j] == 0.0f);
  dead[j] = all_zero ? 1 : 0;
}

// Rows and columns of dead input channels become rows / columns of the identity.  A block covers 16 rows x
// 256 columns and leaves at once when none of its rows and columns is dead (the usual case: nothing is).
__global__ void __launch_bounds__(256) mask_dead_kernel(float* H, int64_t d, const uint8_t* __restrict__ dead) {
  __shared__ uint8_t drow[16];
  const int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t i0 = (int64_t)blockIdx.y * 16;
  if (threadIdx.x < 16) drow[threadIdx.x] = (i0 + threadIdx.x < d) ? dead[i0 + threadIdx.x] : 0;
  const int dj = (j < d && dead[j]) ? 1 : 0;
  const int any_col = __syncthreads_or(dj);       // also publishes drow
  int any_row = 0;
#pragma unroll
  for (int r = 0; r < 16; ++r) any_row |= drow[r];
  if (!any_col && !any_row) return;
  if (j >= d) return;
  for (int r = 0; r < 16; ++r) {
    const int64_t i = i0 + r;
    if (i < d && (drow[r] || dj)) H[i * d + j] = (i == j) ? 1.0f : 0.0f;
  }
}

__global__ void damp_kernel(float* H, int64_t d, float rel_damp) {
  // one block: mean of the diagonal, then diag += rel_damp * mean
  __shared__ double part[256];
  double s = 0.0;
  for (int64_t i = threadIdx.x; i < d; i += blockDim.x) s += (double)H[i * d + i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  const float damp = rel_damp * (float)(part[0] / (double)d);
  for (int64_t i = threadIdx.x; i < d; i += blockDim.x) H[i * d + i] += damp;
}

// ------------------------------------------------------------------ reversal / reflection
__global__ void reverse_copy_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t d) {
  const int64_t n = d * d;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x)
    dst[idx] = src[n - 1 - idx];   // (i, j) <- (d-1-i, d-1-j)
}

__global__ void reflect_inplace_kernel(float* A, int64_t d) {
  const int64_t n = d * d, half = n / 2;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < half; idx += (int64_t)gridDim.x * blockDim.x) {
    const float a = A[idx], b = A[n - 1 - idx];
    A[idx] = b;
    A[n - 1 - idx] = a;
  }
}

// ------------------------------------------------------------------ diagonal block: factor + invert
// One CTA factors the nb x nb (<= 128) diagonal block A (lower Cholesky, in place) and writes
// L^-1 (lower) to Linv.  A non-positive or non-finite pivot sets *status and is replaced by 1 so
// that the kernel always terminates with finite data.
//
// Both matrices live in registers: the 256 threads form a 16 x 16 grid, thread (ty, tx) owns the
// entries (ty + 16 r, tx + 16 c), r, c = 0..7, of A and of X (X starts as the identity).  Step k
// is one right-looking elimination step applied to both: column k of A and row k of X go through
// shared memory (double buffered, so one barrier per step), then
//     L[:, k] = A[:, k] / sqrt(A[k, k]),    X[k, :] /= L[k, k],
//     A[i, j] -= L[i, k] L[j, k]  (i, j > k),    X[i, :] -= L[i, k] X[k, :]  (i > k).
// The loop over the register index k / 16 is unrolled so that every register index is static;
// register blocks that are already final (or still zero) are skipped at compile time.
__global__ void __launch_bounds__(256) chol_diag_kernel(float* A, int64_t lda, float* Linv, int64_t ldi, int nb,
                                                        int32_t* status) {
  // Column k of A and row k of X as the threads need them: entry i sits at perm(i), so that the eight
  // values of a thread (i = t + 16 c) are two contiguous groups of four: perm(i) = (c / 4) * 64 + t * 4 + c % 4.
  __shared__ __align__(16) float colbuf[2][NB];
  __shared__ __align__(16) float rowbuf[2][NB];
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  float a[8][8], x[8][8];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = ty + 16 * r, j = tx + 16 * c;
      a[r][c] = (i < nb && j < nb) ? A[(int64_t)i * lda + j] : (i == j ? 1.0f : 0.0f);
      x[r][c] = i == j ? 1.0f : 0.0f;
    }
  }
#pragma unroll
  for (int cc = 0; cc < 8; ++cc) {
    for (int t = 0; t < 16; ++t) {
      const int k = 16 * cc + t;
      float* cb = colbuf[k & 1];
      float* rb = rowbuf[k & 1];
      if (tx == t) {
#pragma unroll
        for (int r = 0; r < 8; ++r) cb[(r >> 2) * 64 + ty * 4 + (r & 3)] = a[r][cc];
      }
      if (ty == t) {
#pragma unroll
        for (int c = 0; c < 8; ++c) rb[(c >> 2) * 64 + tx * 4 + (c & 3)] = x[cc][c];
      }
      __syncthreads();
      float piv = cb[(cc >> 2) * 64 + t * 4 + (cc & 3)];
      if (!(piv > 0.0f) || !isfinite(piv)) {
        if (tid == 0) atomicExch(status, 1);
        piv = 1.0f;
      }
      // The updates need only 1 / pivot: with c = A[:, k] and y = X[k, :] (both unscaled),
      //   A[i, j] -= c_i c_j / piv,   X[i, :] -= c_i y / piv;
      // the square root is taken off the critical path, by the owners of column k / row k alone.
      const float pinv = __frcp_rn(piv);
      float li[8], lj[8], xr[8];
      {
        const float4 v0 = *reinterpret_cast<const float4*>(&cb[ty * 4]), v1 = *reinterpret_cast<const float4*>(&cb[64 + ty * 4]);
        li[0] = v0.x; li[1] = v0.y; li[2] = v0.z; li[3] = v0.w; li[4] = v1.x; li[5] = v1.y; li[6] = v1.z; li[7] = v1.w;
        const float4 w0 = *reinterpret_cast<const float4*>(&cb[tx * 4]), w1 = *reinterpret_cast<const float4*>(&cb[64 + tx * 4]);
        lj[0] = w0.x; lj[1] = w0.y; lj[2] = w0.z; lj[3] = w0.w; lj[4] = w1.x; lj[5] = w1.y; lj[6] = w1.z; lj[7] = w1.w;
        const float4 y0 = *reinterpret_cast<const float4*>(&rb[tx * 4]), y1 = *reinterpret_cast<const float4*>(&rb[64 + tx * 4]);
        xr[0] = y0.x; xr[1] = y0.y; xr[2] = y0.z; xr[3] = y0.w; xr[4] = y1.x; xr[5] = y1.y; xr[6] = y1.z; xr[7] = y1.w;
      }
      float ljs[8], xrs[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        ljs[c] = lj[c] * pinv;
        xrs[c] = xr[c] * pinv;
      }
      const bool below = ty > t;   // row ty + 16 cc lies below row k
#pragma unroll
      for (int r = cc; r < 8; ++r) {
        if (r > cc || below) {
#pragma unroll
          for (int c = cc; c < 8; ++c)
            if (c > cc || tx > t) a[r][c] = fmaf(-li[r], ljs[c], a[r][c]);
#pragma unroll
          for (int c = 0; c <= cc; ++c) x[r][c] = fmaf(-li[r], xrs[c], x[r][c]);
        }
      }
      if (tx == t || ty == t) {
        float rinv = rsqrtf(piv);
        rinv = rinv * fmaf(-0.5f * piv * rinv, rinv, 1.5f);   // one Newton step: full fp32 accuracy
        if (tx == t) {
#pragma unroll
          for (int r = cc; r < 8; ++r) a[r][cc] = li[r] * rinv;
        }
        if (ty == t) {
#pragma unroll
          for (int c = 0; c <= cc; ++c) x[cc][c] = xr[c] * rinv;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = ty + 16 * r, j = tx + 16 * c;
      if (i < nb && j < nb) {
        A[(int64_t)i * lda + j] = j <= i ? a[r][c] : 0.0f;
        Linv[(int64_t)i * ldi + j] = j <= i ? x[r][c] : 0.0f;
      }
    }
  }
}

int grid1d(int64_t n) {
  int64_t b = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}

// ------------------------------------------------------------------ fp32-accurate products on the tensor cores
// x in fp32 -> three bf16 terms hi + mid + lo that together carry all 24 mantissa bits.
__device__ __forceinline__ void split3(float v, __nv_bfloat16& h, __nv_bfloat16& m, __nv_bfloat16& l) {
  h = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(h);
  m = __float2bfloat16_rn(r1);
  l = __float2bfloat16_rn(r1 - __bfloat162float(m));
}

// in [K, N] fp32 (row stride ld_in) -> out: three planes [K, ld_out] bf16 (hi, mid, lo), plane p at row p * K
__global__ void split3_rows_kernel(const float* __restrict__ in, int64_t ld_in, int64_t K, int64_t N,
                                   __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  const int64_t total = K * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t k = i / N, n = i - k * N;
    __nv_bfloat16 h, m, l;
    split3(in[k * ld_in + n], h, m, l);
    out[k * ld_out + n] = h;
    out[(K + k) * ld_out + n] = m;
    out[(2 * K + k) * ld_out + n] = l;
  }
}

// in [R, K] fp32 (row stride ld_in) -> out: three planes [K, ld_out] bf16 holding the transposed terms:
// plane p, row k, column r = term p of in[r, k].  Tiles of 32 x 32 through shared memory.
__global__ void __launch_bounds__(256) transpose_split3_kernel(const float* __restrict__ in, int64_t ld_in, int64_t R,
                                                               int64_t K, __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  __shared__ float tile[32][33];
  const int64_t r0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int rr = ty; rr < 32; rr += 8)
    tile[rr][tx] = (r0 + rr < R && k0 + tx < K) ? in[(r0 + rr) * ld_in + k0 + tx] : 0.0f;
  __syncthreads();
  for (int kk = ty; kk < 32; kk += 8) {
    if (k0 + kk < K && r0 + tx < ld_out) {
      __nv_bfloat16 h, m, l;
      split3(tile[tx][kk], h, m, l);
      out[(k0 + kk) * ld_out + r0 + tx] = h;
      out[(K + k0 + kk) * ld_out + r0 + tx] = m;
      out[(2 * K + k0 + kk) * ld_out + r0 + tx] = l;
    }
  }
}

int64_t round64(int64_t x) { return (x + 63) & ~(int64_t)63; }

// bf16 elements of workspace tc_gemm3 needs
int64_t tc_gemm3_workspace(int64_t M, int64_t N, int64_t K, bool b_is_a_transposed) {
  return 3 * K * round64(M) + (b_is_a_transposed ? 0 : 3 * K * round64(N));
}

// C[M, N] (row stride ldc) = beta * C + alpha * A B with fp32-level accuracy on the tensor cores:
// A [M, K] row-major (lda); B [K, N] row-major (ldb), or B == nullptr for B = (the first N rows of A)^T:
// with N == M the symmetric rank-K update (only the tiles touching the lower triangle are computed), with
// N < M its first N columns.  Both factors are split
// into three bf16 terms and the six leading cross products (hi*hi, hi*mid, mid*hi, hi*lo, lo*hi, mid*mid;
// the dropped ones are below 2^-24 relative) are accumulated in fp32 in one launch whose K dimension is
// the concatenation of the six slabs.  K must be a multiple of 64.
int tc_gemm3(float* C, int64_t ldc, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
             int64_t ldb, float alpha, float beta, __nv_bfloat16* ws, int32_t* error_flag, cudaStream_t st, int tri = 0) {
  static const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
  const int64_t ldat = round64(M);
  __nv_bfloat16* at3 = ws;
  dim3 tgrid((unsigned)((ldat + 31) / 32), (unsigned)((K + 31) / 32));
  transpose_split3_kernel<<<tgrid, 256, 0, st>>>(A, lda, M, K, at3, ldat);
  FPQ_CHECK_LAUNCH();
  const __nv_bfloat16* b3 = at3;
  int64_t ldbt = ldat;
  if (B) {
    ldbt = round64(N);
    __nv_bfloat16* bw = ws + 3 * K * ldat;
    split3_rows_kernel<<<grid1d(K * N), 256, 0, st>>>(B, ldb, K, N, bw, ldbt);
    FPQ_CHECK_LAUNCH();
    b3 = bw;
  }
  int a_y[6], b_y[6];
  for (int t = 0; t < 6; ++t) {
    a_y[t] = (int)(pa[t] * K);
    b_y[t] = (int)(pb[t] * K);
  }
  return gemm_atb_bf16(C, ldc, M, N, at3, ldat, 3 * K, 0, b3, ldbt, 3 * K, 0, B == nullptr && N == M, false, 6, K, a_y,
                       b_y, alpha, beta, error_flag, st, tri);
}

// Products at least this large go to the tensor cores; smaller ones stay on the fp32 SIMT kernel, whose
// launch is cheaper than the two conversion passes.
bool tc_worthwhile(int64_t M, int64_t N, int64_t K) {
  return K % 64 == 0 && M * N * K >= ((int64_t)1 << 25);
}

// X = L^-1 given the inverses of the diagonal blocks already in X.  The block range [lo, hi) is halved
// recursively: L^-1 = [[X11, 0], [-X22 (L21 X11), X22]], S = L21 X11 (n2 x n1) goes to `scratch`.  The
// nodes of one depth are independent, so the tree is walked level by level from the leaves: the small
// nodes of a level share two launches of the batched fp32 kernel (S for all of them, then X21 for all of
// them), the large ones go to the tensor cores one after the other.
struct TriNode { int lo, mid, hi; };

void tri_collect(std::vector<std::vector<TriNode>>& levels, int lo, int hi, int depth) {
  if (hi - lo <= 1) return;
  const int mid = (lo + hi) / 2;
  if ((int)levels.size() <= depth) levels.resize(depth + 1);
  levels[depth].push_back({lo, mid, hi});
  tri_collect(levels, lo, mid, depth + 1);
  tri_collect(levels, mid, hi, depth + 1);
}

int tri_inverse_levels(const float* L, float* X, float* scratch, __nv_bfloat16* ws, int32_t* error_flag, int64_t d,
                       int nblk, cudaStream_t st) {
  std::vector<std::vector<TriNode>> levels;
  tri_collect(levels, 0, nblk, 0);
  for (int depth = (int)levels.size() - 1; depth >= 0; --depth) {
    std::vector<TriNode> big;
    SgemmBatch s1{}, s2{};
    int64_t used = 0;
    auto flush = [&]() -> int {
      if (s1.count == 0) return FPQ_OK;
      if (int rc = sgemm_batched(s1, false, st)) return rc;
      if (int rc = sgemm_batched(s2, false, st)) return rc;
      s1.count = s2.count = 0;
      used = 0;
      return FPQ_OK;
    };
    for (const TriNode& nd : levels[depth]) {
      const int64_t r0 = (int64_t)nd.lo * NB, r1 = (int64_t)nd.mid * NB;
      const int64_t n1 = r1 - r0;
      int64_t n2 = (int64_t)nd.hi * NB - r1;
      if (r1 + n2 > d) n2 = d - r1;
      if (tc_worthwhile(n2, n1, n1) && n2 % 64 == 0) {
        big.push_back(nd);
        continue;
      }
      if (s1.count == SGEMM_MAX_BATCH)
        if (int rc = flush()) return rc;
      float* S = scratch + used;
      used += n1 * n2;
      SgemmArgs& a = s1.e[s1.count++];          // S = L21 * X11
      a = SgemmArgs{};
      a.A = L + r1 * d + r0; a.lda = d;
      a.B = X + r0 * d + r0; a.ldb = d;
      a.C = S; a.ldc = n1;
      a.M = (int)n2; a.N = (int)n1; a.K = (int)n1; a.alpha = 1.0f; a.beta = 0.0f;
      SgemmArgs& b = s2.e[s2.count++];          // X21 = -X22 * S
      b = SgemmArgs{};
      b.A = X + r1 * d + r1; b.lda = d;
      b.B = S; b.ldb = n1;
      b.C = X + r1 * d + r0; b.ldc = d;
      b.M = (int)n2; b.N = (int)n1; b.K = (int)n2; b.alpha = -1.0f; b.beta = 0.0f;
    }
    if (int rc = flush()) return rc;
    for (const TriNode& nd : big) {
      const int64_t r0 = (int64_t)nd.lo * NB, r1 = (int64_t)nd.mid * NB;
      const int64_t n1 = r1 - r0;
      int64_t n2 = (int64_t)nd.hi * NB - r1;
      if (r1 + n2 > d) n2 = d - r1;
      // S = L21 * X11 (X11 lower triangular), then X21 = -X22 * S (X22 lower triangular): the stages that
      // would only multiply the zero halves are skipped
      if (int rc = tc_gemm3(scratch, n1, n2, n1, n1, L + r1 * d + r0, d, X + r0 * d + r0, d, 1.0f, 0.0f, ws, error_flag, st, 1))
        return rc;
      if (int rc = tc_gemm3(X + r1 * d + r0, d, n2, n1, n2, X + r1 * d + r1, d, scratch, n1, -1.0f, 0.0f, ws, error_flag, st, 2))
        return rc;
    }
  }
  return FPQ_OK;
}

// ------------------------------------------------------------------ GPTQ column block
// Four threads per weight row, each holding 32 of the block's 128 columns in registers.  Columns are
// walked left to right: the owner of column i quantises it with the row's static group scale and
// turns the residual into err = (w - wq) / U[i,i]; the error is broadcast inside the quad and every
// thread subtracts err * U[i, j] from its columns j > i (src/quantization/gptq.py:166-186), in the
// same order as the reference applies them.  U's diagonal block sits in shared memory; a quad reads
// four 16-byte pieces of one row per load.  The outer loop over the four 32-column owners is a real
// loop (the unrolled body of 32 steps stays inside the instruction cache: a fully unrolled
// thread-per-row version was instruction-fetch bound at three warps per SM).  Afterwards each thread
// writes its 32 errors (as the transposed three-term bf16 operand of the trailing update), the dequantised values, rebuilt
// as grid(code) * scale exactly as they were computed, and its 16 code bytes.
constexpr int SUB = 32;   // columns per thread
// Shared-memory image of U's diagonal block: every 32-column piece of a row is shifted by another
// 16 bytes, so that the four pieces a quad reads with one 128-bit load start in different banks.
constexpr int US_LD = NB + 4 * (NB / SUB);
__device__ __forceinline__ int us_col(int col) { return col + 4 * (col / SUB); }

// Correctly rounded y / s from r = rcp(s): multiply and two fused residual corrections (valid while s, r and
// the quotient stay in the normal range; the caller checks s).
__device__ __forceinline__ float div_by(float y, float s, float r) {
  float q = y * r;
  float e = fmaf(-s, q, y);
  q = fmaf(e, r, q);
  e = fmaf(-s, q, y);
  return fmaf(e, r, q);
}
__device__ __forceinline__ bool rcp_safe(float s) {
  const float a = fabsf(s);
  return a > 7.8886e-31f /* 2^-100 */ && a < 1.2676e30f /* 2^100 */;
}
// E2M1 code of v (round to nearest, ties to even, saturating; every zero as 0x8) and its grid value.
__device__ __forceinline__ uint32_t e2m1_code_hw(float v, float& value) {
  uint32_t byte;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(byte) : "f"(0.0f), "f"(v));
  uint32_t code = byte & 0xFu;
  if ((code & 7u) == 0u) code = 8u;
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(code));
  value = __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
  return code;
}

// G = 16 / 32: column c uses scale group c / G.  G = 1: activation order -- the columns were permuted
// beforehand and column c uses group gidx[c] of the n_groups static groups (gptq.py:146-148, 170-171);
// every thread then keeps one scale per column, so blocks are limited to 256 threads.
template <int G>
__global__ void __launch_bounds__(G == 1 ? 256 : 512) gptq_block_kernel(float* __restrict__ W, int64_t rows, int64_t C,
                                                                        int64_t c1, const float* __restrict__ scales,
                                                                        const float* __restrict__ U,
                                                                        __nv_bfloat16* __restrict__ ErrT3, int64_t lda,
                                                                        uint8_t* __restrict__ codes,
                                                                        const int32_t* __restrict__ gidx, int n_groups) {
  extern __shared__ float Us[];   // NB rows of US_LD floats, then the reciprocals of the diagonal
  float* rdiag = Us + NB * US_LD;
  for (int idx = threadIdx.x; idx < NB * NB / 4; idx += blockDim.x) {
    const int i = (idx * 4) / NB, j = (idx * 4) % NB;
    *reinterpret_cast<float4*>(&Us[i * US_LD + us_col(j)]) = *reinterpret_cast<const float4*>(&U[(c1 + i) * C + c1 + j]);
  }
  for (int i = threadIdx.x; i < NB; i += blockDim.x) {
    const float dgl = U[(c1 + i) * C + c1 + i];
    rdiag[i] = rcp_safe(dgl) ? __frcp_rn(dgl) : 0.0f;      // 0 marks "divide the slow way"
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int q = lane & 3;                      // which 32 columns of the block are mine
  int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 2;
  const bool live = row < rows;
  if (!live) row = rows - 1;                   // keep the quad's shuffles uniform; nothing is stored

  constexpr int NGRP = SUB / G;
  float sc[NGRP], rsc[G == 1 ? 1 : NGRP];
#pragma unroll
  for (int g = 0; g < NGRP; ++g) {
    if (G == 1) {
      sc[g] = scales[row * n_groups + gidx[c1 + SUB * q + g]];
    } else {
      sc[g] = scales[row * (C / G) + (c1 + SUB * q) / G + g];
      rsc[g] = rcp_safe(sc[g]) ? __frcp_rn(sc[g]) : 0.0f;
    }
  }
  float w[SUB], err[SUB];
  {
    const float4* wp = reinterpret_cast<const float4*>(W + row * C + c1 + SUB * q);
#pragma unroll
    for (int v = 0; v < SUB / 4; ++v) {
      const float4 t = wp[v];
      w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
    }
  }
  uint32_t cw[SUB / 8];
#pragma unroll
  for (int v = 0; v < SUB / 8; ++v) cw[v] = 0;
#pragma unroll
  for (int j = 0; j < SUB; ++j) err[j] = 0.0f;

#pragma unroll 1
  for (int b = 0; b < NB / SUB; ++b) {
    const bool owner = q == b;
    const float* Ub = Us + (SUB * b) * US_LD;  // rows of U for the owner's columns
#pragma unroll
    for (int ii = 0; ii < SUB; ++ii) {
      float e = 0.0f;
      if (owner) {
        // w / s and (w - wq) / U[i,i] as IEEE divisions (the reference's), computed from reciprocals
        const float s = sc[ii / G];
        const float rs = G == 1 ? (rcp_safe(s) ? __frcp_rn(s) : 0.0f) : rsc[G == 1 ? 0 : ii / G];
        const float qv = rs != 0.0f ? div_by(w[ii], s, rs) : __fdiv_rn(w[ii], s);
        float gv;
        const uint32_t code = e2m1_code_hw(qv, gv);
        cw[ii / 8] |= code << (4 * (ii % 8));
        const float wq = __fmul_rn(gv, s);
        const float dgl = Ub[ii * US_LD + (SUB + 4) * b + ii], rd = rdiag[SUB * b + ii];
        const float diff = __fsub_rn(w[ii], wq);
        e = rd != 0.0f ? div_by(diff, dgl, rd) : __fdiv_rn(diff, dgl);
        err[ii] = e;
      }
      e = __shfl_sync(0xffffffffu, e, (lane & ~3) | b);
      const float e_ge = q >= b ? -e : 0.0f;   // applies to my columns right of ii when I am the owner or later
      const float e_gt = q > b ? -e : 0.0f;    // applies to all my columns only when I come after the owner
      const float4* up = reinterpret_cast<const float4*>(Ub + ii * US_LD + (SUB + 4) * q);
#pragma unroll
      for (int v = 0; v < SUB / 4; ++v) {
        const float4 u = up[v];
        w[4 * v] = fmaf(4 * v > ii ? e_ge : e_gt, u.x, w[4 * v]);
        w[4 * v + 1] = fmaf(4 * v + 1 > ii ? e_ge : e_gt, u.y, w[4 * v + 1]);
        w[4 * v + 2] = fmaf(4 * v + 2 > ii ? e_ge : e_gt, u.z, w[4 * v + 2]);
        w[4 * v + 3] = fmaf(4 * v + 3 > ii ? e_ge : e_gt, u.w, w[4 * v + 3]);
      }
    }
  }
  // The block's errors leave as the operand of the trailing update: three bf16 terms per value, transposed
  // ([3 * 128, lda], plane p of column c at row p * 128 + c).  They are staged in shared memory (the image
  // of U is no longer needed) so that the global stores run along the rows.
  const int rb = (int)(blockDim.x >> 2);            // rows of this block
  const int es_ld = rb + 1;
  const int r_local = (int)(threadIdx.x >> 2);
  __syncthreads();                                  // every warp has finished reading Us
  float* Es = Us;
#pragma unroll
  for (int j = 0; j < SUB; ++j) Es[(SUB * q + j) * es_ld + r_local] = err[j];
  __syncthreads();
  {
    const int64_t row0 = (int64_t)blockIdx.x * rb;
    const int pairs = rb >> 1;
    for (int idx = (int)threadIdx.x; idx < NB * pairs; idx += (int)blockDim.x) {
      const int c = idx / pairs, r0 = 2 * (idx - c * pairs);
      const int64_t g = row0 + r0;
      if (g >= lda) continue;                       // lda is even and >= rows: g + 1 < lda as well
      const float v0 = g < rows ? Es[c * es_ld + r0] : 0.0f;
      const float v1 = g + 1 < rows ? Es[c * es_ld + r0 + 1] : 0.0f;
      __nv_bfloat16 h0, m0, l0, h1, m1, l1;
      split3(v0, h0, m0, l0);
      split3(v1, h1, m1, l1);
      __nv_bfloat16* dst = ErrT3 + (int64_t)c * lda + g;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __halves2bfloat162(h0, h1);
      *reinterpret_cast<__nv_bfloat162*>(dst + (int64_t)NB * lda) = __halves2bfloat162(m0, m1);
      *reinterpret_cast<__nv_bfloat162*>(dst + (int64_t)2 * NB * lda) = __halves2bfloat162(l0, l1);
    }
  }
  if (!live) return;

  float4* op = reinterpret_cast<float4*>(W + row * C + c1 + SUB * q);
#pragma unroll
  for (int v = 0; v < SUB / 4; ++v) {
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = 4 * v + j;
      o[j] = __fmul_rn(e2m1_value((cw[i / 8] >> (4 * (i % 8))) & 15u), sc[i / G]);
    }
    op[v] = make_float4(o[0], o[1], o[2], o[3]);
  }
  if (codes)
    *reinterpret_cast<uint4*>(codes + row * (C / 2) + (c1 + SUB * q) / 2) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
}

__global__ void diff_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = a[i] - b[i];
}

// x (or x - y) in fp32 -> two bf16 terms hi + lo (relative residual ~2^-17)
__global__ void split_bf16_kernel(const float* __restrict__ x, const float* __restrict__ y, __nv_bfloat16* __restrict__ hi,
                                  __nv_bfloat16* __restrict__ lo, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = y ? x[i] - y[i] : x[i];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// Deterministic reductions of the relative-MSE metric: every CTA writes the sum of its part to a slot of
// its own (nothing is added atomically), and one warp adds the slots in a fixed order at the end.
constexpr int MSE_DOT_BLOCKS = 1024;      // CTAs (and slots) of one frobenius_dot_kernel launch
constexpr int MSE_REGION = FPQ_RELATIVE_MSE_ACC_DOUBLES / 2;   // slots per quantity (numerator / denominator)

// partial[blockIdx.x] = weight * sum over this CTA's elements of a .* b
__global__ void __launch_bounds__(256) frobenius_dot_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                            int64_t n, double weight, double* partial) {
  __shared__ double warp_sum[8];
  double s = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    s += (double)a[i] * (double)b[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += warp_sum[w];
    partial[blockIdx.x] = weight * t;
  }
}

// out = mean(num) / (mean(den) + 1e-6), src/quantization/gptq.py:28-30; num / den = the sums of the first
// n_slots slots of the two regions, each lane adding its slots in index order, then a fixed shuffle tree.
__global__ void ratio_kernel(const double* acc, int n_slots, float* out, double count) {
  double v[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    double s = 0.0;
    for (int i = threadIdx.x; i < n_slots; i += 32) s += acc[(size_t)q * MSE_REGION + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    v[q] = s;
  }
  if (threadIdx.x == 0) out[0] = (float)((v[0] / count) / (v[1] / count + 1e-6));
}

}  // namespace
}  // namespace fpq

using namespace fpq;

extern "C" int fpq_hessian_prepare(float* H, int64_t d, const float* W, int64_t rows, float rel_damp,
                                   uint8_t* workspace, fpq_stream_t stream) {
  FPQ_CHECK_ARG(H && W && workspace, "NULL pointer");
  FPQ_CHECK_ARG(d > 0 && d <= (1 << 20) && rows > 0, "bad shape");
  cudaStream_t st = (cudaStream_t)stream;
  dead_columns_kernel<<<(unsigned)((d + 255) / 256), 256, 0, st>>>(W, rows, d, workspace);
  FPQ_CHECK_LAUNCH();
  mask_dead_kernel<<<dim3((unsigned)((d + 255) / 256), (unsigned)((d + 15) / 16)), 256, 0, st>>>(H, d, workspace);
  FPQ_CHECK_LAUNCH();
  damp_kernel<<<1, 256, 0, st>>>(H, d, rel_damp);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

// Scratch of fpq_hessian_prepare_noalloc: one "column is dead" flag per input channel.  It lives in
// the library image, so every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) uint8_t g_prepare_scratch[FPQ_PREPARE_NOALLOC_MAX_D];

extern "C" int fpq_hessian_prepare_noalloc(float* H, int64_t d, const float* W, int64_t rows, float rel_damp,
                                           fpq_stream_t stream) {
  FPQ_CHECK_ARG(H && W, "NULL pointer");
  FPQ_CHECK_ARG(d > 0 && rows > 0, "bad shape");
  FPQ_CHECK_ARG(d <= FPQ_PREPARE_NOALLOC_MAX_D,
                "d = %lld exceeds the built-in scratch of fpq_hessian_prepare_noalloc (%d input channels); "
                "use fpq_hessian_prepare with a caller-provided workspace",
                (long long)d, FPQ_PREPARE_NOALLOC_MAX_D);
  // The array's name is only a host-side handle; kernels need its device address, which differs per
  // GPU.  Resolve it once per device, with that device current.
  static std::atomic<uint8_t*> scratch_of_device[64];      // two threads making the first call store the same address
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  FPQ_CHECK_ARG(dev >= 0 && dev < 64, "device index %d out of range", dev);
  // The scratch is the current device's copy of the array, so H, W and the stream must belong to the
  // current device: a Hessian on another GPU would be masked with flags this GPU never wrote.
  cudaPointerAttributes attr{};
  FPQ_CHECK_CUDA(cudaPointerGetAttributes(&attr, H));
  FPQ_CHECK_ARG(attr.type != cudaMemoryTypeDevice || attr.device == dev,
                "H lives on device %d but the current device is %d: make the device that owns H current", attr.device, dev);
  uint8_t* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    FPQ_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_prepare_scratch));
    FPQ_CHECK_ARG(scratch != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  cudaStream_t st = (cudaStream_t)stream;
  // Every flag in [0, d) is rewritten before it is read, so nothing needs clearing between calls.
  dead_columns_kernel<<<(unsigned)((d + 255) / 256), 256, 0, st>>>(W, rows, d, scratch);
  FPQ_CHECK_LAUNCH();
  mask_dead_kernel<<<dim3((unsigned)((d + 255) / 256), (unsigned)((d + 15) / 16)), 256, 0, st>>>(H, d, scratch);
  FPQ_CHECK_LAUNCH();
  damp_kernel<<<1, 256, 0, st>>>(H, d, rel_damp);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int64_t fpq_cholesky_workspace_floats(int64_t d) {
  // L (d x d) | scratch of the triangular inverse (half x half) | bf16 operand splits (6 half^2 bf16 = 3 half^2 floats)
  const int64_t nblk = (d + NB - 1) / NB;
  const int64_t half = ((nblk + 1) / 2) * NB;
  return d * d + 4 * half * half + 64;
}

extern "C" int fpq_cholesky_inverse_upper(const float* H, float* U, int64_t d, float* workspace, int32_t* status,
                                          int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(H && U && workspace && status && error_flag, "NULL pointer");
  FPQ_CHECK_ARG(d > 0 && d < (1ll << 30), "bad size");
  FPQ_CHECK_ARG(H != U, "U must not alias H");
  FPQ_CHECK_ARG(((uintptr_t)workspace & 15) == 0, "workspace must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int nblk = (int)((d + NB - 1) / NB);
  const int64_t half = (int64_t)((nblk + 1) / 2) * NB;
  float* L = workspace;
  float* scratch = workspace + ((d * d + 3) & ~(int64_t)3);
  __nv_bfloat16* ws = reinterpret_cast<__nv_bfloat16*>(scratch + half * half);
  FPQ_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  reverse_copy_kernel<<<grid1d(d * d), 256, 0, st>>>(H, L, d);
  FPQ_CHECK_LAUNCH();
  FPQ_CHECK_CUDA(cudaMemsetAsync(U, 0, (size_t)d * d * sizeof(float), st));
  // Right-looking blocked Cholesky in two levels.  Inside an outer block of OB diagonal blocks the rank-128
  // updates only touch the outer block's own columns (all rows below); the rest of the trailing matrix gets
  // one rank-(OB*128) update per outer block, which reads and writes it 1/OB as often as a rank-128
  // update per diagonal block would (those updates are bound by that traffic, not by the tensor pipe).
  constexpr int OB = 4;
  const int64_t ws_elems = 6 * half * half;
  for (int ob = 0; ob < nblk; ob += OB) {
    const int64_t R = (int64_t)ob * NB;
    const int64_t Wd = (d - R) < (int64_t)OB * NB ? (d - R) : (int64_t)OB * NB;
    for (int k = ob; k < nblk && k < ob + OB; ++k) {
      const int64_t r = (int64_t)k * NB;
      const int nb = (int)((d - r) < NB ? (d - r) : NB);
      chol_diag_kernel<<<1, 256, 0, st>>>(L + r * d + r, d, U + r * d + r, d, nb, status);
      FPQ_CHECK_LAUNCH();
      const int64_t below = d - (r + nb);
      if (below <= 0) break;
      SgemmArgs a{};
      // panel: L21 = A21 * L11^-T  (in place: every CTA reads only the 128 rows it then overwrites)
      a.A = L + (r + nb) * d + r; a.lda = d;
      a.B = U + r * d + r; a.ldb = d;
      a.C = L + (r + nb) * d + r; a.ldc = d;
      a.M = (int)below; a.N = nb; a.K = nb; a.alpha = 1.0f; a.beta = 0.0f;
      if (int rc = sgemm(a, true, SGEMM_PLAIN, st)) return rc;
      // inner update: columns [r + nb, R + Wd) of the rows below -= L21 * (the first rows of L21)^T
      const int64_t inner = R + Wd - (r + nb);
      if (inner <= 0) continue;
      float* Cin = L + (r + nb) * d + (r + nb);
      if (nb == NB && tc_worthwhile(below, inner, nb) &&
          3 * (int64_t)nb * round64(below) <= ws_elems) {
        if (int rc = tc_gemm3(Cin, d, below, inner, nb, L + (r + nb) * d + r, d, nullptr, 0, -1.0f, 1.0f, ws, error_flag, st))
          return rc;
        continue;
      }
      a.A = L + (r + nb) * d + r; a.lda = d;
      a.B = L + (r + nb) * d + r; a.ldb = d;
      a.C = Cin; a.ldc = d;
      a.M = (int)below; a.N = (int)inner; a.K = nb; a.alpha = -1.0f; a.beta = 1.0f;
      if (int rc = sgemm(a, true, inner == below ? SGEMM_LOWER : SGEMM_PLAIN, st)) return rc;
    }
    // outer update: A22 -= P P^T (lower tiles only), P = the outer block's columns of the rows below it
    const int64_t below_o = d - (R + Wd);
    if (below_o <= 0) break;
    float* C22 = L + (R + Wd) * d + (R + Wd);
    const float* P = L + (R + Wd) * d + R;
    if (Wd % 64 == 0 && tc_worthwhile(below_o, below_o, Wd) && 3 * Wd * round64(below_o) <= ws_elems) {
      if (int rc = tc_gemm3(C22, d, below_o, below_o, Wd, P, d, nullptr, 0, -1.0f, 1.0f, ws, error_flag, st)) return rc;
      continue;
    }
    SgemmArgs a{};
    a.A = P; a.lda = d;
    a.B = P; a.ldb = d;
    a.C = C22; a.ldc = d;
    a.M = (int)below_o; a.N = (int)below_o; a.K = (int)Wd; a.alpha = -1.0f; a.beta = 1.0f;
    if (int rc = sgemm(a, true, SGEMM_LOWER, st)) return rc;
  }
  if (int rc = tri_inverse_levels(L, U, scratch, ws, error_flag, d, nblk, st)) return rc;
  reflect_inplace_kernel<<<grid1d(d * d / 2), 256, 0, st>>>(U, d);   // U <- J X J (upper triangular)
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

namespace {
int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }
int64_t gptq_lda(int64_t rows) { return (rows + 63) & ~(int64_t)63; }
}  // namespace

extern "C" int64_t fpq_gptq_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return align256(rows * NB * (int64_t)sizeof(float)) + align256(3 * NB * gptq_lda(rows) * 2) + align256(3 * cols * cols * 2);
}

extern "C" int fpq_gptq_quantize(float* W, int64_t rows, int64_t cols, const float* scales, int group,
                                 const float* U, uint8_t* codes, void* workspace, int32_t* error_flag,
                                 fpq_stream_t stream) {
  return fpq_gptq_quantize_ordered(W, rows, cols, scales, group, nullptr, U, codes, workspace, error_flag, stream);
}

extern "C" int fpq_gptq_quantize_ordered(float* W, int64_t rows, int64_t cols, const float* scales, int group,
                                         const int32_t* group_index, const float* U, uint8_t* codes, void* workspace,
                                         int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(W && scales && U && workspace && error_flag, "NULL pointer");
  FPQ_CHECK_ARG(group == 16 || group == 32, "group must be 16 (NVFP4) or 32 (MXFP4)");
  FPQ_CHECK_ARG(rows > 0 && cols > 0 && cols % NB == 0, "cols (%lld) must be a multiple of %d", (long long)cols, NB);
  FPQ_CHECK_ARG(rows < (1ll << 30) && 3 * cols < (1ll << 31), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)W & 15) == 0 && ((uintptr_t)U & 15) == 0 && ((uintptr_t)workspace & 255) == 0 &&
                    ((uintptr_t)codes & 15) == 0, "W, U, codes must be 16-byte aligned, the workspace 256-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured[64] = {};
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  const int smem = (NB * US_LD + NB) * (int)sizeof(float);
  if (dev < 64 && !configured[dev]) {
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(gptq_block_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(gptq_block_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(gptq_block_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  // workspace: (unused fp32 slab, kept so that the size helper does not change) | transposed three-term bf16 split of a block's errors | three-term bf16 split of U
  const int64_t lda = gptq_lda(rows);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  __nv_bfloat16* errT3 = reinterpret_cast<__nv_bfloat16*>(ws + align256(rows * NB * (int64_t)sizeof(float)));
  __nv_bfloat16* U3 = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(errT3) + align256(3 * NB * lda * 2));
  if (cols > NB) {
    split3_rows_kernel<<<grid1d(cols * cols), 256, 0, st>>>(U, cols, cols, cols, U3, cols);
    FPQ_CHECK_LAUNCH();
  }
  // The trailing update W[:, c2:] -= Err U[c1:c2, c2:] runs on the tensor cores: both factors are split
  // into three bf16 terms and the six leading cross products (hi*hi, hi*mid, mid*hi, hi*lo, lo*hi,
  // mid*mid; the dropped ones are below 2^-24 relative) are accumulated in fp32 as one GEMM whose K
  // dimension is the concatenation of the six 128-row slabs.
  static const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
  // Four threads per row, eight rows per warp.  The kernel is bound by the latency of its 128 dependent
  // steps, so all rows should be resident at once: warps per block are chosen so that one block per SM
  // covers everything when that is possible (14336 rows: 13 warps on 138 SMs) instead of leaving a
  // handful of blocks for a second pass.
  const int64_t units = (rows + 7) / 8;
  int wpb = (int)((units + sm_count() - 1) / sm_count());
  const int wpb_max = group_index ? 8 : 16;
  wpb = wpb < 4 ? 4 : (wpb > wpb_max ? wpb_max : wpb);
  const unsigned threads = (unsigned)wpb * 32;
  const unsigned grid = (unsigned)((units + wpb - 1) / wpb);
  for (int64_t c1 = 0; c1 < cols; c1 += NB) {
    const int n_groups = (int)(cols / group);
    if (group_index)
      gptq_block_kernel<1><<<grid, threads, smem, st>>>(W, rows, cols, c1, scales, U, errT3, lda, codes, group_index, n_groups);
    else if (group == 16)
      gptq_block_kernel<16><<<grid, threads, smem, st>>>(W, rows, cols, c1, scales, U, errT3, lda, codes, nullptr, n_groups);
    else
      gptq_block_kernel<32><<<grid, threads, smem, st>>>(W, rows, cols, c1, scales, U, errT3, lda, codes, nullptr, n_groups);
    FPQ_CHECK_LAUNCH();
    const int64_t c2 = c1 + NB;
    if (c2 >= cols) break;
    int a_y[6], b_y[6];
    for (int t = 0; t < 6; ++t) {
      a_y[t] = pa[t] * NB;
      b_y[t] = (int)(pb[t] * cols + c1);
    }
    if (int rc = gemm_atb_bf16(W + c2, cols, rows, cols - c2, errT3, lda, 3 * NB, 0, U3, cols, 3 * cols, c2, false, false, 6,
                               NB, a_y, b_y, -1.0f, 1.0f, error_flag, st))
      return rc;
  }
  return FPQ_OK;
}

extern "C" int fpq_relative_mse(const float* Wq, const float* W, const float* H, int64_t rows, int64_t d,
                                float* diff_workspace, double* acc_workspace, float* out, fpq_stream_t stream) {
  FPQ_CHECK_ARG(Wq && W && H && diff_workspace && acc_workspace && out, "NULL pointer");
  const int64_t tiles = ((rows + 127) / 128) * ((d + 127) / 128);      // CTAs of one fp32 product = partial sums
  FPQ_CHECK_ARG(tiles <= MSE_REGION, "matrix too large for the %d partial-sum slots of the workspace", MSE_REGION);
  cudaStream_t st = (cudaStream_t)stream;
  diff_kernel<<<grid1d(rows * d), 256, 0, st>>>(Wq, W, diff_workspace, rows * d);
  FPQ_CHECK_LAUNCH();
  SgemmArgs a{};
  a.lda = d; a.B = H; a.ldb = d; a.M = (int)rows; a.N = (int)d; a.K = (int)d; a.alpha = 1.0f; a.ldd = d;
  a.A = diff_workspace; a.D = diff_workspace; a.dot_out = acc_workspace;
  if (int rc = sgemm(a, false, SGEMM_DOT, st)) return rc;
  a.A = W; a.D = W; a.dot_out = acc_workspace + MSE_REGION;
  if (int rc = sgemm(a, false, SGEMM_DOT, st)) return rc;
  ratio_kernel<<<1, 32, 0, st>>>(acc_workspace, (int)tiles, out, (double)rows * (double)d);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

extern "C" int fpq_hessian_accumulate(float* H, int64_t d, const void* xa_bf16, const void* xb_bf16, int64_t tokens,
                                      float alpha, float beta, int32_t* error_flag, fpq_stream_t stream);

// Tensor-core form of the same metric:  sum((A H) .* A) = <H, A^T A>, and A^T A is a Hessian-type product.
// A (fp32) is split into two bf16 terms hi + lo; <H, A^T A> ~= <H, hi^T hi> + 2 <H, hi^T lo> (H is symmetric),
// accurate to ~1e-5 relative -- ample for a logged error metric, and ~10x faster than the fp32 products.
extern "C" int fpq_relative_mse_tc(const float* Wq, const float* W, const float* H, int64_t rows, int64_t d,
                                   void* bf16_workspace, float* gram_workspace, double* acc_workspace, float* out,
                                   int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(Wq && W && H && bf16_workspace && gram_workspace && acc_workspace && out && error_flag, "NULL pointer");
  FPQ_CHECK_ARG(rows > 0 && d > 0 && d % 8 == 0, "d must be a positive multiple of 8");
  cudaStream_t st = (cudaStream_t)stream;
  __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(bf16_workspace);
  __nv_bfloat16* lo = hi + rows * d;
  // slots [0, 1024) and [1024, 2048) of a region take the two terms of a quantity
  for (int which = 0; which < 2; ++which) {
    double* region = acc_workspace + (size_t)which * MSE_REGION;
    split_bf16_kernel<<<grid1d(rows * d), 256, 0, st>>>(which == 0 ? Wq : W, which == 0 ? W : nullptr, hi, lo, rows * d);
    FPQ_CHECK_LAUNCH();
    if (int rc = fpq_hessian_accumulate(gram_workspace, d, hi, nullptr, rows, 1.0f, 0.0f, error_flag, stream)) return rc;
    frobenius_dot_kernel<<<MSE_DOT_BLOCKS, 256, 0, st>>>(H, gram_workspace, d * d, 1.0, region);
    FPQ_CHECK_LAUNCH();
    if (int rc = fpq_hessian_accumulate(gram_workspace, d, hi, lo, rows, 1.0f, 0.0f, error_flag, stream)) return rc;
    frobenius_dot_kernel<<<MSE_DOT_BLOCKS, 256, 0, st>>>(H, gram_workspace, d * d, 2.0, region + MSE_DOT_BLOCKS);
    FPQ_CHECK_LAUNCH();
  }
  ratio_kernel<<<1, 32, 0, st>>>(acc_workspace, 2 * MSE_DOT_BLOCKS, out, (double)rows * (double)d);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}
