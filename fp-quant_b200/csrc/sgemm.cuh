// fp32 SIMT matrix multiply used where the GPTQ path needs true fp32 accuracy (the reference
// switches TF32 off, model_quant.py:27-29 of IST-DASLab/FP-Quant): trailing updates of the
// Cholesky factorisation, the triangular inverse, the GPTQ error propagation and the
// relative-MSE metric.
//
//   C[M,N] = beta * C + alpha * A[M,K] * op(B)      op(B) = B[K,N] (B_T = false) or B[N,K]^T (B_T = true)
//
// All matrices row-major with explicit leading dimensions.  128 x 128 tile, K step 16,
// 256 threads, 8 x 8 outputs per thread, register-prefetched global loads.
// Epilogue variants: plain, lower-triangle only (tiles strictly above the diagonal are skipped,
// for symmetric rank-k updates), and "dot": sum(C_tile .* D) accumulated into a scalar (C not written).
#pragma once

#include "common.cuh"

namespace fpq {

enum SgemmEpilogue { SGEMM_PLAIN = 0, SGEMM_LOWER = 1, SGEMM_DOT = 2 };

struct SgemmArgs {
  const float* A; int64_t lda;
  const float* B; int64_t ldb;
  float* C; int64_t ldc;
  int M, N, K;
  float alpha, beta;
  const float* D; int64_t ldd;   // SGEMM_DOT: elementwise partner
  double* dot_out;               // SGEMM_DOT: one partial sum per CTA, slot blockIdx.y * gridDim.x + blockIdx.x
};

int sgemm(const SgemmArgs& a, bool b_transposed, int epilogue, cudaStream_t stream);

// Independent plain products in one launch (the small nodes of one level of the triangular inverse).
constexpr int SGEMM_MAX_BATCH = 32;
struct SgemmBatch {
  int count;
  SgemmArgs e[SGEMM_MAX_BATCH];
};
int sgemm_batched(const SgemmBatch& b, bool b_transposed, cudaStream_t stream);

}  // namespace fpq
