// fp32 SIMT GEMM (see sgemm.cuh).
#include "sgemm.cuh"

namespace fpq {
namespace {

constexpr int TM = 128, TN = 128, TK = 16, PAD = 4;

__device__ __forceinline__ float4 ld4_guard(const float* base, int64_t ld, int row, int rows, int k, int kmax,
                                            bool vec_ok) {
  // four consecutive K elements of one row (row-major [rows, K]); zeros outside the matrix
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (row < rows) {
    const float* p = base + (int64_t)row * ld + k;
    if (vec_ok && k + 3 < kmax) {
      v = *reinterpret_cast<const float4*>(p);
    } else {
      if (k + 0 < kmax) v.x = p[0];
      if (k + 1 < kmax) v.y = p[1];
      if (k + 2 < kmax) v.z = p[2];
      if (k + 3 < kmax) v.w = p[3];
    }
  }
  return v;
}

template <bool B_T, int EPI>
__device__ __forceinline__ void sgemm_body(const SgemmArgs& a) {
  __shared__ __align__(16) float As[2][TK][TM + PAD];
  __shared__ __align__(16) float Bs[2][TK][TN + PAD];
  const int tid = threadIdx.x;
  const int bm = blockIdx.y * TM, bn = blockIdx.x * TN;
  if (bm >= a.M || bn >= a.N) return;                   // batched launches size the grid for the largest entry
                                                        // (SGEMM_DOT is never batched: its grid covers the matrix exactly)
  if (EPI == SGEMM_LOWER && bn > bm + TM - 1) return;   // tile strictly above the diagonal

  const int ty = tid >> 4, tx = tid & 15;
  const bool a_vec = ((reinterpret_cast<uintptr_t>(a.A) & 15) == 0) && (a.lda % 4 == 0);
  const bool b_vec = ((reinterpret_cast<uintptr_t>(a.B) & 15) == 0) && (a.ldb % 4 == 0);

  // global -> register staging
  float4 ra[2], rb[2];
  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = (tid >> 2) + 64 * h, kq = (tid & 3) * 4;
      ra[h] = ld4_guard(a.A, a.lda, bm + row, a.M, k0 + kq, a.K, a_vec);
      if (B_T) {
        rb[h] = ld4_guard(a.B, a.ldb, bn + row, a.N, k0 + kq, a.K, b_vec);
      } else {
        const int k = (tid >> 5) + 8 * h, n = (tid & 31) * 4;
        // four consecutive N elements of row k of B[K, N]
        rb[h] = ld4_guard(a.B, a.ldb, k0 + k, a.K, bn + n, a.N, b_vec);
      }
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = (tid >> 2) + 64 * h, kq = (tid & 3) * 4;
      As[buf][kq + 0][row] = ra[h].x;
      As[buf][kq + 1][row] = ra[h].y;
      As[buf][kq + 2][row] = ra[h].z;
      As[buf][kq + 3][row] = ra[h].w;
      if (B_T) {
        Bs[buf][kq + 0][row] = rb[h].x;
        Bs[buf][kq + 1][row] = rb[h].y;
        Bs[buf][kq + 2][row] = rb[h].z;
        Bs[buf][kq + 3][row] = rb[h].w;
      } else {
        const int k = (tid >> 5) + 8 * h, n = (tid & 31) * 4;
        *reinterpret_cast<float4*>(&Bs[buf][k][n]) = rb[h];
      }
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int ksteps = (a.K + TK - 1) / TK;
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  for (int ks = 0; ks < ksteps; ++ks) {
    const int buf = ks & 1;
    if (ks + 1 < ksteps) load_tiles((ks + 1) * TK);
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (ks + 1 < ksteps) {
      store_tiles(buf ^ 1);
      __syncthreads();
    }
  }

  // ---- epilogue
  double local = 0.0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = bm + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= a.M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int col0 = bn + jh * 64 + tx * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = col0 + j;
        if (col >= a.N) continue;
        const float v = a.alpha * acc[i][jh * 4 + j];
        if (EPI == SGEMM_DOT) {
          local += (double)v * (double)a.D[(int64_t)row * a.ldd + col];
        } else {
          float* c = a.C + (int64_t)row * a.ldc + col;
          *c = a.beta == 0.f ? v : fmaf(a.beta, *c, v);
        }
      }
    }
  }
  if (EPI == SGEMM_DOT) {
    // one partial sum per CTA, written (not added) to its own slot: the caller sums the slots in a fixed
    // order, so the result does not depend on the order in which CTAs finish
    __shared__ double warp_sum[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((tid & 31) == 0) warp_sum[tid >> 5] = local;
    __syncthreads();
    if (tid == 0) {
      double t = 0.0;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += warp_sum[w];
      a.dot_out[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = t;
    }
  }
}

template <bool B_T, int EPI>
__global__ void __launch_bounds__(256) sgemm_kernel(const SgemmArgs a) {
  sgemm_body<B_T, EPI>(a);
}

// One launch for up to SGEMM_MAX_BATCH independent products (blockIdx.z picks the entry).
template <bool B_T>
__global__ void __launch_bounds__(256) sgemm_batched_kernel(const __grid_constant__ SgemmBatch b) {
  sgemm_body<B_T, SGEMM_PLAIN>(b.e[blockIdx.z]);
}

template <bool B_T>
int launch(const SgemmArgs& a, int epi, cudaStream_t stream) {
  dim3 grid((a.N + TN - 1) / TN, (a.M + TM - 1) / TM);
  if (epi == SGEMM_PLAIN) sgemm_kernel<B_T, SGEMM_PLAIN><<<grid, 256, 0, stream>>>(a);
  else if (epi == SGEMM_LOWER) sgemm_kernel<B_T, SGEMM_LOWER><<<grid, 256, 0, stream>>>(a);
  else sgemm_kernel<B_T, SGEMM_DOT><<<grid, 256, 0, stream>>>(a);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

}  // namespace

int sgemm(const SgemmArgs& a, bool b_transposed, int epilogue, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return FPQ_OK;
  FPQ_CHECK_ARG(a.K >= 0 && a.A && a.B, "sgemm: bad arguments");
  FPQ_CHECK_ARG((a.N + TN - 1) / TN <= 65535 * 32 && (a.M + TM - 1) / TM <= 65535, "sgemm: matrix too large");
  return b_transposed ? launch<true>(a, epilogue, stream) : launch<false>(a, epilogue, stream);
}

int sgemm_batched(const SgemmBatch& b, bool b_transposed, cudaStream_t stream) {
  if (b.count <= 0) return FPQ_OK;
  FPQ_CHECK_ARG(b.count <= SGEMM_MAX_BATCH, "sgemm_batched: too many entries");
  int max_m = 0, max_n = 0;
  for (int i = 0; i < b.count; ++i) {
    FPQ_CHECK_ARG(b.e[i].K >= 0 && b.e[i].A && b.e[i].B && b.e[i].C, "sgemm_batched: bad arguments");
    if (b.e[i].M > max_m) max_m = b.e[i].M;
    if (b.e[i].N > max_n) max_n = b.e[i].N;
  }
  if (max_m <= 0 || max_n <= 0) return FPQ_OK;
  dim3 grid((max_n + TN - 1) / TN, (max_m + TM - 1) / TM, b.count);
  FPQ_CHECK_ARG(grid.y <= 65535, "sgemm_batched: matrix too large");
  if (b_transposed) sgemm_batched_kernel<true><<<grid, 256, 0, stream>>>(b);
  else sgemm_batched_kernel<false><<<grid, 256, 0, stream>>>(b);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

}  // namespace fpq

// C ABI: plain fp32 GEMM, exposed for tests and for host code that needs fp32-accurate products.
extern "C" int fpq_sgemm(const float* A, int64_t lda, const float* B, int64_t ldb, int b_transposed, float* C,
                         int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                         fpq_stream_t stream) {
  FPQ_CHECK_ARG(A && B && C, "NULL pointer");
  FPQ_CHECK_ARG(M >= 0 && N >= 0 && K >= 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "bad shape");
  fpq::SgemmArgs a{};
  a.A = A; a.lda = lda; a.B = B; a.ldb = ldb; a.C = C; a.ldc = ldc;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.alpha = alpha; a.beta = beta;
  return fpq::sgemm(a, b_transposed != 0, fpq::SGEMM_PLAIN, (cudaStream_t)stream);
}
