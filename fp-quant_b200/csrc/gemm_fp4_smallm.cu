// Block-scaled FP4 GEMM for few activation rows (M <= 128; decode) on sm_100a -- the small-M path of
// fpq_gemm_fp4.  Here the run time is the time to stream the weights once, so the kernel is built
// to put every SM on a different slice of the weight matrix:
//   * operands are swapped: 128 weight rows fill the 128-row side of the MMA, the (padded) activation
//     rows are its N side (16..128), so a tile wastes little tensor work however small M is;
//   * K is split over the CTAs of a thread-block cluster (1, 2, 4 or 8); each CTA accumulates its
//     K-range in tensor memory, writes the fp32 partial tile to its own shared memory, and after a
//     cluster barrier every CTA sums one row-slice of the tile over all CTAs through distributed shared
//     memory, applies alpha (+ bias) and stores bf16.  One launch, no global workspace, no atomics.
// Loads are plain TMA into the CTA's own shared memory; all waits are bounded.

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace fpq {
namespace {

using namespace ptx;

constexpr int WROWS = 128;            // weight rows per tile (MMA M)
constexpr int BK_BYTES = 128;
constexpr int BK_ELEMS = 256;
constexpr int STAGES = 5;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int SF_TMEM_BASE = 128;
constexpr int SF_TMEM_BUF = 32;       // A scales (16 columns) + B scales (16 columns)

struct SmallParams {
  int M, N, K;
  int num_k_stages;       // all stages of K
  int stages_per_cta;     // ceil(num_k_stages / cluster size)
  int sf_blocks_k;
  const float* alpha;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int* error_flag;
};

template <bool NVFP4, int NPAD>
struct SmallSmem {
  static constexpr int SFBLK = NVFP4 ? 4 : 2;
  static constexpr int W_BYTES = WROWS * BK_BYTES;       // 16 KiB
  static constexpr int X_BYTES = NPAD * BK_BYTES;
  static constexpr int SF_BYTES = SFBLK * 512;           // per operand
  static constexpr int STAGE_TX = W_BYTES + X_BYTES + 2 * SF_BYTES;
  static constexpr int OFF_W = 0;
  static constexpr int OFF_X = OFF_W + STAGES * W_BYTES;
  static constexpr int X_STRIDE = X_BYTES < 1024 ? 1024 : X_BYTES;   // keep every tile 1024-byte aligned
  static constexpr int OFF_SFW = OFF_X + STAGES * X_STRIDE;
  static constexpr int OFF_SFX = OFF_SFW + STAGES * SF_BYTES;
  static constexpr int OFF_BAR = OFF_SFX + STAGES * SF_BYTES;        // full[S], empty[S], acc_full
  static constexpr int OFF_MISC = OFF_BAR + (2 * STAGES + 1) * 8;
  static constexpr int TOTAL = OFF_MISC + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
  static_assert(STAGES * W_BYTES >= WROWS * NPAD * 4, "the partial tile reuses the weight stages");
};

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}

template <bool NVFP4, int NPAD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp4_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                       const __grid_constant__ CUtensorMap tmap_sfw, const __grid_constant__ CUtensorMap tmap_sfx,
                       const SmallParams p) {
  using L = SmallSmem<NVFP4, NPAD>;
  constexpr int SFBLK = L::SFBLK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_full = sbase + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_acc_full = bar_empty + STAGES * 8;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

  // warp index through a shuffle (known to be the same in all lanes) and single-thread roles through
  // elect.sync: the role code then runs on the uniform datapath, where the operands of tcgen05 / TMA
  // instructions live; with `threadIdx.x >> 5` and `lane == 0` every such instruction cost its thread
  // 75-150 cycles of register moves
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
  const int n_blk = blockIdx.x / csize;                       // 128 weight rows per cluster
  const int ks_begin = (int)rank * p.stages_per_cta;
  int ks_end = ks_begin + p.stages_per_cta;
  if (ks_end > p.num_k_stages) ks_end = p.num_k_stages;
  const int my_stages = ks_end > ks_begin ? ks_end - ks_begin : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_sfw);
    prefetch_tensormap(&tmap_sfx);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      for (int i = 0; i < my_stages; ++i) {
        const int ks = ks_begin + i, s = i % STAGES;
        if (!mbar_wait_bounded(bar_empty + 8 * s, ((i / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const uint32_t full = bar_full + 8 * s;
        mbar_arrive_expect_tx(full, L::STAGE_TX);
        tma_load_2d(sbase + L::OFF_W + s * L::W_BYTES, &tmap_w, ks * BK_BYTES, n_blk * WROWS, full);
        tma_load_2d(sbase + L::OFF_X + s * L::X_STRIDE, &tmap_x, ks * BK_BYTES, 0, full);
        tma_load_2d(sbase + L::OFF_SFW + s * L::SF_BYTES, &tmap_sfw, ks * SFBLK * 64, n_blk, full);
        tma_load_2d(sbase + L::OFF_SFX + s * L::SF_BYTES, &tmap_sfx, ks * SFBLK * 64, 0, full);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
      const int first = my_stages > STAGES ? my_stages - STAGES : 0;
      volatile int never = 0;
      for (int j = first; j < my_stages; ++j)
        (void)mbar_wait_bounded(bar_full + 8 * (j % STAGES), (j / STAGES) & 1, &never, 200000000LL);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = true;
      for (int i = 0; i < my_stages; ++i) {
        const int ks = ks_begin + i, s = i % STAGES;
        if (!mbar_wait_bounded(bar_full + 8 * s, (i / STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sf_buf = tmem_base + SF_TMEM_BASE + (i & 1) * SF_TMEM_BUF;
        const uint32_t sfa_t = sf_buf, sfb_t = sf_buf + 16;
        int nblk = p.sf_blocks_k - ks * SFBLK;
        if (nblk > SFBLK) nblk = SFBLK;
        for (int j = 0; j < nblk; ++j) {
          tc_cp_32x128b_warpx4(sfa_t + 4 * j, make_desc_sf_block(sbase + L::OFF_SFW + s * L::SF_BYTES + j * 512));
          tc_cp_32x128b_warpx4(sfb_t + 4 * j, make_desc_sf_block(sbase + L::OFF_SFX + s * L::SF_BYTES + j * 512));
        }
        int kmma = (p.K - ks * BK_ELEMS + 63) / 64;
        if (kmma > 4) kmma = 4;
        const uint64_t a_desc = make_desc_k_sw128(sbase + L::OFF_W + s * L::W_BYTES);
        const uint64_t b_desc = make_desc_k_sw128(sbase + L::OFF_X + s * L::X_STRIDE);
        for (int k = 0; k < kmma; ++k) {
          uint32_t blk, sf_id;
          if (NVFP4) { blk = k; sf_id = 0; }
          else { blk = k >> 1; sf_id = (k & 1) * 2; }
          const uint32_t idesc = make_idesc_fp4(WROWS, NPAD, !NVFP4, sf_id, sf_id);
          tc_mma_fp4_block_scaled<NVFP4>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa_t + 4 * blk,
                                         sfb_t + 4 * blk, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar_empty + 8 * s);
      }
      if (ok) tc_commit(bar_acc_full);
      else {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
  } else {
    // epilogue warps: partial tile (tensor memory) -> fp32 in shared memory, red[m][n]
    const int quarter = warp & 3;
    float* red = reinterpret_cast<float*>(smem + L::OFF_W);
    const int n_local = quarter * 32 + lane;
    bool have = my_stages > 0;
    if (have && !mbar_wait_bounded(bar_acc_full, 0, abort_flag)) {
      have = false;
      if (lane == 0) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < NPAD / 16; ++c) {
      uint32_t r[16];
      if (have) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16)
            : "memory");
        tc_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) red[(c * 16 + j) * WROWS + n_local] = __uint_as_float(r[j]);
    }
  }

  // ---- split-K reduction across the cluster through distributed shared memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp >= 2) {
    const int t = threadIdx.x - 64;                       // 0..127
    const int rows_per_cta = WROWS / (int)csize;          // my slice of the tile's weight rows (>= 16)
    const int quads_per_row = rows_per_cta / 4;           // groups of four consecutive weight rows
    const int n_quads = quads_per_row * NPAD;
    const float alpha = *p.alpha;
    const uint32_t red_addr = sbase + L::OFF_W;
    uint32_t peer[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) peer[c] = map_to_cta(red_addr, (uint32_t)c < csize ? (uint32_t)c : 0u);
    for (int e = t; e < n_quads; e += 128) {
      const int m = e / quads_per_row;
      const int n_local = (int)rank * rows_per_cta + (e % quads_per_row) * 4;
      const int n = n_blk * WROWS + n_local;
      if (m < p.M && n < p.N) {
        // all remote loads first (they are independent), then the sum
        float4 part[8];
        const uint32_t off = (uint32_t)(m * WROWS + n_local) * 4u;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          part[c] = (uint32_t)c < csize ? ld_cluster_f32x4(peer[c] + off) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = part[0];
#pragma unroll
        for (int c = 1; c < 8; ++c) {
          acc.x += part[c].x; acc.y += part[c].y; acc.z += part[c].z; acc.w += part[c].w;
        }
        float v[4] = {acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha};
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] += __bfloat162float(p.bias[n + j]);
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 w;
        w.x = *reinterpret_cast<uint32_t*>(&lo);
        w.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + (size_t)m * p.N + n) = w;
      }
    }
  }
  cluster_sync_all();                                     // nobody leaves while its partial is still being read
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool NVFP4, int NPAD>
int launch_small(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tsw, const CUtensorMap& tsx,
                 const SmallParams& p, int clusters, int csize, cudaStream_t stream) {
  using L = SmallSmem<NVFP4, NPAD>;
  auto kern = gemm_fp4_smallm_kernel<NVFP4, NPAD>;
  static bool configured[64] = {};
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * csize), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L::DYN_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tw, tx, tsw, tsx, p));
  return FPQ_OK;
}

template <bool NVFP4>
int dispatch_npad(int npad, const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tsw,
                  const CUtensorMap& tsx, const SmallParams& p, int clusters, int csize, cudaStream_t stream) {
  switch (npad) {
    case 16: return launch_small<NVFP4, 16>(tw, tx, tsw, tsx, p, clusters, csize, stream);
    case 32: return launch_small<NVFP4, 32>(tw, tx, tsw, tsx, p, clusters, csize, stream);
    case 64: return launch_small<NVFP4, 64>(tw, tx, tsw, tsx, p, clusters, csize, stream);
    default: return launch_small<NVFP4, 128>(tw, tx, tsw, tsx, p, clusters, csize, stream);
  }
}

}  // namespace

int make_tensor_map_2d_u64(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer);

// Small-M path of fpq_gemm_fp4 (M <= 128).  Shapes and pointers were validated by the caller.
int gemm_fp4_smallm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                    const void* bias, void* out, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                    cudaStream_t stream) {
  const int g = format == FPQ_FMT_NVFP4 ? 16 : 32;
  const int sfblk = format == FPQ_FMT_NVFP4 ? 4 : 2;
  const int npad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  SmallParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.num_k_stages = (int)((K + BK_ELEMS - 1) / BK_ELEMS);
  p.sf_blocks_k = (int)((K / g + 3) / 4);
  p.alpha = alpha;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.error_flag = error_flag;
  const int clusters = (int)((N + WROWS - 1) / WROWS);
  // split K so that about one CTA per SM is busy, but keep at least two stages per CTA
  int csize = 1;
  while (csize < 8 && clusters * csize * 2 <= sm_count() + sm_count() / 2 && p.num_k_stages / (csize * 2) >= 2) csize *= 2;
  p.stages_per_cta = (p.num_k_stages + csize - 1) / csize;
  CUtensorMap tw, tx, tsw, tsx;
  if (int rc = make_tensor_map_2d(&tw, b, 1, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, BK_BYTES, WROWS, 1)) return rc;
  if (int rc = make_tensor_map_2d(&tx, a, 1, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, BK_BYTES, (uint32_t)npad, 1)) return rc;
  const uint64_t sf_row_words = (uint64_t)p.sf_blocks_k * 64;
  if (int rc = make_tensor_map_2d_u64(&tsw, sfb, sf_row_words, (uint64_t)((N + 127) / 128), sf_row_words * 8,
                                      (uint32_t)sfblk * 64, 1)) return rc;
  if (int rc = make_tensor_map_2d_u64(&tsx, sfa, sf_row_words, (uint64_t)((M + 127) / 128), sf_row_words * 8,
                                      (uint32_t)sfblk * 64, 1)) return rc;
  return format == FPQ_FMT_NVFP4 ? dispatch_npad<true>(npad, tw, tx, tsw, tsx, p, clusters, csize, stream)
                                 : dispatch_npad<false>(npad, tw, tx, tsw, tsx, p, clusters, csize, stream);
}

}  // namespace fpq
