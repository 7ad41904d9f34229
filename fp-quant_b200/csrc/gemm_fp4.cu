// Block-scaled FP4 x FP4 -> bf16 matmul for sm_100a:  Y[M,N] = alpha * dq(A)[M,K] * dq(B)[N,K]^T (+ bias).
//
// Replaces qutlass.matmul_mxf4_bf16_tn / matmul_nvf4_bf16_tn as called from
// inference_lib/src/fp_quant/module/qutlass_ops.py:111-168 of IST-DASLab/FP-Quant.
//
// Structure (one persistent CTA per SM, 6 warps):
//   warp 0   TMA producer: 128-byte x rows boxes of packed E2M1 codes (128B swizzle) plus the
//            matching 512-byte scale-factor blocks, 4-stage ring guarded by mbarriers
//   warp 1   allocates tensor memory; one lane copies scale blocks shared->tensor memory
//            (tcgen05.cp) and issues tcgen05.mma.kind::mxf4 / mxf4nvf4 .block_scale
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulator, * alpha (+ bias), -> bf16, global stores
// Tile 128 x BN x 256 (K elements per stage = one 128-byte swizzle row); BN = 256 or 128.
// Tensor memory: accumulator in columns [0, BN), two alternating scale-factor buffers above it.
// Every mbarrier wait is bounded; on a timeout the CTA raises *error_flag and leaves.

#include "common.cuh"
#include "sm100_ptx.cuh"

#include <cstdlib>

namespace fpq {
namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK_BYTES = 128;          // packed bytes of K per stage
constexpr int BK_ELEMS = 256;
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SF_TMEM_BASE = 256;      // first scale-factor column
constexpr int SF_TMEM_BUF = 64;        // columns per scale-factor buffer (16 for A, up to 32 for B)

struct GemmParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_tiles;
  int num_k_stages;        // ceil(K / 256)
  int sf_blocks_k;         // 512-byte scale blocks per 128 rows along K: ceil((K/g)/4)
  int sfa_row_blocks, sfb_row_blocks;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int* error_flag;
  int raster_group;        // m-blocks per rasterisation band
};

// Tile index -> (m block, n block): bands of `raster_group` m-blocks, n-blocks swept inside a band with
// m fastest, so that CTAs running at the same time share both A and B tiles through L2 instead of
// all asking for the same B tile.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_blk, int& n_blk) {
  const int band_tiles = p.raster_group * p.num_n_blocks;
  const int band = tile / band_tiles;
  const int first_m = band * p.raster_group;
  int rows = p.num_m_blocks - first_m;
  if (rows > p.raster_group) rows = p.raster_group;
  const int in_band = tile - band * band_tiles;
  m_blk = first_m + in_band % rows;
  n_blk = in_band / rows;
}

template <int BN, bool NVFP4>
struct SmemLayout {
  static constexpr int SFB_PER_STAGE = NVFP4 ? 4 : 2;             // 512-byte blocks per 128 rows per stage
  static constexpr int A_BYTES = BM * BK_BYTES;                   // 16 KiB
  static constexpr int B_BYTES = BN * BK_BYTES;                   // 32 KiB
  static constexpr int SFA_BYTES = SFB_PER_STAGE * 512;
  static constexpr int SFB_BYTES = (BN / 128) * SFB_PER_STAGE * 512;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_SFA = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_SFB = OFF_SFA + STAGES * SFA_BYTES;
  static constexpr int OFF_BAR = OFF_SFB + STAGES * SFB_BYTES;   // full[S], empty[S], acc_full, acc_empty
  static constexpr int OFF_MISC = OFF_BAR + (2 * STAGES + 2) * 8; // tmem base, abort flag
  static constexpr int TOTAL = OFF_MISC + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;                  // slack for 1024-byte alignment
};

template <int BN, bool NVFP4>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmParams p) {
  using L = SmemLayout<BN, NVFP4>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_full = sbase + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_acc_full = bar_empty + STAGES * 8;
  const uint32_t bar_acc_empty = bar_acc_full + 8;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

  // warp index through a shuffle (known to be the same in all lanes) and single-thread roles through
  // elect.sync: the role code then runs on the uniform datapath, where the operands of tcgen05 / TMA
  // instructions live; with `threadIdx.x >> 5` and `lane == 0` every such instruction cost its thread
  // 75-150 cycles of register moves
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 4);   // one arrive per epilogue warp
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  constexpr int SFBLK = L::SFB_PER_STAGE;
  constexpr uint32_t STAGE_TX_AB = L::A_BYTES + L::B_BYTES;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t it = 0;   // global stage counter
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(p, tile, m_blk, n_blk);
        for (int ks = 0; ks < p.num_k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1, abort_flag)) { ok = false; break; }
          int nblk = p.sf_blocks_k - ks * SFBLK;
          if (nblk > SFBLK) nblk = SFBLK;
          int nb_rowblocks = 0;
          for (int h = 0; h < BN / 128; ++h)
            if (n_blk * (BN / 128) + h < p.sfb_row_blocks) ++nb_rowblocks;
          const uint32_t tx = STAGE_TX_AB + (uint32_t)nblk * 512u * (1 + nb_rowblocks);
          mbar_arrive_expect_tx(bar_full + 8 * s, tx);
          tma_load_2d(sbase + L::OFF_A + s * L::A_BYTES, &tmap_a, ks * BK_BYTES, m_blk * BM, bar_full + 8 * s);
          tma_load_2d(sbase + L::OFF_B + s * L::B_BYTES, &tmap_b, ks * BK_BYTES, n_blk * BN, bar_full + 8 * s);
          bulk_load(sbase + L::OFF_SFA + s * L::SFA_BYTES,
                    p.sfa + ((size_t)m_blk * p.sf_blocks_k + (size_t)ks * SFBLK) * 512, (uint32_t)nblk * 512u,
                    bar_full + 8 * s);
          for (int h = 0; h < BN / 128; ++h) {
            const int rb = n_blk * (BN / 128) + h;
            if (rb < p.sfb_row_blocks)
              bulk_load(sbase + L::OFF_SFB + s * L::SFB_BYTES + h * SFBLK * 512,
                        p.sfb + ((size_t)rb * p.sf_blocks_k + (size_t)ks * SFBLK) * 512, (uint32_t)nblk * 512u,
                        bar_full + 8 * s);
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
      // Drain: every load issued must have landed before this CTA's shared memory is released.
      // The consumer releases a stage only after its full barrier completed, so it is enough to
      // see the last min(it, STAGES) stages complete.
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      volatile int never = 0;   // the drain must not be cut short by the abort flag
      for (uint32_t j = first; j < it; ++j)
        (void)mbar_wait_bounded(bar_full + 8 * (j % STAGES), (j / STAGES) & 1, &never, 200000000LL);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0;
      uint32_t tile_count = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tile_count) {
        // accumulator must have been drained by the epilogue of the previous tile
        if (!mbar_wait_bounded(bar_acc_empty, (tile_count & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int ks = 0; ks < p.num_k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(bar_full + 8 * s, ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sf_buf = tmem_base + SF_TMEM_BASE + (it & 1) * SF_TMEM_BUF;
          const uint32_t sfa_t = sf_buf;            // 4 columns per 512-byte block
          const uint32_t sfb_t = sf_buf + 16;       // (BN/32) columns per block
          int nblk = p.sf_blocks_k - ks * SFBLK;
          if (nblk > SFBLK) nblk = SFBLK;
          for (int j = 0; j < nblk; ++j) {
            tc_cp_32x128b_warpx4(sfa_t + 4 * j, make_desc_sf_block(sbase + L::OFF_SFA + s * L::SFA_BYTES + j * 512));
            for (int h = 0; h < BN / 128; ++h)
              tc_cp_32x128b_warpx4(sfb_t + (BN / 32) * j + 4 * h,
                                   make_desc_sf_block(sbase + L::OFF_SFB + s * L::SFB_BYTES + (h * SFBLK + j) * 512));
          }
          int kmma = (p.K - ks * BK_ELEMS + 63) / 64;   // K=64 MMAs in this stage
          if (kmma > 4) kmma = 4;
          const uint64_t a_desc = make_desc_k_sw128(sbase + L::OFF_A + s * L::A_BYTES);
          const uint64_t b_desc = make_desc_k_sw128(sbase + L::OFF_B + s * L::B_BYTES);
          for (int k = 0; k < kmma; ++k) {
            uint32_t blk, sf_id;
            if (NVFP4) { blk = k; sf_id = 0; }           // 4 scales of 16 per MMA: one whole block
            else { blk = k >> 1; sf_id = (k & 1) * 2; }  // 2 scales of 32 per MMA: half a block
            const uint32_t idesc = make_idesc_fp4(BM, BN, !NVFP4, sf_id, sf_id);
            tc_mma_fp4_block_scaled<NVFP4>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa_t + 4 * blk,
                                           sfb_t + (BN / 32) * blk, (ks > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * s);   // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(bar_acc_full);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
    const float alpha = *p.alpha;
    uint32_t tile_count = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tile_count) {
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      if (!mbar_wait_bounded(bar_acc_full, tile_count & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      __nv_bfloat16* orow = p.out + (size_t)row * p.N;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 32, r);
        tc_wait_ld();
        const int col0 = n_blk * BN + c * 32;
        if (row < p.M && col0 + 32 <= p.N) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v0 = __uint_as_float(r[2 * j]) * alpha;
            float v1 = __uint_as_float(r[2 * j + 1]) * alpha;
            if (p.bias) {
              v0 += __bfloat162float(p.bias[col0 + 2 * j]);
              v1 += __bfloat162float(p.bias[col0 + 2 * j + 1]);
            }
            __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + col0);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else if (row < p.M && col0 < p.N) {
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) {   // ragged right edge
            float v = __uint_as_float(r[j]) * alpha;
            if (p.bias) v += __bfloat162float(p.bias[col0 + j]);
            orow[col0 + j] = __float2bfloat16_rn(v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicExch(p.error_flag, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, bool NVFP4>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t stream) {
  using L = SmemLayout<BN, NVFP4>;
  auto kern = gemm_fp4_kernel<BN, NVFP4>;
  static bool configured[64] = {};
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    configured[dev] = true;
  }
  p.num_n_blocks = (p.N + BN - 1) / BN;
  p.num_tiles = p.num_m_blocks * p.num_n_blocks;
  p.raster_group = 8;
  int grid = sm_count();
  if (grid > p.num_tiles) grid = p.num_tiles;
  kern<<<grid, NUM_THREADS, L::DYN_BYTES, stream>>>(ta, tb, p);
  FPQ_CHECK_LAUNCH();
  return FPQ_OK;
}

}  // namespace

// ---------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Encoding a tensor map costs about a microsecond of host time; weights and their scales are the same
// buffers call after call, so the most recent encodings are kept per thread.
struct MapKey {
  const void* base; uint64_t inner, outer, stride; uint32_t box_inner, box_outer; int kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
           box_outer == o.box_outer && kind == o.kind;
  }
};
struct MapCache {
  static constexpr int N = 32;
  MapKey keys[N];
  CUtensorMap maps[N];
  int used = 0, next = 0;
  const CUtensorMap* find(const MapKey& k) const {
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) return &maps[i];
    return nullptr;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    const int slot = used < N ? used++ : (next++ % N);
    keys[slot] = k;
    maps[slot] = m;
  }
};
static thread_local MapCache g_map_cache;

int make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_128b) {
  const MapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, elem_bytes * 2 + (swizzle_128b ? 1 : 0)};
  if (const CUtensorMap* hit = g_map_cache.find(key)) {
    *map = *hit;
    return FPQ_OK;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return FPQ_ERR_CUDA;
  }
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                         : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu stride=%llu box=%ux%u)", (int)r,
              (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_bytes, box_inner,
              box_outer);
    return FPQ_ERR_CUDA;
  }
  g_map_cache.put(key, *map);
  return FPQ_OK;
}

int make_tensor_map_2d_u64(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer) {
  const MapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, 64};
  if (const CUtensorMap* hit = g_map_cache.find(key)) {
    *map = *hit;
    return FPQ_OK;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return FPQ_ERR_CUDA;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (scale tiles) failed with CUresult %d (inner=%llu outer=%llu box=%ux%u)", (int)r,
              (unsigned long long)inner, (unsigned long long)outer, box_inner, box_outer);
    return FPQ_ERR_CUDA;
  }
  g_map_cache.put(key, *map);
  return FPQ_OK;
}

int gemm_fp4_pair(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                  const void* bias, void* out, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                  cudaStream_t stream, int64_t ldc = 0, void* const* peers = nullptr, int n_peers = 0);
int gemm_fp4_smallm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                    const void* bias, void* out, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                    cudaStream_t stream);

}  // namespace fpq

using namespace fpq;

extern "C" int fpq_gemm_fp4(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* a_scales_swizzled,
                            const uint8_t* b_scales_swizzled, const float* alpha, const void* bias_bf16,
                            void* out_bf16, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                            fpq_stream_t stream) {
  FPQ_CHECK_ARG(a_codes && b_codes && a_scales_swizzled && b_scales_swizzled && alpha && out_bf16 && error_flag,
                "NULL pointer");
  FPQ_CHECK_ARG(format == FPQ_FMT_MXFP4 || format == FPQ_FMT_NVFP4, "bad format");
  FPQ_CHECK_ARG(M >= 0 && N > 0 && K > 0, "bad shape");
  FPQ_CHECK_ARG(K % 64 == 0, "K (%lld) must be a multiple of 64", (long long)K);
  FPQ_CHECK_ARG(N % 8 == 0, "N (%lld) must be a multiple of 8", (long long)N);
  FPQ_CHECK_ARG(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)a_codes & 15) == 0 && ((uintptr_t)b_codes & 15) == 0 &&
                    ((uintptr_t)a_scales_swizzled & 15) == 0 && ((uintptr_t)b_scales_swizzled & 15) == 0 &&
                    ((uintptr_t)out_bf16 & 15) == 0,
                "pointers must be 16-byte aligned");
  FPQ_CHECK_ARG((K / 2) % 16 == 0, "K/2 must be a multiple of 16 bytes");
  if (M == 0) return FPQ_OK;
  {
    // Large M: CTA pairs (256 x 256 tiles).  Small M streams the weights once and stays on single CTAs.
    // Up to 64 tokens the swap-AB kernel always wins; up to 128 it wins when the 128-row weight blocks
    // leave SMs free for split-K (measured under graph replay: 9.6 vs 18.4 us at N = K = 4096,
    // 14.4 vs 39.0 us at K = 12288, but 25.1 vs 20.0 us at N = 12288).
    const bool small = M <= 64 || (M <= 128 && (N + 127) / 128 <= sm_count() / 2);
    if (small)
      return gemm_fp4_smallm(a_codes, b_codes, a_scales_swizzled, b_scales_swizzled, alpha, bias_bf16, out_bf16, M, N,
                             K, format, error_flag, (cudaStream_t)stream);
    if (M > 128 && N >= 256)
      return gemm_fp4_pair(a_codes, b_codes, a_scales_swizzled, b_scales_swizzled, alpha, bias_bf16, out_bf16, M, N, K,
                           format, error_flag, (cudaStream_t)stream);
  }
  const int g = format == FPQ_FMT_NVFP4 ? 16 : 32;
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.num_m_blocks = (int)((M + BM - 1) / BM);
  p.num_k_stages = (int)((K + BK_ELEMS - 1) / BK_ELEMS);
  p.sf_blocks_k = (int)((K / g + 3) / 4);
  p.sfa_row_blocks = (int)((M + 127) / 128);
  p.sfb_row_blocks = (int)((N + 127) / 128);
  p.sfa = a_scales_swizzled; p.sfb = b_scales_swizzled;
  p.alpha = alpha;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias_bf16);
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.error_flag = error_flag;
  const bool bn256 = N >= 256;
  const int bn = bn256 ? 256 : 128;
  CUtensorMap ta, tb;
  if (int rc = make_tensor_map_2d(&ta, a_codes, 1, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, BK_BYTES, BM, 1)) return rc;
  if (int rc = make_tensor_map_2d(&tb, b_codes, 1, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, BK_BYTES, bn, 1)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (format == FPQ_FMT_NVFP4)
    return bn256 ? launch_gemm<256, true>(ta, tb, p, st) : launch_gemm<128, true>(ta, tb, p, st);
  return bn256 ? launch_gemm<256, false>(ta, tb, p, st) : launch_gemm<128, false>(ta, tb, p, st);
}

extern "C" int fpq_gemm_mxf8(const uint8_t* a_e4m3, const uint8_t* b_e4m3, const uint8_t* a_scales_swizzled,
                             const uint8_t* b_scales_swizzled, const float* alpha, void* out_bf16, int64_t M, int64_t N,
                             int64_t K, int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(a_e4m3 && b_e4m3 && a_scales_swizzled && b_scales_swizzled && alpha && out_bf16 && error_flag,
                "NULL pointer");
  FPQ_CHECK_ARG(M >= 0 && N > 0 && K > 0, "bad shape");
  FPQ_CHECK_ARG(K % 32 == 0, "K (%lld) must be a multiple of 32", (long long)K);
  FPQ_CHECK_ARG(N % 8 == 0, "N (%lld) must be a multiple of 8", (long long)N);
  FPQ_CHECK_ARG(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)a_e4m3 & 15) == 0 && ((uintptr_t)b_e4m3 & 15) == 0 &&
                    ((uintptr_t)a_scales_swizzled & 15) == 0 && ((uintptr_t)b_scales_swizzled & 15) == 0 &&
                    ((uintptr_t)out_bf16 & 15) == 0,
                "pointers must be 16-byte aligned");
  if (M == 0) return FPQ_OK;
  // one kernel for every shape: rows beyond M or N are zero-filled by the loads and clipped by the stores
  return gemm_fp4_pair(a_e4m3, b_e4m3, a_scales_swizzled, b_scales_swizzled, alpha, nullptr, out_bf16, M, N, K,
                       FPQ_FMT_MXFP8, error_flag, (cudaStream_t)stream);
}

extern "C" int fpq_gemm_fp4_push(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* a_scales_swizzled,
                                 const uint8_t* b_scales_swizzled, const float* alpha, const void* bias_bf16,
                                 void* out_bf16, void* const* peer_outs, int n_peers, int64_t ldc, int64_t col_offset,
                                 int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(a_codes && b_codes && a_scales_swizzled && b_scales_swizzled && alpha && out_bf16 && error_flag,
                "NULL pointer");
  FPQ_CHECK_ARG(format == FPQ_FMT_MXFP4 || format == FPQ_FMT_NVFP4, "bad format");
  FPQ_CHECK_ARG(n_peers >= 0 && n_peers <= 7 && (n_peers == 0 || peer_outs), "0..7 peer buffers");
  FPQ_CHECK_ARG(M > 128 && N >= 256 && K > 0, "the pushing GEMM is the large-M kernel: M > 128, N >= 256");
  FPQ_CHECK_ARG(K % 64 == 0 && (K / 2) % 16 == 0 && N % 8 == 0, "K must be a multiple of 64, N of 8");
  FPQ_CHECK_ARG(ldc >= col_offset + N && ldc % 8 == 0 && col_offset % 8 == 0, "bad output stride / column offset");
  FPQ_CHECK_ARG(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)out_bf16 & 15) == 0, "pointers must be 16-byte aligned");
  void* peers[7] = {};
  for (int i = 0; i < n_peers; ++i) {
    FPQ_CHECK_ARG(peer_outs[i] && ((uintptr_t)peer_outs[i] & 15) == 0, "peer pointers must be 16-byte aligned");
    peers[i] = reinterpret_cast<__nv_bfloat16*>(peer_outs[i]) + col_offset;
  }
  return gemm_fp4_pair(a_codes, b_codes, a_scales_swizzled, b_scales_swizzled, alpha, bias_bf16,
                       reinterpret_cast<__nv_bfloat16*>(out_bf16) + col_offset, M, N, K, format, error_flag,
                       (cudaStream_t)stream, ldc, peers, n_peers);
}
