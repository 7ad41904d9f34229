// Hessian accumulation for GPTQ on sm_100a:  H[d,d] (fp32) = beta * H + alpha * X^T X,  X [T,d] bf16.
//
// Replaces the Triton kernel accumulate_hessian_triton_kernel
// (src/quantization/accumulate_hessian.py:20-109 of IST-DASLab/FP-Quant) and the rescaling around it in
// GPTQ.update (src/quantization/gptq.py:94-102).  bf16 x bf16 products are exact in the fp32
// accumulator, so the result is more accurate than the reference's TF32 dot of fp32-cast inputs.
//
// X^T X is a GEMM whose two operands are the same row-major matrix read "MN-major": a TMA box of
// 64 columns x 64 tokens with the 128-byte swizzle lands in shared memory exactly in the canonical
// MN-major layout of tcgen05.mma (8 token rows of 128 bytes per swizzle atom).  Persistent CTAs walk
// tiles that are 256 columns wide (an MMA instruction costs the same ~180 cycles for N = 128 and N = 256,
// so only the wide tile keeps the tensor pipe busy) and 128 or 256 rows high (see Shape below), those that
// touch the lower triangle or all of them for the general A^T B form.  Of a tile on the diagonal only the
// 128-column blocks at or below it are written; blocks below the diagonal are also written mirrored, so
// H stays fully symmetric like the reference's.  Warp roles and bounded waits as in the FP4 GEMM.  The
// 256 x 256 shape runs on CTA pairs (hessian_pair_kernel below): measured against the single-CTA form in one
// process, 4.55 instead of 5.13 ms for the Hessian of 262144 tokens x 4096 and 45.5 instead of 55.5 ms for 14336.
//
// The same kernel is the package's general bf16 A^T B product: K may be a concatenation of segments (the
// cross products of multi-term bf16 splits in one launch), operands may start at a column offset, and the
// stages that would only multiply the zero half of a triangular factor can be skipped.

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace fpq {
namespace {

using namespace ptx;

constexpr int TILE = 128;            // output tile rows (A^T side) and the unit of the triangle
constexpr int TILE_N = 256;          // output tile columns
constexpr int BK = 64;               // tokens per stage
constexpr int BOX_BYTES = BK * 128;  // one 64-column x 64-token box
constexpr int B_BOXES = TILE_N / 64;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;       // two 256-column accumulators

// Two tile shapes.  128 x 256 on single CTAs with two accumulators in flight (the epilogue of a tile overlaps
// the next tile's MMAs) for short K; 256 x 256 on CTA pairs (PairShape below) for long K, where what limits
// the kernel is the operand traffic from L2.  (BIG = true describes the 256-row tiling the pair kernel walks;
// the single-CTA kernel is only instantiated for BIG = false.)
template <bool BIG>
struct Shape {
  static constexpr int TM = BIG ? 256 : 128;
  static constexpr int HALVES = TM / 128;
  static constexpr int A_BOXES = TM / 64;
  static constexpr int STAGES = BIG ? 3 : 4;
  static constexpr int NBUF = BIG ? 1 : 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BOXES * BOX_BYTES;
  static constexpr int OFF_BAR = OFF_B + STAGES * B_BOXES * BOX_BYTES;   // full[S], empty[S], acc_full[2], acc_empty[2]
  static constexpr int OFF_MISC = OFF_BAR + (2 * STAGES + 4) * 8;
  static constexpr int TOTAL = OFF_MISC + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

constexpr int MAX_SEGMENTS = 6;

struct HessParams {
  int64_t d1, d2, ldc;  // output rows (A's width), columns (B's width), row stride of the output
  int num_blocks;      // ceil(d1 / 128)
  int num_blocks_n;    // ceil(d2 / 256)
  int num_tiles;
  int n_seg;           // K segments
  int seg_stages;      // stages per segment: stage ks reads rows a_seg_y[ks / seg_stages] + (ks % seg_stages) * 64
  int symmetric;       // only tiles that touch the lower triangle
  int mirror;          // symmetric form: also write the transposed blocks above the diagonal
  int a_x0, b_x0;      // first column of A / B inside their matrices (added to the TMA x coordinate)
  int tri;             // 0: dense; 1: B is lower triangular (B[k, j] = 0 for k < j): stages below the tile's first
                       // column are skipped; 2: A^T is lower triangular (A[k, i] = 0 for k > i): stages beyond the
                       // tile's last row are skipped
  int a_seg_y[MAX_SEGMENTS], b_seg_y[MAX_SEGMENTS];
  float alpha, beta;
  float* H;
  int* error_flag;
};


// MN-major operand, 128-byte swizzle: 64 contiguous MN elements per 128-byte row, 8 K rows per atom
// (`sbo` bytes between atoms along K), further 64-wide MN blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Symmetric form, 128 x 256 tiles: row block ib (128 rows) needs the column tiles jb2 = 0 .. ib / 2 (256 columns
// each).  Tiles are numbered row by row; rows 0 .. ib-1 hold q (q + 1) tiles for ib = 2 q and (q + 1)^2 for
// ib = 2 q + 1.  256 x 256 tiles: the plain lower triangle of 256-blocks, ib (ib + 1) / 2 tiles before row ib.
__host__ __device__ inline int tiles_before_row(int ib, bool big) {
  if (big) return ib * (ib + 1) / 2;
  const int q = ib >> 1;
  return (ib & 1) ? (q + 1) * (q + 1) : q * (q + 1);
}

template <bool BIG>
__device__ __forceinline__ void tile_coords(const HessParams& p, int tile, int& ib, int& jb2) {
  if (p.symmetric) {
    int i = (int)((BIG ? 1.41421356f : 2.0f) * sqrtf((float)tile)) - 1;
    if (i < 0) i = 0;
    while (tiles_before_row(i + 1, BIG) <= tile) ++i;
    while (tiles_before_row(i, BIG) > tile) --i;
    ib = i;
    jb2 = tile - tiles_before_row(i, BIG);
  } else {
    ib = tile / p.num_blocks_n;
    jb2 = tile - ib * p.num_blocks_n;
  }
}

// Stages [lo, hi) of every K segment that can contribute to tile (ib, jb2).
__device__ __forceinline__ void stage_range(const HessParams& p, int ib, int jb2, int& lo, int& hi) {
  lo = 0;
  hi = p.seg_stages;
  if (p.tri == 1) lo = min(jb2 * (TILE_N / BK), p.seg_stages - 1);
  if (p.tri == 2) hi = max(1, min(p.seg_stages, (ib + 1) * (TILE / BK)));
}

template <bool BIG>
__global__ void __launch_bounds__(NUM_THREADS, 1)
hessian_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const HessParams p) {
  using Smem = Shape<BIG>;
  constexpr int STAGES = Smem::STAGES, A_BOXES = Smem::A_BOXES, TM = Smem::TM, HALVES = Smem::HALVES, NBUF = Smem::NBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_full = sbase + Smem::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_acc_full = bar_empty + STAGES * 8;   // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;       // [2]
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::OFF_MISC + 4);
  // warp index through a shuffle (known to be the same in all lanes) and single-thread roles through
  // elect.sync: the role code then runs on the uniform datapath, where the operands of tcgen05 / TMA
  // instructions live; with `threadIdx.x >> 5` and `lane == 0` every such instruction cost its thread
  // 75-150 cycles of register moves
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
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
  // Barriers, tensor memory and descriptors touched nothing another kernel wrote: with a programmatic
  // dependent launch all of the above overlaps the tail of the previous kernel; operands and the output
  // (read-modify-write) are only touched from here on.
  launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int ib, jb;
        tile_coords<BIG>(p, tile, ib, jb);
        int lo, hi;
        stage_range(p, ib, jb, lo, hi);
        const int per_seg = hi - lo, n_st = per_seg * p.n_seg;
        for (int ks = 0; ks < n_st; ++ks, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_bounded(bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_full + 8 * s, (A_BOXES + B_BOXES) * BOX_BYTES);
          const uint32_t a_dst = sbase + Smem::OFF_A + s * A_BOXES * BOX_BYTES;
          const uint32_t b_dst = sbase + Smem::OFF_B + s * B_BOXES * BOX_BYTES;
          const int seg = ks / per_seg, kk = lo + (ks - seg * per_seg);
          const int ya = p.a_seg_y[seg] + kk * BK;
          const int yb = p.b_seg_y[seg] + kk * BK;
#pragma unroll
          for (int b = 0; b < A_BOXES; ++b)
            tma_load_2d(a_dst + b * BOX_BYTES, &tmap_a, p.a_x0 + ib * TM + 64 * b, ya, bar_full + 8 * s);
#pragma unroll
          for (int b = 0; b < B_BOXES; ++b)
            tma_load_2d(b_dst + b * BOX_BYTES, &tmap_b, p.b_x0 + jb * TILE_N + 64 * b, yb, bar_full + 8 * s);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      volatile int never = 0;
      for (uint32_t j = first; j < it; ++j)
        (void)mbar_wait_bounded(bar_full + 8 * (j % STAGES), (j / STAGES) & 1, &never, 200000000LL);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(TILE, TILE_N, true, true);   // per 128-row half
      uint32_t it = 0, tile_count = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tile_count) {
        const uint32_t buf = NBUF == 2 ? (tile_count & 1) : 0;
        const uint32_t acc_parity = NBUF == 2 ? ((tile_count >> 1) & 1) : (tile_count & 1);
        if (!mbar_wait_bounded(bar_acc_empty + 8 * buf, acc_parity ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * TILE_N;
        int ib, jb, lo, hi;
        tile_coords<BIG>(p, tile, ib, jb);
        stage_range(p, ib, jb, lo, hi);
        const int n_st = (hi - lo) * p.n_seg;
        // one barrier wait, four MMAs and one commit per stage: every other instruction here is time the
        // tensor pipe idles (the operands come through TMA, which needs no tcgen05 fence)
        for (int ks = 0; ks < n_st; ++ks, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_bounded_spin(bar_full + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          const uint64_t a_desc = make_desc_mn_sw128(sbase + Smem::OFF_A + s * A_BOXES * BOX_BYTES, BOX_BYTES, 1024);
          const uint64_t b_desc = make_desc_mn_sw128(sbase + Smem::OFF_B + s * B_BOXES * BOX_BYTES, BOX_BYTES, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {  // 16 tokens per MMA = two 8-row atoms = 2048 bytes
#pragma unroll
            for (int h = 0; h < HALVES; ++h)   // 128-row halves of the tile: boxes 2h, 2h+1 of A, accumulator h
              tc_mma_f16(acc + h * TILE_N, a_desc + (uint64_t)((h * 2 * BOX_BYTES + k * 2048) >> 4),
                         b_desc + (uint64_t)(k * (2048 >> 4)), idesc, (ks > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * s);
        }
        if (ok) tc_commit(bar_acc_full + 8 * buf);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t tile_count = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tile_count) {
      int ib, jb;
      tile_coords<BIG>(p, tile, ib, jb);
      const uint32_t buf = NBUF == 2 ? (tile_count & 1) : 0;
      const uint32_t acc_parity = NBUF == 2 ? ((tile_count >> 1) & 1) : (tile_count & 1);
      if (!mbar_wait_bounded(bar_acc_full + 8 * buf, acc_parity, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int hc = 0; hc < HALVES * (TILE_N / 32); ++hc) {
        const int h = hc / (TILE_N / 32), c = hc % (TILE_N / 32);
        const int rb = ib * HALVES + h;                      // 128-row block of this half
        const int64_t i = (int64_t)rb * TILE + quarter * 32 + lane;
        const int64_t j0 = (int64_t)jb * TILE_N + c * 32;
        const int jblock = (int)(j0 / TILE);                 // 128-column block of this chunk
        if (j0 >= p.d2 || (p.symmetric && jblock > rb)) continue;   // beyond the matrix / above the diagonal
        const bool mirror = p.mirror && jblock < rb;
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TILE_N + h * TILE_N + c * 32, r);
        tc_wait_ld();
        if (i < p.d1) {
          float* hrow = p.H + i * p.ldc + j0;
          if (j0 + 32 <= p.d2 && (p.ldc & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 h = p.beta == 0.0f ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(hrow)[q];
              h.x = fmaf(p.beta, h.x, p.alpha * __uint_as_float(r[4 * q]));
              h.y = fmaf(p.beta, h.y, p.alpha * __uint_as_float(r[4 * q + 1]));
              h.z = fmaf(p.beta, h.z, p.alpha * __uint_as_float(r[4 * q + 2]));
              h.w = fmaf(p.beta, h.w, p.alpha * __uint_as_float(r[4 * q + 3]));
              reinterpret_cast<float4*>(hrow)[q] = h;
              r[4 * q] = __float_as_uint(h.x); r[4 * q + 1] = __float_as_uint(h.y);
              r[4 * q + 2] = __float_as_uint(h.z); r[4 * q + 3] = __float_as_uint(h.w);
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              if (j0 + jj < p.d2) {
                const float old = p.beta == 0.0f ? 0.0f : hrow[jj];
                const float v = fmaf(p.beta, old, p.alpha * __uint_as_float(r[jj]));
                hrow[jj] = v;
                r[jj] = __float_as_uint(v);
              }
            }
          }
          if (mirror) {
            // H[j, i]: consecutive lanes hold consecutive i, so each store instruction is coalesced
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              if (j0 + jj < p.d2) p.H[(j0 + jj) * p.ldc + i] = __uint_as_float(r[jj]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
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

// ---------------------------------------------------------------------------------------------------------
// The 256 x 256 shape on CTA pairs (tcgen05 cta_group::2).  Each CTA of a cluster of two loads its 128 of the
// tile's 256 rows (of A^T) and its 128 of the 256 columns of B, so an SM pulls 32 KB per stage from L2 instead
// of the 64 KB the single-CTA form needs for the same eight MMAs' worth of work, the ring holds six stages
// instead of three, and tensor memory has room for two accumulators: the epilogue of a tile (a read-modify-
// write of H) overlaps the next tile's MMAs.  Barriers as in the FP4 pair GEMM: "full" lives in the leader
// and collects both producers' bytes, one multicast commit frees a stage in both CTAs, "accumulator full" is
// committed to both, "accumulator empty" lives in the leader and collects the epilogue warps of both.
struct PairShape {
  static constexpr int STAGES = 6;
  static constexpr int BOXES = 2;                                   // 64-wide boxes per operand and CTA
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * BOXES * BOX_BYTES;
  static constexpr int OFF_BAR = OFF_B + STAGES * BOXES * BOX_BYTES;  // full[S], empty[S], acc_full[2], acc_empty[2]
  static constexpr int OFF_MISC = OFF_BAR + (2 * STAGES + 4) * 8;
  static constexpr int TOTAL = OFF_MISC + 16;
  static constexpr int DYN_BYTES = TOTAL;                           // declared 1024-byte aligned
  static constexpr int STAGE_TX = 2 * BOXES * BOX_BYTES;            // bytes one CTA contributes to a stage
  static_assert(DYN_BYTES <= 227 * 1024, "stages exceed the shared memory of an SM");
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
hessian_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const HessParams p) {
  using L = PairShape;
  constexpr int STAGES = L::STAGES, BOXES = L::BOXES;
  extern __shared__ __align__(1024) uint8_t smem_pair[];
  uint8_t* smem = smem_pair;
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0) {                 // same in both CTAs: nobody waits for anybody
    if (threadIdx.x == 0) atomicExch(p.error_flag, 1);
    return;
  }
  const uint32_t bar_full = sbase + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_acc_full = bar_empty + STAGES * 8;   // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;       // [2]
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();               // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 2);        // both producers' announcements (used in the leader)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 8);   // four epilogue warps per CTA (used in the leader)
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                        // peer barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  launch_dependents();
  grid_dependency_wait();
  const uint32_t lead_full = map_to_cta(bar_full, 0);
  const uint32_t lead_acc_empty = map_to_cta(bar_acc_empty, 0);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs) {
        int ib, jb, lo, hi;
        tile_coords<true>(p, tile, ib, jb);
        stage_range(p, ib, jb, lo, hi);
        const int per_seg = hi - lo, n_st = per_seg * p.n_seg;
        const int xa = p.a_x0 + ib * 256 + (int)rank * 128, xb = p.b_x0 + jb * TILE_N + (int)rank * 128;
        for (int ks = 0; ks < n_st; ++ks, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_bounded(bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t full = lead_full + 8 * s;
          mbar_arrive_expect_tx_cluster(full, L::STAGE_TX);
          const uint32_t a_dst = sbase + L::OFF_A + s * BOXES * BOX_BYTES;
          const uint32_t b_dst = sbase + L::OFF_B + s * BOXES * BOX_BYTES;
          const int seg = ks / per_seg, kk = lo + (ks - seg * per_seg);
          const int ya = p.a_seg_y[seg] + kk * BK, yb = p.b_seg_y[seg] + kk * BK;
#pragma unroll
          for (int b = 0; b < BOXES; ++b) tma_load_2d_pair(a_dst + b * BOX_BYTES, &tmap_a, xa + 64 * b, ya, full);
#pragma unroll
          for (int b = 0; b < BOXES; ++b) tma_load_2d_pair(b_dst + b * BOX_BYTES, &tmap_b, xb + 64 * b, yb, full);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
      // Drain: a stage is freed (in both CTAs, by the issuing thread's commit) only after it was complete, so
      // waiting for my last min(it, STAGES) stages to be freed proves that every load of mine has landed.
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      volatile int never = 0;
      for (uint32_t j = first; j < it; ++j)
        (void)mbar_wait_bounded(bar_empty + 8 * (j % STAGES), (j / STAGES) & 1, &never, 400000000LL);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      const uint32_t peer_acc_full = map_to_cta(bar_acc_full, 1);
      const uint32_t idesc = make_idesc_bf16(256, TILE_N, true, true);
      uint32_t it = 0, tile_count = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs, ++tile_count) {
        const uint32_t buf = tile_count & 1, acc_parity = (tile_count >> 1) & 1;
        if (!mbar_wait_bounded_spin(bar_acc_empty + 8 * buf, acc_parity ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * TILE_N;
        int ib, jb, lo, hi;
        tile_coords<true>(p, tile, ib, jb);
        stage_range(p, ib, jb, lo, hi);
        const int n_st = (hi - lo) * p.n_seg;
        for (int ks = 0; ks < n_st; ++ks, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait_bounded_spin(bar_full + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = make_desc_mn_sw128(sbase + L::OFF_A + s * BOXES * BOX_BYTES, BOX_BYTES, 1024);
          const uint64_t b_desc = make_desc_mn_sw128(sbase + L::OFF_B + s * BOXES * BOX_BYTES, BOX_BYTES, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)   // 16 tokens per MMA = two 8-row atoms = 2048 bytes
            tc_mma_f16_pair(acc, a_desc + (uint64_t)(k * (2048 >> 4)), b_desc + (uint64_t)(k * (2048 >> 4)), idesc,
                            (ks > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair_multicast(bar_empty + 8 * s, 3);   // frees the stage in both CTAs
        }
        if (ok) {
          tc_commit_pair(bar_acc_full + 8 * buf);
          tc_commit_pair(peer_acc_full + 8 * buf);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs): H = beta H + alpha acc
    const int quarter = warp & 3;
    uint32_t tile_count = 0;
    bool ok = true;
    for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs, ++tile_count) {
      int ib, jb;
      tile_coords<true>(p, tile, ib, jb);
      const uint32_t buf = tile_count & 1, acc_parity = (tile_count >> 1) & 1;
      if (!mbar_wait_bounded(bar_acc_full + 8 * buf, acc_parity, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int rb = ib * 2 + (int)rank;                     // my 128-row block
      const int64_t i = (int64_t)rb * TILE + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < TILE_N / 32; ++c) {
        const int64_t j0 = (int64_t)jb * TILE_N + c * 32;
        const int jblock = (int)(j0 / TILE);
        if (j0 >= p.d2 || (p.symmetric && jblock > rb)) continue;   // beyond the matrix / above the diagonal
        const bool mirror = p.mirror && jblock < rb;
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TILE_N + c * 32, r);
        tc_wait_ld();
        if (i < p.d1) {
          float* hrow = p.H + i * p.ldc + j0;
          if (j0 + 32 <= p.d2 && (p.ldc & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 h = p.beta == 0.0f ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(hrow)[q];
              h.x = fmaf(p.beta, h.x, p.alpha * __uint_as_float(r[4 * q]));
              h.y = fmaf(p.beta, h.y, p.alpha * __uint_as_float(r[4 * q + 1]));
              h.z = fmaf(p.beta, h.z, p.alpha * __uint_as_float(r[4 * q + 2]));
              h.w = fmaf(p.beta, h.w, p.alpha * __uint_as_float(r[4 * q + 3]));
              reinterpret_cast<float4*>(hrow)[q] = h;
              r[4 * q] = __float_as_uint(h.x); r[4 * q + 1] = __float_as_uint(h.y);
              r[4 * q + 2] = __float_as_uint(h.z); r[4 * q + 3] = __float_as_uint(h.w);
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              if (j0 + jj < p.d2) {
                const float old = p.beta == 0.0f ? 0.0f : hrow[jj];
                const float v = fmaf(p.beta, old, p.alpha * __uint_as_float(r[jj]));
                hrow[jj] = v;
                r[jj] = __float_as_uint(v);
              }
            }
          }
          if (mirror) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              if (j0 + jj < p.d2) p.H[(j0 + jj) * p.ldc + i] = __uint_as_float(r[jj]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_acc_empty + 8 * buf);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicExch(p.error_flag, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // neither CTA leaves while its peer may still signal its barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace
}  // namespace fpq

namespace fpq {

// out[d1, d2] (row stride ldc) = beta * out + alpha * A^T B with A [*, d1] and B [*, d2] bf16 row-major
// matrices of a_rows / b_rows rows (row strides lda, ldb in elements; the operands start at columns
// a_x0 / b_x0).  The K dimension is the concatenation of n_seg segments of seg_rows rows each, segment
// i starting at row a_seg_y[i] of A and b_seg_y[i] of B (one segment from row 0: the plain product).
// With more than one segment seg_rows must be a multiple of 64.  symmetric: only tiles that touch the
// lower triangle are computed (d1 == d2); mirror: the blocks below the diagonal are also written
// transposed.  tri = 1: B (as the [K, d2] matrix of one segment) is lower triangular, tri = 2: A^T (the
// [d1, K] matrix) is lower triangular -- the stages that only multiply zeros are skipped.
int gemm_atb_bf16(float* out, int64_t ldc, int64_t d1, int64_t d2, const void* A, int64_t lda, int64_t a_rows,
                  int64_t a_x0, const void* B, int64_t ldb, int64_t b_rows, int64_t b_x0, bool symmetric, bool mirror,
                  int n_seg, int64_t seg_rows, const int* a_seg_y, const int* b_seg_y, float alpha, float beta,
                  int32_t* error_flag, cudaStream_t stream, int tri) {
  if (n_seg < 1 || n_seg > MAX_SEGMENTS || (n_seg > 1 && seg_rows % BK != 0)) {
    set_error("bad K segmentation (%d segments of %lld rows)", n_seg, (long long)seg_rows);
    return FPQ_ERR_INVALID_ARGUMENT;
  }
  if (d1 <= 0 || d2 <= 0 || seg_rows <= 0) return FPQ_OK;
  HessParams p{};
  p.d1 = d1; p.d2 = d2; p.ldc = ldc;
  // no triangular skipping, enough 256-row tiles to fill the GPU: the 256 x 256 shape on CTA pairs (measured
  // with the threshold at 64, 24 and 8 stages of K: the d = 14336 Cholesky-inverse chain 25.7, 25.0, 24.9 ms)
  const int64_t total_stages = (int64_t)n_seg * ((seg_rows + BK - 1) / BK);
  const int64_t rows256 = (d1 + 255) / 256, cols256 = (d2 + TILE_N - 1) / TILE_N;
  const int64_t big_tiles = symmetric ? rows256 * (rows256 + 1) / 2 : rows256 * cols256;
  const bool big = tri == 0 && total_stages >= 8 && big_tiles >= sm_count() / 2 && sm_count() >= 2;
  const int tm = big ? 256 : TILE;
  p.num_blocks = (int)((d1 + tm - 1) / tm);
  p.num_blocks_n = (int)((d2 + TILE_N - 1) / TILE_N);
  p.num_tiles = symmetric ? tiles_before_row(p.num_blocks, big) : p.num_blocks * p.num_blocks_n;
  p.symmetric = symmetric ? 1 : 0;
  p.mirror = (symmetric && mirror) ? 1 : 0;
  p.a_x0 = (int)a_x0; p.b_x0 = (int)b_x0;
  p.seg_stages = (int)((seg_rows + BK - 1) / BK);
  p.n_seg = n_seg;
  p.tri = tri;
  for (int i = 0; i < n_seg; ++i) {
    p.a_seg_y[i] = a_seg_y ? a_seg_y[i] : 0;
    p.b_seg_y[i] = b_seg_y ? b_seg_y[i] : 0;
  }
  p.alpha = alpha; p.beta = beta; p.H = out; p.error_flag = error_flag;
  CUtensorMap ta, tb;
  if (int rc = make_tensor_map_2d(&ta, A, 2, (uint64_t)lda, (uint64_t)a_rows, (uint64_t)lda * 2, 64, BK, 1)) return rc;
  if (int rc = make_tensor_map_2d(&tb, B, 2, (uint64_t)ldb, (uint64_t)b_rows, (uint64_t)ldb * 2, 64, BK, 1)) return rc;
  static bool configured[64] = {};
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(hessian_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Shape<false>::DYN_BYTES));
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(hessian_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        PairShape::DYN_BYTES));
    configured[dev] = true;
  }
  if (big) {
    // the 256 x 256 shape on CTA pairs
    int pairs = sm_count() / 2;
    if (pairs > p.num_tiles) pairs = p.num_tiles;
    if (pairs < 1) return FPQ_OK;
    cudaLaunchConfig_t pc = {};
    pc.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    pc.blockDim = dim3(NUM_THREADS, 1, 1);
    pc.dynamicSmemBytes = PairShape::DYN_BYTES;
    pc.stream = stream;
    cudaLaunchAttribute pa[2];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2;
    pa[0].val.clusterDim.y = 1;
    pa[0].val.clusterDim.z = 1;
    pa[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pa[1].val.programmaticStreamSerializationAllowed = 1;
    pc.attrs = pa;
    pc.numAttrs = use_dependent_launch() ? 2 : 1;
    FPQ_CHECK_CUDA(cudaLaunchKernelEx(&pc, hessian_pair_kernel, ta, tb, p));
    return FPQ_OK;
  }
  int grid = sm_count();
  if (grid > p.num_tiles) grid = p.num_tiles;
  if (grid < 1) return FPQ_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Shape<false>::DYN_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_dependent_launch() ? 1 : 0;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, hessian_kernel<false>, ta, tb, p));
  return FPQ_OK;
}

}  // namespace fpq

using namespace fpq;

extern "C" int fpq_hessian_accumulate(float* H, int64_t d, const void* xa_bf16, const void* xb_bf16, int64_t tokens,
                                      float alpha, float beta, int32_t* error_flag, fpq_stream_t stream) {
  FPQ_CHECK_ARG(H && xa_bf16 && error_flag, "NULL pointer");
  FPQ_CHECK_ARG(d > 0 && tokens >= 0 && d % 8 == 0, "d (%lld) must be a positive multiple of 8", (long long)d);
  FPQ_CHECK_ARG(d < (1ll << 30) && tokens < (1ll << 31), "shape too large");
  FPQ_CHECK_ARG(((uintptr_t)xa_bf16 & 15) == 0 && ((uintptr_t)xb_bf16 & 15) == 0 && ((uintptr_t)H & 15) == 0,
                "pointers must be 16-byte aligned");
  if (tokens == 0) return FPQ_OK;
  const bool symmetric = xb_bf16 == nullptr || xb_bf16 == xa_bf16;
  // The tensor core truncates when it adds into its fp32 accumulator: measured on B200, every 1024 tokens
  // of one accumulation chain lower a (positive) diagonal entry by 2e-6 of its value, 1.4e-4 after 32768
  // tokens.  The tokens are therefore taken 4096 at a time, each slab's product added to H with a correctly
  // rounded fp32 addition in the epilogue: 4.5e-6 relative Frobenius error for any number of tokens.  Only
  // the last slab writes the mirrored upper triangle.
  constexpr int64_t SLAB = 4096;
  const __nv_bfloat16* xa = reinterpret_cast<const __nv_bfloat16*>(xa_bf16);
  const __nv_bfloat16* xb = symmetric ? xa : reinterpret_cast<const __nv_bfloat16*>(xb_bf16);
  for (int64_t t0 = 0; t0 < tokens; t0 += SLAB) {
    const int64_t n = tokens - t0 < SLAB ? tokens - t0 : SLAB;
    const bool last = t0 + n >= tokens;
    if (int rc = gemm_atb_bf16(H, d, d, d, xa + t0 * d, d, n, 0, xb + t0 * d, d, n, 0, symmetric, last, 1, n, nullptr,
                               nullptr, alpha, t0 == 0 ? beta : 1.0f, error_flag, (cudaStream_t)stream, 0))
      return rc;
  }
  return FPQ_OK;
}
