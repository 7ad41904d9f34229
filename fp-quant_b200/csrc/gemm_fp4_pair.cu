// Block-scaled FP4 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a -- the large-M path of
// fpq_gemm_fp4 (see gemm_fp4.cu for the interface it serves).
//
// A pair of CTAs (cluster of 2, two neighbouring SMs) owns a 256 x 256 output tile.  Each CTA loads
// its own 128 rows of A and its own 128 of the 256 rows of B, so every byte of the operands is fetched
// from L2 once per pair; one thread of the leader CTA issues MMAs that span both SMs (M = 256), each
// SM accumulating its 128 x 256 half in its own tensor memory.
//
// Warps per CTA (22): 0 TMA producer, 1 MMA issuer (leader CTA only) and tensor-memory owner, 2-5
// scale-factor movers, 6-21 epilogue (one per 32 rows x 64 columns of the CTA's half tile).  Scale tiles
// go shared -> registers -> tensor memory (tcgen05.st, each of the four mover warps filling its own
// 32-lane quarter) so that the MMA queue carries nothing but MMAs.  The epilogue first drains the whole
// accumulator into registers in one round of loads, hands it back, and only then converts and writes
// to global memory, so conversion and stores overlap the next tile's MMAs.
//
// Barriers: the "full" barrier of a stage lives in the leader and collects everything the MMAs of that
// stage need: the operand bytes of both CTAs (both producers announce theirs on it) and one arrival
// per scale-mover warp of both CTAs once the stage's scales sit in tensor memory.  Scale tiles land on
// a per-CTA "sf_full" barrier that only the movers watch.  The issuing thread's loop is one wait, four
// MMAs and one commit per stage; the commit frees the stage in both CTAs at once (tcgen05.commit with
// a CTA mask: a signal, no data).  "accumulator full" exists in both CTAs (one commit each per tile),
// "accumulator empty" lives in the leader and collects the epilogue warps of both CTAs.  Every wait is
// bounded.  No load is broadcast between the CTAs.
//
// What limits it (measured on B200 with timing-only variants of this kernel, 8192 x 4096 x K): MMAs alone,
// without operand traffic, take 0.28 us per stage of four; the full loop 0.39 us; with half-width MMAs
// (N = 128) still 0.33 us.  The three fit one model: per stage a CTA's shared memory takes 35 KB of TMA
// writes and gives 48 KB of operand reads (A, its half of B for itself and again for the peer), 83 KB at
// 128 bytes per cycle.  cuBLASLt's kernel for the same problem (a CUTLASS 256 x 256 x 64 block-scaled
// 2-SM kernel, by its name in the profiler) runs within 2 % of this one.

#include "common.cuh"
#include "sm100_ptx.cuh"

#include <atomic>

namespace fpq {
namespace {

using namespace ptx;

constexpr int BM_CTA = 128;            // rows of A per CTA
constexpr int BN = 256;                // columns of the pair tile
constexpr int BN_CTA = 128;            // rows of B per CTA
constexpr int BK_BYTES = 128;           // operand bytes per row and stage: 256 four-bit or 128 eight-bit elements
constexpr int KIND_MXFP4 = 0, KIND_NVFP4 = 1, KIND_MXFP8 = 2;
constexpr int NUM_THREADS = 704;       // 22 warps: producer, MMA, 4 scale movers, 16 epilogue (one per 32 rows x 64 columns)
constexpr int TMEM_COLS = 512;
constexpr int SF_TMEM_BASE = 256;




struct PairParams {
  int M, N, K;
  int num_m_pairs, num_n_blocks, num_tiles;
  int num_k_stages;
  int sf_blocks_k;
  const float* alpha;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int* error_flag;
  int raster_group;
  int stagger_step;        // cycles between the time slots in which the epilogue warps convert and store (see the epilogue)
};

// Tensor-parallel push: the tile also goes to the same place of up to seven other GPUs' output buffers
// (P2P-mapped pointers, already offset to this rank's first column), row stride ld elements.
struct PushParams {
  __nv_bfloat16* out[7];
  int n;
  long long ld;
};

// Operand ring and epilogue staging.  What bounds the main loop is how many operand bytes are in flight
// between L2 and shared memory: a stage is refilled ~1.5 us after it was consumed, the tensor pipe consumes
// one (32 KiB of operands per CTA) every ~0.28 us, so four stages (measured: 0.405 us per stage) starve it and
// six do not.  Shared memory is therefore spent on stages, and the sixteen epilogue warps share a few
// staging boxes in turn (a barrier per box) instead of owning one each.
template <int KIND>
struct PairSmem {
  static constexpr bool NVFP4 = KIND == KIND_NVFP4;
  static constexpr int BK_ELEMS = KIND == KIND_MXFP8 ? 128 : 256;   // K elements per stage
  static constexpr int MMA_K = KIND == KIND_MXFP8 ? 32 : 64;        // K elements per instruction (32 bytes)
  static constexpr int STAGES = NVFP4 ? 5 : 6;                // NVFP4: 5 x 48 tensor-memory columns of scales is all that fits
  static constexpr int NBOX = NVFP4 ? 8 : 4;                  // 32-row x 128-byte staging boxes of the epilogue
  static constexpr int SFBLK = NVFP4 ? 4 : KIND == KIND_MXFP8 ? 1 : 2;   // 512-byte scale tiles per 128 rows per stage
  static constexpr int SFA_COLS = 4 * SFBLK;                  // tensor-memory columns of one stage's A scales
  static constexpr int SF_TMEM_BUF = 12 * SFBLK;              // A scales + B scales (256 rows) of one stage
  static constexpr int A_BYTES = BM_CTA * BK_BYTES;           // 16 KiB
  static constexpr int B_BYTES = BN_CTA * BK_BYTES;           // 16 KiB
  static constexpr int SFA_BYTES = SFBLK * 512;
  static constexpr int SFB_BYTES = 2 * SFBLK * 512;           // scales of all 256 B rows
  static constexpr int STAGE_TX = A_BYTES + B_BYTES;           // operand bytes per CTA (leader's barrier)
  static constexpr int SF_TX = SFA_BYTES + SFB_BYTES;          // scale bytes per CTA (own barrier)
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_SFA = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_SFB = OFF_SFA + STAGES * SFA_BYTES;
  static constexpr int OFF_OUT = OFF_SFB + STAGES * SFB_BYTES;
  static constexpr int OUT_BOX_BYTES = 32 * 128;
  // full[S], empty[S], sf_full[S], acc_full, acc_empty, box_read[16]
  static constexpr int OFF_BAR = OFF_OUT + NBOX * OUT_BOX_BYTES;
  static constexpr int OFF_MISC = OFF_BAR + (3 * STAGES + 2 + 16) * 8;
  static constexpr int TOTAL = OFF_MISC + 16;
  static constexpr int DYN_BYTES = TOTAL;                      // the dynamic shared memory is declared 1024-byte aligned
  static_assert(DYN_BYTES <= 227 * 1024, "stages and staging boxes exceed the shared memory of an SM");
  static_assert(SF_TMEM_BASE + STAGES * SF_TMEM_BUF <= TMEM_COLS, "scale buffers exceed tensor memory");
};

__device__ __forceinline__ void pair_tile_coords(const PairParams& p, int tile, int& m_pair, int& n_blk) {
  const int band_tiles = p.raster_group * p.num_n_blocks;
  const int band = tile / band_tiles;
  const int first_m = band * p.raster_group;
  int rows = p.num_m_pairs - first_m;
  if (rows > p.raster_group) rows = p.raster_group;
  const int in_band = tile - band * band_tiles;
  m_pair = first_m + in_band % rows;
  n_blk = in_band / rows;
}

template <int KIND, bool PUSH>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp4_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                     const __grid_constant__ CUtensorMap tmap_out, const PairParams p, const PushParams push) {
  using L = PairSmem<KIND>;
  constexpr bool NVFP4 = L::NVFP4;
  constexpr int STAGES = L::STAGES;
  constexpr int SFBLK = L::SFBLK;
  constexpr int BK_ELEMS = L::BK_ELEMS;
  extern __shared__ __align__(1024) uint8_t smem_raw[];      // 128-byte-swizzled TMA boxes need 1024-byte alignment
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0) {                                 // same in both CTAs of the pair: nobody waits for anybody
    if (threadIdx.x == 0) atomicExch(p.error_flag, 1);
    return;
  }
  const uint32_t bar_full = sbase + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_sf_full = bar_empty + STAGES * 8;
  const uint32_t bar_acc_full = bar_sf_full + STAGES * 8;
  const uint32_t bar_acc_empty = bar_acc_full + 8;
  const uint32_t bar_box = bar_acc_empty + 8;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

  // The warp index goes through a shuffle so that the compiler knows it is the same in all lanes, and the
  // single-thread roles are chosen with elect.sync: both keep the role code on the uniform datapath, where
  // the descriptors and addresses of the tcgen05 / TMA instructions have to live anyway.  With
  // `threadIdx.x >> 5` and `lane == 0` every tcgen05.mma cost its issuing thread 75-150 cycles (operands
  // moved from vector to uniform registers one by one) and the loop ran at 755 cycles per stage of four
  // MMAs; like this it runs at the rate shared memory sustains (see PairSmem).
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 2 + 8);  // both producers' announcements + four mover warps per CTA (leader)
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_sf_full + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 32);          // sixteen epilogue warps per CTA (used in the leader)
    for (int b = 0; b < 16; ++b) mbar_init(bar_box + 8 * b, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_sfa);
    prefetch_tensormap(&tmap_sfb);
    prefetch_tensormap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                       // peer barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // Everything above (barriers, tensor memory, descriptor prefetch) touched nothing another kernel wrote and
  // may overlap the tail of the previous kernel; from here on operands and outputs are accessed.
  launch_dependents();
  grid_dependency_wait();

  // addresses of the leader's barriers as seen from this CTA
  const uint32_t lead_full = map_to_cta(bar_full, 0);
  const uint32_t lead_acc_empty = map_to_cta(bar_acc_empty, 0);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs) {
        int m_pair, n_blk;
        pair_tile_coords(p, tile, m_pair, n_blk);
        const int m_row = m_pair * 256 + (int)rank * BM_CTA;            // my rows of A
        const int n_row = n_blk * BN + (int)rank * BN_CTA;              // my rows of B
        for (int ks = 0; ks < p.num_k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_bounded(bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t full = lead_full + 8 * s;
          // scale tiles first (the movers need them earliest): 64 eight-byte words per 512-byte tile,
          // rows of the map are 128-row blocks; they complete on this CTA's own barrier
          mbar_arrive_expect_tx(bar_sf_full + 8 * s, L::SF_TX);
          tma_load_2d(sbase + L::OFF_SFA + s * L::SFA_BYTES, &tmap_sfa, ks * SFBLK * 64, m_pair * 2 + (int)rank,
                      bar_sf_full + 8 * s);
          tma_load_2d(sbase + L::OFF_SFB + s * L::SFB_BYTES, &tmap_sfb, ks * SFBLK * 64, n_blk * 2, bar_sf_full + 8 * s);
          mbar_arrive_expect_tx_cluster(full, L::STAGE_TX);
          tma_load_2d_pair(sbase + L::OFF_A + s * L::A_BYTES, &tmap_a, ks * BK_BYTES, m_row, full);
          tma_load_2d_pair(sbase + L::OFF_B + s * L::B_BYTES, &tmap_b, ks * BK_BYTES, n_row, full);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
      // Drain: my loads complete on the leader's barrier, which I cannot poll from the follower; a stage
      // is freed (in both CTAs, by the MMA thread's commit) only after it was complete, so waiting for my
      // last min(it, STAGES) stages to be freed proves that every load has landed.
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      volatile int never = 0;
      for (uint32_t j = first; j < it; ++j) {
        (void)mbar_wait_bounded(bar_empty + 8 * (j % STAGES), (j / STAGES) & 1, &never, 400000000LL);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      const uint32_t peer_acc_full = map_to_cta(bar_acc_full, 1);
      uint32_t idesc_k[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // which of a column's four scale bytes instruction k reads: NVFP4 all four, MXFP4 a pair, MXFP8 one
        const uint32_t sf_id = NVFP4 ? 0u : KIND == KIND_MXFP8 ? (uint32_t)k : (uint32_t)((k & 1) * 2);
        idesc_k[k] = KIND == KIND_MXFP8 ? make_idesc_mxf8(256, BN, sf_id, sf_id) : make_idesc_fp4(256, BN, !NVFP4, sf_id, sf_id);
      }
      uint32_t it = 0, tile_count = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs, ++tile_count) {
        if (!mbar_wait_bounded_spin(bar_acc_empty, (tile_count & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // per stage: one barrier wait, four MMAs, one commit; everything else is uniform address arithmetic
        for (int ks = 0; ks < p.num_k_stages; ++ks, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait_bounded_spin(bar_full + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sf_buf = tmem_base + SF_TMEM_BASE + s * L::SF_TMEM_BUF;
          const uint32_t sfa_t = sf_buf, sfb_t = sf_buf + L::SFA_COLS;
          const uint64_t a_desc = make_desc_k_sw128(sbase + L::OFF_A + s * L::A_BYTES);
          const uint64_t b_desc = make_desc_k_sw128(sbase + L::OFF_B + s * L::B_BYTES);
          const int k_left = p.K - ks * BK_ELEMS;
          if (k_left >= BK_ELEMS) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t blk = NVFP4 ? (uint32_t)k : KIND == KIND_MXFP8 ? 0u : (uint32_t)(k >> 1);
              tc_mma_fp4_block_scaled_pair<KIND>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc_k[k], sfa_t + 4 * blk,
                                                 sfb_t + 8 * blk, (ks > 0 || k > 0) ? 1u : 0u);
            }
          } else {
            const int kmma = (k_left + L::MMA_K - 1) / L::MMA_K;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (k < kmma) {
                const uint32_t blk = NVFP4 ? (uint32_t)k : KIND == KIND_MXFP8 ? 0u : (uint32_t)(k >> 1);
                tc_mma_fp4_block_scaled_pair<KIND>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc_k[k], sfa_t + 4 * blk,
                                                   sfb_t + 8 * blk, (ks > 0 || k > 0) ? 1u : 0u);
              }
            }
          }
          tc_commit_pair_multicast(bar_empty + 8 * s, 3);   // frees the stage in both CTAs
        }
        if (ok) {
          tc_commit_pair(bar_acc_full);
          tc_commit_pair(peer_acc_full);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 1);
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------- scale-factor movers (both CTAs)
    // A 512-byte tile is 32 rows x 16 bytes: lane l takes row l and writes it to lane l of this warp's
    // quarter of tensor memory, columns [c, c+4) -- the four warps together produce the replicated
    // layout the block-scaled MMA reads.  One tensor-memory buffer per stage: the scales of a stage can
    // only have landed (sf_full) after the producer saw the stage freed, i.e. after the MMAs that read
    // the buffer's previous contents completed.
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // Stages form one flat sequence over this pair's tiles.
    const int my_tiles = pair_id < p.num_tiles ? (p.num_tiles - pair_id + num_pairs - 1) / num_pairs : 0;
    const uint32_t n_it = (uint32_t)my_tiles * (uint32_t)p.num_k_stages;
    bool ok = true;
    for (uint32_t it = 0; it < n_it && ok; ++it) {
      const int s = it % STAGES;
      if (!mbar_wait_bounded(bar_sf_full + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t sf_buf = tmem_base + SF_TMEM_BASE + s * L::SF_TMEM_BUF + lane_base;
      const uint8_t* sfa_s = smem + L::OFF_SFA + s * L::SFA_BYTES + lane * 16;
      const uint8_t* sfb_s = smem + L::OFF_SFB + s * L::SFB_BYTES + lane * 16;
#pragma unroll
      for (int j = 0; j < SFBLK; ++j) {
        const uint4 a = *reinterpret_cast<const uint4*>(sfa_s + j * 512);
        tc_st_32x32b_x4(sf_buf + 4 * j, a.x, a.y, a.z, a.w);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 b = *reinterpret_cast<const uint4*>(sfb_s + (h * SFBLK + j) * 512);
          tc_st_32x32b_x4(sf_buf + L::SFA_COLS + 8 * j + 4 * h, b.x, b.y, b.z, b.w);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_full + 8 * s);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicExch(p.error_flag, 1);
    }
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;                // the 32 lanes of tensor memory this warp may read
    const int col_q = (warp - 6) >> 2;           // which 64 of the tile's 256 columns
    const float alpha = *p.alpha;
    uint32_t tile_count = 0;
    bool ok = true;
    for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs, ++tile_count) {
      int m_pair, n_blk;
      pair_tile_coords(p, tile, m_pair, n_blk);
      if (!mbar_wait_bounded(bar_acc_full, tile_count & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      // 1) drain this warp's 64 fp32 columns in one round (two 32-column loads in flight): with sixteen
      //    warps the whole accumulator is in registers after a single load latency
      const int row0 = m_pair * 256 + (int)rank * BM_CTA + quarter * 32;
      const int col_w = n_blk * BN + col_q * 64;               // first of my 64 columns
      const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) + col_q * 64;
      uint32_t ra[32], rb[32];
      tc_ld_32x32b_x32(tsrc, ra);
      tc_ld_32x32b_x32(tsrc + 32, rb);
      tc_wait_ld();
      // 2) hand the accumulator back: the next tile's MMAs may start while we convert and write out
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
      // 3) wait for this warp's slot.  All sixteen warps converting and storing at once costs the next
      //    tile about 1400 cycles: the four warps that share the MMA thread's scheduler take its issue
      //    slots just when the tensor pipe is empty, and sixteen 4 KiB TMA stores in one burst hold up the
      //    operand loads behind them.  Spread over the next tile's main loop both disappear in its slack.
      if (tile + num_pairs < p.num_tiles) {          // not after the last tile: there is nothing left to protect
        const long long due = clock64() + (long long)(col_q * 4 + quarter) * p.stagger_step;
        while (clock64() < due) __nanosleep(64);
      }
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const uint32_t* rr = j < 16 ? ra : rb;
        float v0 = __uint_as_float(rr[(2 * j) & 31]) * alpha;
        float v1 = __uint_as_float(rr[(2 * j + 1) & 31]) * alpha;
        if (p.bias) {
          const int col = col_w + 2 * j;
          if (col < p.N) {
            v0 += __bfloat162float(p.bias[col]);
            v1 += __bfloat162float(p.bias[col + 1]);
          }
        }
        __nv_bfloat162 hh = __floats2bfloat162_rn(v0, v1);
        pk[j] = *reinterpret_cast<uint32_t*>(&hh);
      }
      // 4) write out through shared memory: a 32-row x 128-byte staging box (128-byte swizzle, so the
      //    16-byte row pieces of the 32 lanes spread over all banks) sent with one TMA store, which clips
      //    rows >= M and columns >= N.
      //    The boxes are shared: slot i uses box i % NBOX after slot i - NBOX (the last user of the previous
      //    tile for the first NBOX slots).  Every slot has a barrier of its own on which it announces that
      //    its store has read the box, once per tile, and the next user of the box waits for exactly that
      //    phase (one arriving and one waiting warp per barrier, never more than a phase apart).
      const int slot = col_q * 4 + quarter;
      const uint32_t box_off = (uint32_t)(L::OFF_OUT + (slot % L::NBOX) * L::OUT_BOX_BYTES);
      const uint32_t stage_out = sbase + box_off;
      if (slot >= L::NBOX) {
        if (!mbar_wait_bounded(bar_box + 8 * (slot - L::NBOX), tile_count & 1, abort_flag)) { ok = false; break; }
      } else if (tile_count > 0) {
        if (!mbar_wait_bounded(bar_box + 8 * (slot + 16 - L::NBOX), (tile_count - 1) & 1, abort_flag)) { ok = false; break; }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        st_shared_v4(stage_out + (uint32_t)lane * 128u + (uint32_t)((q ^ (lane & 7)) * 16), pk[4 * q], pk[4 * q + 1],
                     pk[4 * q + 2], pk[4 * q + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0 && row0 < p.M && col_w < p.N) {
        tma_store_2d(&tmap_out, stage_out, col_w, row0);
        bulk_commit_group();
      }
      if (PUSH && push.n > 0) {
        // Same box to the peers with ordinary 16-byte stores over NVLink: eight lanes cover the 128 bytes
        // of one row, so every instruction writes four full lines (the box is read back un-swizzled).
        const int rsub = lane >> 3, chunk = lane & 7;
        const int col = col_w + chunk * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rsub + 4 * i;
          const uint4 v = *reinterpret_cast<const uint4*>(smem + box_off + r * 128 + ((chunk ^ (r & 7)) * 16));
          if (row0 + r < p.M && col < p.N) {
#pragma unroll
            for (int pr = 0; pr < 7; ++pr)
              if (pr < push.n) *reinterpret_cast<uint4*>(push.out[pr] + (long long)(row0 + r) * push.ld + col) = v;
          }
        }
        __syncwarp();
      }
      if (lane == 0) {
        bulk_wait_group_read0();                   // the store has read the box: the next user may overwrite it
        mbar_arrive(bar_box + 8 * slot);
      }
    }
    if (lane == 0) bulk_wait_group0();   // my stores are complete before the CTA may exit
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

template <int KIND>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                const CUtensorMap& tout, PairParams p, const PushParams& push, cudaStream_t stream) {
  using L = PairSmem<KIND>;
  auto kern = push.n > 0 ? gemm_fp4_pair_kernel<KIND, true> : gemm_fp4_pair_kernel<KIND, false>;
  // one-time per device (idempotent: concurrent first calls set the same attribute)
  static std::atomic<bool> configured[64];
  int dev = 0;
  FPQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(gemm_fp4_pair_kernel<KIND, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    FPQ_CHECK_CUDA(cudaFuncSetAttribute(gemm_fp4_pair_kernel<KIND, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    configured[dev].store(true, std::memory_order_release);
  }
  int pairs = sm_count() / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L::DYN_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_dependent_launch() ? 2 : 1;
  FPQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, tout, p, push));
  return FPQ_OK;
}

}  // namespace

int make_tensor_map_2d_u64(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer);

// Large-M path of fpq_gemm_fp4, and the whole of fpq_gemm_mxf8 (format FPQ_FMT_MXFP8: one byte per element).
// Shapes and pointers were validated by the caller.
int gemm_fp4_pair(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                  const void* bias, void* out, int64_t M, int64_t N, int64_t K, int format, int32_t* error_flag,
                  cudaStream_t stream, int64_t ldc, void* const* peers, int n_peers) {
  if (ldc <= 0) ldc = N;
  const bool fp8 = format == FPQ_FMT_MXFP8;
  const int g = format == FPQ_FMT_NVFP4 ? 16 : 32;
  const int sfblk = format == FPQ_FMT_NVFP4 ? 4 : fp8 ? 1 : 2;
  const int BK_ELEMS = fp8 ? 128 : 256;
  const uint64_t row_bytes = fp8 ? (uint64_t)K : (uint64_t)K / 2;
  PairParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.num_m_pairs = (int)((M + 255) / 256);
  p.num_n_blocks = (int)((N + BN - 1) / BN);
  p.num_tiles = p.num_m_pairs * p.num_n_blocks;
  p.num_k_stages = (int)((K + BK_ELEMS - 1) / BK_ELEMS);
  p.sf_blocks_k = (int)((K / g + 3) / 4);
  p.alpha = alpha;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.error_flag = error_flag;
  PushParams push{};
  push.n = n_peers;
  push.ld = ldc;
  for (int i = 0; i < n_peers && i < 7; ++i) push.out[i] = reinterpret_cast<__nv_bfloat16*>(peers[i]);
  // Time slots of the sixteen epilogue warps: together at most 60 % of a tile's main loop (~740 cycles per
  // K stage), and never more than 300 cycles apart (larger steps delay the next tile's drain).
  p.stagger_step = (int)(p.num_k_stages * 740 * 6 / 10 / 16);
  if (p.stagger_step > 300) p.stagger_step = 300;
  p.raster_group = 8;
  CUtensorMap ta, tb, tsa, tsb, tout;
  // output as 64-column x 32-row boxes of bf16 (128 bytes per box row, 128-byte swizzle)
  if (int rc = make_tensor_map_2d(&tout, out, 2, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 32, 1)) return rc;
  if (int rc = make_tensor_map_2d(&ta, a, 1, row_bytes, (uint64_t)M, row_bytes, BK_BYTES, BM_CTA, 1)) return rc;
  if (int rc = make_tensor_map_2d(&tb, b, 1, row_bytes, (uint64_t)N, row_bytes, BK_BYTES, BN_CTA, 1)) return rc;
  const uint64_t sf_row_words = (uint64_t)p.sf_blocks_k * 64;      // 8-byte words per 128-row block
  const uint64_t a_blocks = (uint64_t)((M + 127) / 128), b_blocks = (uint64_t)((N + 127) / 128);
  if (int rc = make_tensor_map_2d_u64(&tsa, sfa, sf_row_words, a_blocks, sf_row_words * 8, (uint32_t)sfblk * 64, 1)) return rc;
  if (int rc = make_tensor_map_2d_u64(&tsb, sfb, sf_row_words, b_blocks, sf_row_words * 8, (uint32_t)sfblk * 64, 2)) return rc;
  if (fp8) return launch_pair<KIND_MXFP8>(ta, tb, tsa, tsb, tout, p, push, stream);
  return format == FPQ_FMT_NVFP4 ? launch_pair<KIND_NVFP4>(ta, tb, tsa, tsb, tout, p, push, stream)
                                 : launch_pair<KIND_MXFP4>(ta, tb, tsa, tsb, tout, p, push, stream);
}

}  // namespace fpq
