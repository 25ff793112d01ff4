// Block-scaled grouped GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster
// compute one 256 x 256 output tile.  Each CTA loads its own 128 rows of A, its own 128 of
// the tile's 256 B rows, the scales of its A rows and the scales of all 256 B rows, and keeps
// its 128 x 256 fp32 accumulator in its own TMEM; the even CTA issues every tcgen05
// instruction for both.  Sharing B between two SMs cuts the L2->SM operand stream per MMA
// by 30 % against a 128 x 256 single-CTA tile, which is what bounds that kernel.
//
// A tile whose group ends inside it (the last tile of a ragged group, a masked batch) loads only
// the A rows that exist, in 32-row boxes, and none at all for a CTA whose 128 rows lie wholly
// beyond the group's end: the ring is bound by the bytes that reach shared memory, so a short
// tile then runs at the tensor pipe's pace instead of the loads'.  The rows not loaded keep
// whatever the stage held before; they only ever reach accumulator rows that are not stored.
//
// No load here is multicast: every CTA fetches its own boxes.  The only cluster-wide
// signalling is tcgen05.commit arriving on both CTAs' barriers and plain remote
// mbarrier arrives.
//
// Barriers.  full[s] lives in the leader: its producer arrives once with the byte count of
// BOTH CTAs' loads, every load (cta_group::2 form) credits the leader's barrier.  empty[s]
// and acc_full are per CTA and are signalled in both by one commit.  acc_empty lives in
// the leader and collects the arrives of both CTAs' epilogue warps.
//
// Same arithmetic, operand layout and masking rules as gemm_blockscaled.cu.
#include "gemm_common.cuh"
#include "quantize_common.cuh"

namespace msc {

template <int STAGES, bool SFW = false, bool SCATTER = false>
struct PairSmem {
  static constexpr int kHeader = 1024;
  static constexpr int kA = 128 * 128;
  static constexpr int kB = 128 * 128;       // this CTA's half of the 256 B rows
  static constexpr int kSfa = 4 * 512;
  static constexpr int kSfb = 2 * 4 * 512;   // scales of all 256 B rows
  static constexpr int kOffA = kHeader;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffSfa = kOffB + STAGES * kB;
  static constexpr int kOffSfb = kOffSfa + STAGES * kSfa;
  static constexpr int kOffC = kOffSfb + STAGES * kSfb;
  static constexpr int kEpiWarps = 8;
  static constexpr int kSfWarps = SFW ? 4 : 0;   // warps that write scale factors into TMEM
  static constexpr int kThreads = (kEpiWarps + 2 + kSfWarps) * 32;
  // two 4 KB store boxes per epilogue warp when the ring leaves room (up to 4 stages), so the
  // second 64-column half never waits for the first half's store to drain
  // the row-scatter epilogue stages 32 linear rows of 256 B at a 272-byte pitch (conflict-free
  // 16-byte stores: bank = 4 (row + chunk) mod 32)
  static constexpr int kScatterPitch = 272;
  static constexpr int kCPerWarp = SCATTER ? 32 * kScatterPitch : (STAGES <= 4) ? 8192 : 4096;
  static constexpr int kC = kEpiWarps * kCPerWarp;
  static constexpr int kTotal = kOffC + kC;
  static constexpr int kAlloc = kTotal + 1024;
  static_assert(kAlloc <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

template <int KIND, int STAGES, bool SFW, bool SWIGLU, bool SCATTER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairSmem<STAGES, SFW, SCATTER>::kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa,
                 const __grid_constant__ CUtensorMap tmap_sfb,
                 const __grid_constant__ CUtensorMap tmap_c,
                 const __grid_constant__ CUtensorMap tmap_a32, const GemmParams p) {
  using L = PairSmem<STAGES, SFW, SCATTER>;
  static_assert(!(SWIGLU && SCATTER), "one epilogue at a time");
  constexpr int kTileN = 256;
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr int kFirstSfWarp = L::kEpiWarps + 2;
  constexpr int kSfaCols = 16, kSfbCols = 32, kSlotCols = kSfaCols + kSfbCols;
  constexpr int kSfCol0 = kTileN;
  static_assert(kSfCol0 + STAGES * kSlotCols <= 512, "scale slots do not fit in TMEM");
  constexpr int kChunksPerStage = (KIND == KIND_NVFP4) ? 4 : 1;
  constexpr uint32_t kSfBoxBytes = kChunksPerStage * 512;
  constexpr uint32_t kIdescBase =
      (KIND == KIND_NVFP4)
          ? ((1u << 7) | (1u << 10) | (uint32_t(kTileN >> 3) << 17) | (16u << 24))
          : ((uint32_t(kTileN >> 3) << 17) | (1u << 23) | (16u << 24));

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);

  const uint32_t bar_full = sbase;                    // STAGES x 8 (used in the leader)
  const uint32_t bar_empty = sbase + 8 * STAGES;      // STAGES x 8
  const uint32_t bar_acc_full = sbase + 16 * STAGES;  // 8
  const uint32_t bar_acc_empty = bar_acc_full + 8;    // 8 (used in the leader)
  const uint32_t bar_sf_full = bar_acc_empty + 8;     // STAGES x 8: this CTA's scale boxes landed
  const uint32_t bar_sf_ready = bar_sf_full + 8 * STAGES;  // STAGES x 8 (leader): scales in TMEM
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + 512);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + 516);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int ntiles = p.n / kTileN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 2 * L::kEpiWarps);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_sf_full + 8 * s, 1);
      mbar_init(bar_sf_ready + 8 * s, 8);
    }
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
    tma_prefetch_desc(&tmap_c);
    tma_prefetch_desc(&tmap_a32);
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers are initialised before either touches the other's
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  // set-up is done: from here on global memory is touched, so wait for the previous kernel in
  // the stream (no-op unless launched with programmatic stream serialization), and let the
  // next one begin its own set-up as SMs free up
  grid_dependency_wait();
  grid_launch_dependents();
#ifdef MSC_DEBUG
  if (p.trace && threadIdx.x == 0) {
    p.trace[(size_t)gridDim.x * 48 + blockIdx.x * 2] = clock64();
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    p.trace[(size_t)gridDim.x * 50 + (size_t)blockIdx.x * 32 + 30] = gt;
  }
#endif

  if (warp == kProducerWarp) {
    // ------------------------------ producer (both CTAs) ------------------------
    TileCursor cur;
    cur.mshift = 8;
    uint32_t bits = 0;  // per-stage use parity
    bool ok = true;
    int tl = 0;
    for (int t = pair; ok; t += npairs, ++tl) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      const int row0 = cur.off + (2 * mt + (int)rank) * 128;
      // 32-row boxes of A that hold rows of the group, for this CTA and for its peer
      const int left = cur.rows - 2 * mt * 128;
      const int boxes_own = (min(max(left - (int)rank * 128, 0), 128) + 31) >> 5;
      const int boxes_peer = (min(max(left - (int)(rank ^ 1u) * 128, 0), 128) + 31) >> 5;
      const uint32_t sf_own = (boxes_own ? 3u : 2u) * kSfBoxBytes;
      const uint32_t sf_peer = (boxes_peer ? 3u : 2u) * kSfBoxBytes;
      const uint32_t ab_both = 2 * L::kB + uint32_t(boxes_own + boxes_peer) * 4096u;
      // plain: the tile's 256 B rows are consecutive, this CTA takes its half.  SwiGLU: the
      // tile pairs 128 gate rows (first half of B) with the 128 up rows of the same output
      // columns (second half); the even CTA feeds the gate rows, the odd CTA the up rows, so
      // accumulator columns 0-127 are gate and 128-255 are up.
      const int brow0 = SWIGLU ? cur.g * p.n + (int)rank * (p.n >> 1) + nt * 128
                               : cur.g * p.n + nt * kTileN + (int)rank * 128;
      const int sfa_row = (row0 >> 7) * p.sf_chunks * 4;
      const int sfb_row = SWIGLU ? (cur.g * (p.n >> 7) + nt) * p.sf_chunks * 4
                                 : (cur.g * (p.n >> 7) + nt * 2) * p.sf_chunks * 4;
      const int sfb_row1 = sfb_row + (SWIGLU ? (p.n >> 8) : 1) * p.sf_chunks * 4;
      uint32_t s = 0;
      MSC_STAMP(0, tl, 0);
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_empty + 8 * s, ((bits >> s) & 1u) ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t full = bar_full + 8 * s;
        // scale boxes report to this CTA's own barrier when its scale warps consume them
        const uint32_t sff = SFW ? bar_sf_full + 8 * s : full;
        const int c4 = kb * kChunksPerStage * 4;
        if (elect_one()) {
          if (SFW) {
            if (leader) mbar_arrive_expect_tx(full, ab_both);
            mbar_arrive_expect_tx(sff, sf_own);
          } else if (leader) {
            mbar_arrive_expect_tx(full, ab_both + sf_own + sf_peer);
          }
          const uint32_t a_dst = sbase + L::kOffA + s * L::kA;
          if (boxes_own == 4) {
            tma_load_2d_pair(a_dst, &tmap_a, full, kb * 128, row0);
          } else {
            for (int i = 0; i < boxes_own; ++i)
              tma_load_2d_pair(a_dst + i * 4096, &tmap_a32, full, kb * 128, row0 + 32 * i);
          }
          tma_load_2d_pair(sbase + L::kOffB + s * L::kB, &tmap_b, full, kb * 128, brow0);
          if (SFW) {
            if (boxes_own) tma_load_2d(sbase + L::kOffSfa + s * L::kSfa, &tmap_sfa, sff, 0, sfa_row + c4);
            tma_load_2d(sbase + L::kOffSfb + s * L::kSfb, &tmap_sfb, sff, 0, sfb_row + c4);
            tma_load_2d(sbase + L::kOffSfb + s * L::kSfb + 2048, &tmap_sfb, sff, 0, sfb_row1 + c4);
          } else {
            if (boxes_own)
              tma_load_2d_pair(sbase + L::kOffSfa + s * L::kSfa, &tmap_sfa, full, 0, sfa_row + c4);
            tma_load_2d_pair(sbase + L::kOffSfb + s * L::kSfb, &tmap_sfb, full, 0, sfb_row + c4);
            tma_load_2d_pair(sbase + L::kOffSfb + s * L::kSfb + 2048, &tmap_sfb, full, 0,
                             sfb_row1 + c4);
          }
        }
        __syncwarp();
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
      MSC_STAMP(0, tl, 1);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer (leader only) --------------------
    if (leader) {
      TileCursor cur;
      cur.mshift = 8;
      uint32_t bits = 0;
      int tl = 0;
      bool ok = true;
      const uint64_t adesc0 = operand_desc_sw128(sbase + L::kOffA);
      const uint64_t bdesc0 = operand_desc_sw128(sbase + L::kOffB);
      const uint64_t sfa_d0 = scale_desc(sbase + L::kOffSfa);
      const uint64_t sfb_d0 = scale_desc(sbase + L::kOffSfb);
      const uint32_t acc = tmem_base;
      for (int t = pair; ok; t += npairs, ++tl) {
        int mt, nt;
        if (!cur.seek(p, ntiles, t, mt, nt)) break;
        ok = warp_wait(bar_acc_empty, (uint32_t)(tl & 1) ^ 1u, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after_sync();
        MSC_STAMP(1, tl, 0);
        for (int kb0 = 0; kb0 < p.k_stages && ok; kb0 += STAGES) {
#pragma unroll
          for (int s = 0; s < STAGES; ++s) {
            const int kb = kb0 + s;
            if (kb >= p.k_stages) break;
            ok = warp_wait(bar_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 3);
            if (!ok) break;
            if (SFW) {
              ok = warp_wait(bar_sf_ready + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 5);
              if (!ok) break;
            }
            bits ^= 1u << s;
            tc_fence_after_sync();
            const int nch = min(kChunksPerStage, p.sf_chunks - kb * kChunksPerStage);
            const int nmma = (KIND == KIND_NVFP4) ? nch : 4;
            const uint32_t sfa_t = tmem_base + kSfCol0 + s * kSlotCols;
            const uint32_t sfb_t = sfa_t + kSfaCols;
            // descriptor low words count 16-byte units: +32 per 512-byte scale chunk, +128
            // per 2048-byte block of 128 B rows, +2 per 32 bytes of K in the operand tile
            const uint64_t sfa_d = sfa_d0 + s * (L::kSfa >> 4);
            const uint64_t sfb_d = sfb_d0 + s * (L::kSfb >> 4);
            const uint64_t adesc = adesc0 + s * (L::kA >> 4);
            const uint64_t bdesc = bdesc0 + s * (L::kB >> 4);
            if (elect_one()) {
#pragma unroll
              for (int c = 0; c < kChunksPerStage && !SFW; ++c) {
                if (c < nch) {
                  tc_cp_32x128b_warpx4_pair(sfa_t + 4 * c, sfa_d + 32 * c);
                  tc_cp_32x128b_warpx4_pair(sfb_t + 8 * c, sfb_d + 32 * c);
                  tc_cp_32x128b_warpx4_pair(sfb_t + 8 * c + 4, sfb_d + 128 + 32 * c);
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < nmma) {
                  const uint32_t accumulate = (j > 0 || kb > 0) ? 1u : 0u;
                  if (KIND == KIND_NVFP4) {
                    tc_mma_nvfp4_pair(acc, adesc + 2 * j, bdesc + 2 * j, kIdescBase, sfa_t + 4 * j,
                                      sfb_t + 8 * j, accumulate);
                  } else {
                    const uint32_t idesc = kIdescBase | (uint32_t(j) << 29) | (uint32_t(j) << 4);
                    tc_mma_mxf8_pair(acc, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t, sfb_t,
                                     accumulate);
                  }
                }
              }
              tc_commit_pair(bar_empty + 8 * s, 3);  // frees this stage in both CTAs
            }
            __syncwarp();
          }
        }
        if (ok && elect_one()) tc_commit_pair(bar_acc_full, 3);
        __syncwarp();
        MSC_STAMP(1, tl, 1);
      }
    }
  } else if (SFW && warp >= kFirstSfWarp) {
    // ------------------------------ scale writers (both CTAs) -------------------
    // Four warps, one per TMEM lane quadrant, move each stage's scale factors from shared
    // memory into TMEM through registers (tcgen05.st) instead of tcgen05.cp: the copies then
    // no longer take turns with the MMAs in the tensor pipe.  Lane b reads the 16 bytes of
    // row b of every 512-byte chunk (scales of rows b, 32+b, 64+b, 96+b for 64 K-elements) and
    // writes them to its own lane in the four columns of that chunk; every quadrant holds the
    // same copy, which is the layout the MMA expects.
    TileCursor cur;
    cur.mshift = 8;
    uint32_t bits = 0;
    bool ok = true;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    constexpr int kA4 = 4 * kChunksPerStage;        // columns of A scales per stage
    constexpr int kB4 = 8 * kChunksPerStage;        // columns of B scales per stage
    for (int t = pair; ok; t += npairs) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      uint32_t s = 0;
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_sf_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 6);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t sa = sbase + L::kOffSfa + s * L::kSfa + lane * 16;
        const uint32_t sb = sbase + L::kOffSfb + s * L::kSfb + lane * 16;
        uint32_t ra[kA4], rb[kB4];
#pragma unroll
        for (int c = 0; c < kChunksPerStage; ++c) {
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(ra[4 * c]), "=r"(ra[4 * c + 1]), "=r"(ra[4 * c + 2]), "=r"(ra[4 * c + 3])
                       : "r"(sa + c * 512) : "memory");
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(rb[8 * c + 4 * sub]), "=r"(rb[8 * c + 4 * sub + 1]),
                           "=r"(rb[8 * c + 4 * sub + 2]), "=r"(rb[8 * c + 4 * sub + 3])
                         : "r"(sb + sub * 2048 + c * 512) : "memory");
        }
        const uint32_t sfa_t = tmem_base + lane_base + kSfCol0 + s * kSlotCols;
        const uint32_t sfb_t = sfa_t + kSfaCols;
        if (KIND == KIND_NVFP4) {
          tmem_st_32x32b_x16(sfa_t, ra);
          tmem_st_32x32b_x32(sfb_t, rb);
        } else {
          tmem_st_32x32b_x4(sfa_t, ra);
          tmem_st_32x32b_x8(sfb_t, rb);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster((bar_sf_ready + 8 * s) & kLeaderMask);
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------
    // As in the single-CTA kernel: warp w drains lane quadrant w % 4, 128-column slab w / 4.
    TileCursor cur;
    cur.mshift = 8;
    int tl = 0;
    const int quad = warp & 3;
    const int slab = warp >> 2;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t box0 = sbase + L::kOffC + warp * L::kCPerWarp;
    constexpr bool kTwoBoxes = (L::kCPerWarp == 8192);
    for (int t = pair;; t += npairs, ++tl) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      bool ok = true;
      if (lane == 0) ok = mbar_wait_bounded(bar_acc_full, tl & 1, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 0) MSC_STAMP(2, tl, 0);
      const int row_warp = (2 * mt + (int)rank) * 128 + quad * 32;
      const bool valid = row_warp + lane < cur.rows;
      const bool whole_warp = row_warp + 32 <= cur.rows;
      const size_t out_row = (size_t)cur.off + row_warp + lane;
      float scale = p.alpha ? __ldg(p.alpha + cur.g) : 1.0f;
      if (p.row_scale && valid) scale *= __ldg(p.row_scale + out_row);

      uint32_t v[4][32];
      if (SWIGLU) {
        // this warp's 64 output columns: gate from accumulator columns [64 slab, +64), up from
        // [128 + 64 slab, +64)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tmem_ld_32x32b_x32(tmem_base + lane_base + slab * 64 + c * 32, v[c]);
          tmem_ld_32x32b_x32(tmem_base + lane_base + 128 + slab * 64 + c * 32, v[2 + c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tmem_ld_32x32b_x32(tmem_base + lane_base + slab * 128 + c * 32, v[c]);
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(bar_acc_empty & kLeaderMask);
      if (warp == 0) MSC_STAMP(2, tl, 1);
      if (MSC_FLAG(1)) continue;

      if (SWIGLU) {
        // gate and up are rounded to bf16 exactly as the unfused path stores them
        // (gemm1_silu_quantize.py:195-197), the activation stays fp32 (nvfp4.py:81-88), then the
        // thread quantises its four 16-column blocks: 32 bytes of e2m1 and one scale word,
        // which is one unit of the tiled scale layout the second GEMM reads.
        if (valid) {
          const float gs = __ldg(p.out_gs + cur.g);
          const int width = p.n >> 1;                       // columns of the activation
          const int col = nt * 128 + slab * 64;             // first output column of this thread
          uint32_t q8[8], sfw = 0;
#pragma unroll
          for (int blk = 0; blk < 4; ++blk) {
            float act[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int c = blk >> 1, e = (blk & 1) * 16 + i;
              const float gt = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[c][e]) * scale));
              const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[2 + c][e]) * scale));
              act[i] = silu_mul(gt, up);
            }
            uint2 q2;
            uint32_t sfb;
            quantize_16(act, gs, q2, sfb);
            q8[2 * blk] = q2.x;
            q8[2 * blk + 1] = q2.y;
            sfw |= sfb << (8 * blk);
          }
          uint4* qdst = reinterpret_cast<uint4*>(p.out_q + out_row * (width >> 1) + (col >> 1));
          qdst[0] = make_uint4(q8[0], q8[1], q8[2], q8[3]);
          qdst[1] = make_uint4(q8[4], q8[5], q8[6], q8[7]);
          *reinterpret_cast<uint32_t*>(p.out_sf + tiled_sf_word((int)out_row, col >> 6, width >> 6)) = sfw;
        }
        continue;
      }

      const int col0 = nt * kTileN + slab * 128;
      if (SCATTER) {
        // Every row goes to its own destination (another GPU's memory included): the lane
        // stages its row's 128 bf16 columns linearly and sends them as one 256-byte bulk copy.
        // A lane only ever touches its own staging row, so no warp-level ordering is needed.
        const int dcode = valid ? __ldg(p.row_dest + out_row) : -1;
        bulk_wait_group_read0();   // this lane's previous copy has left its staging row
        const uint32_t rowaddr = box0 + lane * L::kScatterPitch;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
              const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
              __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
              w[e] = *reinterpret_cast<uint32_t*>(&pr);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (c * 4 + q) * 16),
                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        }
        fence_proxy_async_smem();
        // the codes were written by other ranks: one that names a destination or a row this
        // launch was not given is refused and reported, never turned into an address
        uint8_t* base = nullptr;
        if (dcode >= 0) {
          const int drank = dcode >> 26, drow = dcode & 0x03ffffff;
          if (drank < p.scatter_count && drow < p.scatter_rows) base = p.scatter_base[drank];
          else atomicOr(reinterpret_cast<unsigned int*>(p.status), 0x00C00000u);
        }
        if (base) bulk_store_1d(base + ((size_t)(dcode & 0x03ffffff) * p.n + col0) * 2, rowaddr, 256);
        bulk_commit_group();
        continue;
      }
      if (whole_warp) {
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const uint32_t box = box0 + (kTwoBoxes ? sub * 4096 : 0);
          if (!kTwoBoxes || sub == 0) {
            if (lane == 0) bulk_wait_group_read0();  // earlier stores have left the staging box
            __syncwarp();
          }
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = sub * 2 + cc;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
                const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
                __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                w[e] = *reinterpret_cast<uint32_t*>(&pr);
              }
              const int j = cc * 4 + q;
              const uint32_t addr = box + lane * 128 + ((j ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]),
                           "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_c, box, col0 + sub * 64, cur.off + row_warp);
            bulk_commit_group();
          }
        }
      } else if (valid) {
        __nv_bfloat16* dst = p.out + out_row * p.n + col0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
              const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
              __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
              w[e] = *reinterpret_cast<uint32_t*>(&pr);
            }
            d4[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    if (SCATTER) {
      bulk_wait_group0();        // the row copies are complete, not just read
      __threadfence_system();    // they may have gone to other GPUs
    } else if (lane == 0) {
      bulk_wait_group_read0();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
#ifdef MSC_DEBUG
  if (p.trace && threadIdx.x == 0) {
    p.trace[(size_t)gridDim.x * 48 + blockIdx.x * 2 + 1] = clock64();
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    p.trace[(size_t)gridDim.x * 50 + (size_t)blockIdx.x * 32 + 31] = gt;
  }
#endif
  if (*abort_flag) {
    // a wait gave up somewhere: give loads still in flight time to land before the shared
    // memory they target is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync();  // neither CTA leaves while the other may still read its memory or signal it
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int KIND, int STAGES, bool SFW, bool SWIGLU = false, bool SCATTER = false>
static int launch_pair(const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = PairSmem<STAGES, SFW, SCATTER>;
  auto kern = gemm_pair_kernel<KIND, STAGES, SFW, SWIGLU, SCATTER>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  // programmatic stream serialization: this kernel's set-up may overlap the tail of the kernel
  // before it in the stream (it waits for that kernel before touching global memory)
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc = pdl_launch_config(grid, L::kThreads, L::kAlloc, stream, attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p));
  return MSC_OK;
}

template <int KIND, int STAGES>
static int launch_pair_v(const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream,
                         bool sf_by_warps) {
  if (p.out_q) {
    if (KIND != KIND_NVFP4 || STAGES != 5)
      return fail(MSC_ERR_UNSUPPORTED, "the fused SwiGLU epilogue is built for NVFP4 with 5 stages");
    return launch_pair<KIND_NVFP4, 5, false, true>(maps, p, grid, stream);
  }
  if (p.row_dest) {
    if (KIND != KIND_NVFP4 || STAGES != 4)
      return fail(MSC_ERR_UNSUPPORTED, "the row-scatter epilogue is built for NVFP4 with 4 stages");
    return launch_pair<KIND_NVFP4, 4, false, false, true>(maps, p, grid, stream);
  }
  if (sf_by_warps) {
    if (STAGES != 4) return fail(MSC_ERR_UNSUPPORTED, "scale-writer warps are built for 4 stages");
    return launch_pair<KIND, 4, true>(maps, p, grid, stream);
  }
  return launch_pair<KIND, STAGES, false>(maps, p, grid, stream);
}

int launch_pair_gemm(int kind, const void* a_q, const void* b_q, long long rows_total,
                     long long k_bytes, const GemmParams& p, int stages, int max_ctas,
                     cudaStream_t stream, bool sf_by_warps) {
  if (p.n % 256) return fail(MSC_ERR_BAD_ARG, "the CTA-pair kernel needs n %% 256 == 0, got n=%d", p.n);
  const int chunks_per_stage = (kind == KIND_NVFP4) ? 4 : 1;
  CUtensorMap maps[6];
  int rc = make_tmap_bytes_2d(&maps[0], a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&maps[5], a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 32);   // short tiles
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&maps[1], b_q, (uint64_t)p.l * p.n, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  const uint64_t row_tiles = (uint64_t)(rows_total + 127) / 128;
  rc = make_tmap_sf_2d(&maps[2], p.sfa, row_tiles * p.sf_chunks * 4, chunks_per_stage * 4);
  if (rc) return rc;
  rc = make_tmap_sf_2d(&maps[3], p.sfb, (uint64_t)p.l * (p.n / 128) * p.sf_chunks * 4,
                       chunks_per_stage * 4);
  if (rc) return rc;
  if (p.out_q) {
    maps[4] = maps[0];  // the fused epilogue stores with plain writes: no store map needed
    stages = 5;
  } else if (p.row_dest) {
    maps[4] = maps[0];  // rows leave as untiled bulk copies: no store map needed
    stages = 4;
  } else {
    rc = make_tmap_bf16_2d(&maps[4], p.out, (uint64_t)rows_total, (uint64_t)p.n, 32);
    if (rc) return rc;
  }

  const long long max_tiles = ((rows_total + 255) / 256 + p.l) * (long long)(p.n / 256);
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  if (pairs > max_tiles) pairs = (int)max_tiles;
  const int grid = 2 * pairs;
  // the ring is latency-bound: every extra stage in flight pays (8192^3 NVFP4: 307 / 224 / 196 /
  // 189 us with 2 / 3 / 4 / 5 stages), and five is what fits beside the store staging
  if (stages <= 0) stages = sf_by_warps ? 4 : 5;
  if (stages > 5) stages = 5;
  if (stages < 2) stages = 2;
  if (kind == KIND_NVFP4) {
    switch (stages) {
      case 2: return launch_pair_v<KIND_NVFP4, 2>(maps, p, grid, stream, sf_by_warps);
      case 3: return launch_pair_v<KIND_NVFP4, 3>(maps, p, grid, stream, sf_by_warps);
      case 4: return launch_pair_v<KIND_NVFP4, 4>(maps, p, grid, stream, sf_by_warps);
      default: return launch_pair_v<KIND_NVFP4, 5>(maps, p, grid, stream, sf_by_warps);
    }
  }
  switch (stages) {
    case 2: return launch_pair_v<KIND_MXFP8, 2>(maps, p, grid, stream, sf_by_warps);
    case 3: return launch_pair_v<KIND_MXFP8, 3>(maps, p, grid, stream, sf_by_warps);
    case 4: return launch_pair_v<KIND_MXFP8, 4>(maps, p, grid, stream, sf_by_warps);
    default: return launch_pair_v<KIND_MXFP8, 5>(maps, p, grid, stream, sf_by_warps);
  }
}

}  // namespace msc
