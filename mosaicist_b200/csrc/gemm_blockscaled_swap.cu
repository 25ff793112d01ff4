// Block-scaled grouped GEMM (NVFP4, and MXFP8 with the plain epilogue) on CTA pairs with the
// operands' roles exchanged: the WEIGHTS are the MMA's M side (256 rows of B per pair tile, 128
// per CTA) and the TOKENS its N side.  N has a granularity of 16, so one tile takes up to 320
// rows of a group: up to 256 as one MMA, more as two MMAs (the first 128 tokens, then the
// rest) that share the weight stage.  A group of 272
// rows - the routed MoE layer under uniform routing gives every expert 256 +- 16 - then costs
// 1.06 tiles of tensor time and one pass over the weights, instead of the two 256-row tiles
// (the second one almost empty but as expensive in the tensor pipe as a full one) of the
// row-major kernel.  The cost of an MMA follows its N down to a floor of about 50 cycles, which
// is why the two MMAs split the tokens 128 + rest and not 256 + a few.
//
// The accumulator is the transpose of the output: TMEM lane = weight row = output column,
// TMEM column = token (token t of the tile in column t, whichever MMA produced it).  The plain
// epilogue turns 32 tokens x 32 columns per warp around in shared memory and writes them out
// with 16-byte stores; the fused SwiGLU epilogue transposes 64 tokens at a time through shared
// memory and then activates and quantises one 16-column block per thread.
//
// The fused form reads w1 with gate and up rows interleaved in blocks of 64 (rows [128 i, +64)
// are gate rows 64 i .. 64 i + 63, rows [128 i + 64, +64) the up rows of the same columns), so
// that a CTA's 128 weight rows hold both halves of 64 output columns; msc_swiglu_interleave_w1
// produces that layout once, when the weights are loaded.
//
// Barriers, the ring and the TMEM hand-over are those of gemm_blockscaled_pair.cu.  Scale
// factors are staged in two rotating 80-column TMEM slots (weights 16, tokens of the first MMA
// 32, of the second 32); tcgen05.cp and tcgen05.mma execute in issue order, so a slot is reused
// two stages later without a barrier.  No load is multicast.
#include "gemm_common.cuh"
#include "quantize_common.cuh"

namespace msc {

template <int KIND, int STAGES, bool SWIGLU>
struct SwapSmem {
  static constexpr int kChunks = (KIND == KIND_NVFP4) ? 4 : 1;   // 512-byte scale chunks per 128-row block and stage
  static constexpr int kHeader = 1024;
  static constexpr int kW = 128 * 128;        // this CTA's 128 weight rows
  static constexpr int kT = 160 * 128;        // this CTA's half of the tile's (up to) 320 tokens
  static constexpr int kSfw = kChunks * 512;
  static constexpr int kSft = 3 * kChunks * 512;    // scales of all (up to) 384 token rows
  static constexpr int kOffW = kHeader;
  static constexpr int kOffT = kOffW + STAGES * kW;
  static constexpr int kOffSfw = kOffT + STAGES * kT;
  static constexpr int kOffSft = kOffSfw + STAGES * kSfw;
  static constexpr int kOffC = kOffSft + STAGES * kSft;
  static constexpr int kEpiWarps = 8;
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
  // SwiGLU: two buffers of 64 tokens x 128 bf16 at a 272-byte pitch (16-byte reads of
  // consecutive tokens then fall in different banks).  Plain: one [32 tokens][32 columns] fp32
  // box per epilogue warp.
  static constexpr int kPitch = 272;
  static constexpr int kBoxPitch = 36 * 4;            // plain: a token's 32 fp32 columns, padded
  static constexpr int kBoxBytes = 32 * kBoxPitch;    // one box of 32 tokens per epilogue warp
  static constexpr int kC = SWIGLU ? 2 * 64 * kPitch : kEpiWarps * kBoxBytes;
  static constexpr int kTotal = kOffC + kC;
  static constexpr int kAlloc = kTotal + 1024;
  static_assert(kAlloc <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// Token tiles of a group: 256 rows each, the last one also taking a remainder of up to 64.
__device__ __forceinline__ int swap_token_tiles(int rows) {
  if (rows <= 0) return 0;
  const int full = rows >> 8, rem = rows & 255;
  if (rem == 0) return full;
  return (rem <= 64 && full >= 1) ? full : full + 1;
}

// Walks (group, token tile, weight tile) in increasing tile id; weight tiles vary fastest.
struct SwapCursor {
  int g = 0, base = 0, ttiles = 0, rows = 0, off = 0;
  bool primed = false;
  __device__ __forceinline__ bool seek(const GemmParams& p, int ntiles, int t, int& tt, int& nt) {
    while (true) {
      if (!primed) {
        if (g >= p.l) return false;
        rows = __shfl_sync(0xffffffffu, __ldg(p.group_rows + g), 0);
        off = __shfl_sync(0xffffffffu, __ldg(p.group_offsets + g), 0);
        if (rows < 0) rows = 0;
        // a group table that reaches beyond the buffers is cut to what the buffers hold
        if (off < 0 || off >= p.rows_total) rows = 0;
        else if (rows > p.rows_total - off) rows = p.rows_total - off;
        ttiles = swap_token_tiles(rows);
        primed = true;
      }
      const int tiles = ttiles * ntiles;
      if (t < base + tiles) break;
      base += tiles;
      ++g;
      primed = false;
    }
    const int u = t - base;
    tt = u / ntiles;
    nt = u - tt * ntiles;
    return true;
  }
  // tokens of tile tt, and the widths (multiples of 16) of the MMAs that cover them: one MMA up
  // to 256 tokens, otherwise the first 128 tokens and the rest (up to 192)
  __device__ __forceinline__ void widths(int tt, int& tn, int& n0, int& n1) const {
    tn = (tt == ttiles - 1) ? rows - tt * 256 : 256;
    if (tn <= 256) {
      n0 = (tn + 15) & ~15;
      n1 = 0;
    } else {
      n0 = 128;
      n1 = (tn - 128 + 15) & ~15;
    }
  }
};

template <int KIND, int STAGES, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SwapSmem<KIND, STAGES, SWIGLU>::kThreads, 1)
gemm_swap_kernel(const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_t,
                 const __grid_constant__ CUtensorMap tmap_t32,
                 const __grid_constant__ CUtensorMap tmap_sfw,
                 const __grid_constant__ CUtensorMap tmap_sft, const GemmParams p) {
  using L = SwapSmem<KIND, STAGES, SWIGLU>;
  static_assert(KIND == KIND_NVFP4 || !SWIGLU, "the fused epilogue quantises to NVFP4");
  constexpr int kChunks = L::kChunks;
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr int kAcc1Col = 128;                 // second accumulator: tokens 128 .. 319
  // a slot: weights 4 columns per chunk, tokens of the first MMA 8, of the second 8
  constexpr int kSfCol0 = 320, kSlotCols = 20 * kChunks, kSlots = 2;
  constexpr int kSfwCols = 0, kSft0Cols = 4 * kChunks, kSft1Cols = 12 * kChunks;   // offsets inside a slot
  constexpr uint32_t kSfBoxBytes = kChunks * 512;
  constexpr uint32_t kIdescBase = (KIND == KIND_NVFP4) ? ((1u << 7) | (1u << 10) | (16u << 24))
                                                       : ((1u << 23) | (16u << 24));

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);

  const uint32_t bar_full = sbase;                    // STAGES x 8 (used in the leader)
  const uint32_t bar_empty = sbase + 8 * STAGES;      // STAGES x 8
  const uint32_t bar_acc_full = sbase + 16 * STAGES;  // 8
  const uint32_t bar_acc_empty = bar_acc_full + 8;    // 8 (used in the leader)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + 512);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + 516);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int ntiles = p.n >> 8;   // weight tiles of 256 rows

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 2 * L::kEpiWarps);
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_t);
    tma_prefetch_desc(&tmap_t32);
    tma_prefetch_desc(&tmap_sfw);
    tma_prefetch_desc(&tmap_sft);
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
  grid_dependency_wait();
  grid_launch_dependents();
#ifdef MSC_DEBUG
  if (p.trace && threadIdx.x == 0) p.trace[(size_t)gridDim.x * 48 + blockIdx.x * 2] = clock64();
#endif

  if (warp == kProducerWarp) {
    // ------------------------------ producer (both CTAs) ------------------------
    SwapCursor cur;
    uint32_t bits = 0;  // per-stage use parity
    bool ok = true;
    uint32_t s = 0;
    int tl = 0;
    for (int t = pair; ok; t += npairs, ++tl) {
      int tt, nt;
      if (!cur.seek(p, ntiles, t, tt, nt)) break;
      int tn, n0, n1;
      cur.widths(tt, tn, n0, n1);
      MSC_STAMP(0, tl, 0);
      const int wrow0 = cur.g * p.n + nt * 256 + (int)rank * 128;
      // this CTA's tokens: half of each MMA's, 32-row boxes, the second MMA's behind the first's
      const int trow0 = cur.off + tt * 256 + (int)rank * (n0 >> 1);
      const int trow1 = cur.off + tt * 256 + 128 + (int)rank * (n1 >> 1);
      const int boxes0 = ((n0 >> 1) + 31) >> 5, boxes1 = ((n1 >> 1) + 31) >> 5;
      const int sfw_row = (cur.g * (p.n >> 7) + nt * 2 + (int)rank) * p.sf_chunks * 4;
      const int sft_row = ((cur.off + tt * 256) >> 7) * p.sf_chunks * 4;
      const int blocks = (tn + 127) >> 7;                       // 128-token scale blocks, 1 .. 3
      // both CTAs load the same amounts
      const uint32_t bytes = L::kW + (uint32_t)(boxes0 + boxes1) * 4096u + (1u + (uint32_t)blocks) * kSfBoxBytes;
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_empty + 8 * s, ((bits >> s) & 1u) ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t full = bar_full + 8 * s;
        const int c4 = kb * kChunks * 4;
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(full, 2 * bytes);
          tma_load_2d_pair(sbase + L::kOffW + s * L::kW, &tmap_w, full, kb * 128, wrow0);
          const uint32_t t_dst = sbase + L::kOffT + s * L::kT;
          if (boxes0 == 4) {
            tma_load_2d_pair(t_dst, &tmap_t, full, kb * 128, trow0);
          } else {
            for (int i = 0; i < boxes0; ++i)
              tma_load_2d_pair(t_dst + i * 4096, &tmap_t32, full, kb * 128, trow0 + 32 * i);
          }
          for (int i = 0; i < boxes1; ++i)   // behind the 64 rows of the first MMA
            tma_load_2d_pair(t_dst + 8192 + i * 4096, &tmap_t32, full, kb * 128, trow1 + 32 * i);
          tma_load_2d_pair(sbase + L::kOffSfw + s * L::kSfw, &tmap_sfw, full, 0, sfw_row + c4);
          const uint32_t sft_dst = sbase + L::kOffSft + s * L::kSft;
          for (int bl = 0; bl < blocks; ++bl)
            tma_load_2d_pair(sft_dst + bl * kSfBoxBytes, &tmap_sft, full, 0, sft_row + bl * p.sf_chunks * 4 + c4);
        }
        __syncwarp();
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer (leader only) --------------------
    if (leader) {
      SwapCursor cur;
      uint32_t bits = 0;
      int tl = 0;
      bool ok = true;
      uint32_t s = 0, slot = 0;
      const uint64_t wdesc0 = operand_desc_sw128(sbase + L::kOffW);
      const uint64_t tdesc0 = operand_desc_sw128(sbase + L::kOffT);
      const uint64_t sfw_d0 = scale_desc(sbase + L::kOffSfw);
      const uint64_t sft_d0 = scale_desc(sbase + L::kOffSft);
      for (int t = pair; ok; t += npairs, ++tl) {
        int tt, nt;
        if (!cur.seek(p, ntiles, t, tt, nt)) break;
        int tn, n0, n1;
        cur.widths(tt, tn, n0, n1);
        const uint32_t idesc0 = kIdescBase | (uint32_t(n0 >> 3) << 17);
        const uint32_t idesc1 = kIdescBase | (uint32_t(n1 >> 3) << 17);
        ok = warp_wait(bar_acc_empty, (uint32_t)(tl & 1) ^ 1u, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after_sync();
        MSC_STAMP(1, tl, 0);
        for (int kb = 0; kb < p.k_stages; ++kb) {
          ok = warp_wait(bar_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 3);
          if (!ok) break;
          bits ^= 1u << s;
          tc_fence_after_sync();
          const int nch = min(kChunks, p.sf_chunks - kb * kChunks);
          const int nmma = (KIND == KIND_NVFP4) ? nch : 4;
          const uint32_t slot_t = tmem_base + kSfCol0 + slot * kSlotCols;
          const uint32_t sfw_t = slot_t + kSfwCols, sft0_t = slot_t + kSft0Cols, sft1_t = slot_t + kSft1Cols;
          // descriptor low words count 16-byte units: +32 per 512-byte scale chunk, +kBlk per
          // block of 128 rows, +2 per 32 bytes of K in the operand tile, +512 per 64 operand rows
          constexpr int kBlk = kChunks * 32;
          const uint64_t sfw_d = sfw_d0 + s * (L::kSfw >> 4);
          const uint64_t sft_d = sft_d0 + s * (L::kSft >> 4);
          const uint64_t wdesc = wdesc0 + s * (L::kW >> 4);
          const uint64_t tdesc = tdesc0 + s * (L::kT >> 4);
          if (elect_one()) {
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              if (c < nch) {
                tc_cp_32x128b_warpx4_pair(sfw_t + 4 * c, sfw_d + 32 * c);
                tc_cp_32x128b_warpx4_pair(sft0_t + 8 * c, sft_d + 32 * c);
                if (n1) {   // second MMA: tokens from 128 on, i.e. scale blocks 1 (and 2)
                  tc_cp_32x128b_warpx4_pair(sft1_t + 8 * c, sft_d + kBlk + 32 * c);
                  if (n1 > 128) tc_cp_32x128b_warpx4_pair(sft1_t + 8 * c + 4, sft_d + 2 * kBlk + 32 * c);
                } else if (n0 > 128) {
                  tc_cp_32x128b_warpx4_pair(sft0_t + 8 * c + 4, sft_d + kBlk + 32 * c);
                }
              }
            }
            // NVFP4: one MMA per 64-element chunk, each with its own scale columns; MXFP8: four
            // MMAs of 32 elements share the chunk's columns and pick their byte through the
            // descriptor's scale ids
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < nmma) {
                const uint32_t accumulate = (j > 0 || kb > 0) ? 1u : 0u;
                if (KIND == KIND_NVFP4)
                  tc_mma_nvfp4_pair(tmem_base, wdesc + 2 * j, tdesc + 2 * j, idesc0, sfw_t + 4 * j,
                                    sft0_t + 8 * j, accumulate);
                else
                  tc_mma_mxf8_pair(tmem_base, wdesc + 2 * j, tdesc + 2 * j,
                                   idesc0 | (uint32_t(j) << 29) | (uint32_t(j) << 4), sfw_t, sft0_t, accumulate);
              }
            }
            if (n1 && !MSC_FLAG(8)) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < nmma) {
                  const uint32_t accumulate = (j > 0 || kb > 0) ? 1u : 0u;
                  if (KIND == KIND_NVFP4)
                    tc_mma_nvfp4_pair(tmem_base + kAcc1Col, wdesc + 2 * j, tdesc + 512 + 2 * j, idesc1,
                                      sfw_t + 4 * j, sft1_t + 8 * j, accumulate);
                  else
                    tc_mma_mxf8_pair(tmem_base + kAcc1Col, wdesc + 2 * j, tdesc + 512 + 2 * j,
                                     idesc1 | (uint32_t(j) << 29) | (uint32_t(j) << 4), sfw_t, sft1_t, accumulate);
                }
              }
            }
            tc_commit_pair(bar_empty + 8 * s, 3);  // frees this stage in both CTAs
          }
          __syncwarp();
          s = (s + 1 == STAGES) ? 0u : s + 1;
          slot = (slot + 1 == kSlots) ? 0u : slot + 1;
        }
        if (ok && elect_one()) tc_commit_pair(bar_acc_full, 3);
        __syncwarp();
        MSC_STAMP(1, tl, 1);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------
    // warp w reads lane quadrant w % 4 (32 weight rows = 32 output columns); the two halves
    // w / 4 split the tokens.
    SwapCursor cur;
    int tl = 0;
    int pass_no = 0;   // SwiGLU: passes so far, over all tiles (selects the staging buffer)
    const int quad = warp & 3;
    const int half = warp >> 2;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    for (int t = pair;; t += npairs, ++tl) {
      int tt, nt;
      if (!cur.seek(p, ntiles, t, tt, nt)) break;
      int tn, n0, n1;
      cur.widths(tt, tn, n0, n1);
      // the row scales of this warp's tokens, one token per lane and chunk, while the K loop
      // still runs: every later use takes them from here with a shuffle
      float rsv[5];
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        const int tok = (2 * i + half) * 32 + lane;
        rsv[i] = (p.row_scale && tok < tn) ? __ldg(p.row_scale + (size_t)cur.off + (size_t)tt * 256 + tok) : 1.0f;
      }
      bool ok = true;
      if (lane == 0) ok = mbar_wait_bounded(bar_acc_full, tl & 1, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (SWIGLU) {
        // the passes below meet at a named barrier: all eight warps go on or none does, or a
        // warp whose wait gave up would leave the others waiting there for good
        uint32_t all_ok;
        asm volatile(
            "{\n"
            " .reg .pred p, q;\n"
            " setp.ne.u32 p, %1, 0;\n"
            " bar.red.and.pred q, 1, 256, p;\n"
            " selp.u32 %0, 1, 0, q;\n"
            "}\n"
            : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
        ok = all_ok != 0;
      }
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 0) MSC_STAMP(2, tl, 0);
      const float alpha = p.alpha ? __ldg(p.alpha + cur.g) : 1.0f;
      const size_t row0 = (size_t)cur.off + (size_t)tt * 256;   // first token row of the tile
      // 32 tokens of this lane's row, as read from TMEM -> alpha (and the tokens' row scales)
      // applied, rounded to bf16, two tokens per register
      auto pack = [&](const uint32_t* raw, float rs_lane, uint32_t* pk) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float s0 = alpha, s1 = alpha;
          if (p.row_scale) {
            s0 *= __shfl_sync(0xffffffffu, rs_lane, 2 * i);
            s1 *= __shfl_sync(0xffffffffu, rs_lane, 2 * i + 1);
          }
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(raw[2 * i]) * s0,
                                                         __uint_as_float(raw[2 * i + 1]) * s1);
          pk[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
      };
      const int nchunks = (tn + 31) >> 5;   // 32-token chunks of the tile, up to 10

      // Token t of the tile sits in accumulator column t; the warps of half h take the 32-token
      // chunks h, h + 2, ... (five each cover the 320 columns).  The accumulator must be free
      // again quickly - the next tile's MMAs wait for it - and 160 raw registers do not fit: a
      // fifth chunk, which only a two-MMA tile has, is read and packed first (16 registers),
      // then the other four are read with one wait, as 128 raw registers, and the accumulator is
      // released; they are packed one by one where they are used.
      uint32_t pk4[16];
      const bool have4 = 8 + half < nchunks;
      if (have4) {
        uint32_t tmp[32];
        tmem_ld_32x32b_x32(tmem_base + lane_base + (8 + half) * 32, tmp);
        tmem_ld_wait();
        pack(tmp, rsv[4], pk4);
      }
      uint32_t raw[4][32];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (2 * i + half < nchunks) tmem_ld_32x32b_x32(tmem_base + lane_base + (2 * i + half) * 32, raw[i]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(bar_acc_empty & kLeaderMask);
      if (warp == 0) MSC_STAMP(2, tl, 1);

      if (!SWIGLU) {
        if (MSC_FLAG(1)) continue;
        const int colw = nt * 256 + (int)rank * 128 + quad * 32;   // first output column of this warp
        const uint32_t box0 = sbase + L::kOffC + warp * L::kBoxBytes;
        // A chunk (32 tokens x this warp's 32 columns) is turned around in the warp's shared box
        // as raw fp32 ([token][column], rows 36 words apart so that neither phase has a bank
        // conflict); then four lanes take a token's 32 columns, eight each: they apply alpha and
        // the token's row scale, round to bf16 and write 16 bytes - a token's 64 bytes are two
        // full sectors, eight tokens go out per instruction.  Tiled bulk stores were slower here:
        // they queue behind the ring's loads in the copy engine, and with a tile only eight stages
        // long the epilogue then outlasts the K loop.
        const int piece = lane & 3;
        auto store_chunk = [&](const uint32_t* vals, int tok_first, float rs_lane, bool scaled) {
          float sc[4];   // alpha x the row scale of each of this lane's four tokens
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const float rs = __shfl_sync(0xffffffffu, rs_lane, r * 8 + (lane >> 2));
            sc[r] = scaled ? 1.0f : alpha * rs;
          }
          __syncwarp();   // the previous chunk has been read out of the box
#pragma unroll
          for (int e = 0; e < 32; ++e)
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(box0 + e * L::kBoxPitch + lane * 4), "r"(vals[e]) : "memory");
          __syncwarp();
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int tl_ = r * 8 + (lane >> 2);
            const int tok = tok_first + tl_;
            float f[8];
#pragma unroll
            for (int h = 0; h < 2; ++h)
              asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(f[4 * h]), "=f"(f[4 * h + 1]), "=f"(f[4 * h + 2]), "=f"(f[4 * h + 3])
                           : "r"(box0 + tl_ * L::kBoxPitch + piece * 32 + h * 16) : "memory");
            if (tok < tn) {
              uint32_t w[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const __nv_bfloat162 pr = __floats2bfloat162_rn(f[2 * h] * sc[r], f[2 * h + 1] * sc[r]);
                w[h] = *reinterpret_cast<const uint32_t*>(&pr);
              }
              *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) +
                                        ((row0 + tok) * (size_t)p.n + colw) * 2 + piece * 16) =
                  make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        };
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ci = 2 * i + half;
          if (ci >= nchunks) break;
          store_chunk(raw[i], ci * 32, rsv[i], false);
        }
        if (have4) {
          // the fifth chunk was scaled and rounded when it was packed: bf16 -> fp32 is exact, and
          // so is rounding it back
          uint32_t vals[32];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            vals[2 * e] = pk4[e] << 16;
            vals[2 * e + 1] = pk4[e] & 0xffff0000u;
          }
          store_chunk(vals, (8 + half) * 32, 1.0f, true);
        }
        if (warp == 0) MSC_STAMP(0, tl, 1);   // debug builds: end of this tile's epilogue
        continue;
      }

      // ---- fused SwiGLU + quantise --------------------------------------------------
      // This CTA's lanes 0-63 are gate rows, 64-127 the up rows of the same 64 output columns
      // (columns [64 (2 nt + rank), +64) of the activation).  Passes of 64 tokens (this warp's
      // half of pass ps is chunk 2 ps + half): every warp puts its 32 rows x 32 tokens, already
      // rounded to bf16 (gemm1_silu_quantize.py:195-197), into a shared [token][row] tile; after
      // a barrier thread (token, 16-column block) activates (nvfp4.py:81-88) and quantises its
      // block.
      const float gs = __ldg(p.out_gs + cur.g);
      const int width = p.n >> 1;                       // columns of the activation
      const int col0 = (nt * 2 + (int)rank) * 64;       // first activation column of this CTA
      const uint32_t cbase = sbase + L::kOffC;
      // phase 2: thread (token, 16-column block) with the four blocks of a token in adjacent
      // lanes, so that a warp's 8-byte stores fill whole 32-byte sectors and the four scale bytes
      // of a token's 64 columns leave as one word (the epilogue warps are warps 0-7)
      const int p_tok = threadIdx.x >> 2, p_blk = threadIdx.x & 3;
      const int npasses = (tn + 63) >> 6;
#pragma unroll
      for (int ps = 0; ps < 5; ++ps) {
        if (ps >= npasses) break;                       // uniform over the CTA's epilogue warps
        const int tok_first = ps * 64;
        const uint32_t buf = cbase + (pass_no & 1) * (64 * L::kPitch);
        ++pass_no;
        const uint32_t dst = buf + (half * 32) * L::kPitch + (quad * 32 + lane) * 2;
        if (2 * ps + half < nchunks) {                  // tokens beyond the tile are never read back
          uint32_t pk[16];
          if (ps < 4) {
            // (the index is clamped for the unrolled ps == 4 copy of this branch, which never runs)
            pack(raw[ps < 4 ? ps : 0], rsv[ps < 4 ? ps : 0], pk);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pk4[i];
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst + (2 * i) * L::kPitch),
                         "h"((uint16_t)(pk[i] & 0xffffu)) : "memory");
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst + (2 * i + 1) * L::kPitch),
                         "h"((uint16_t)(pk[i] >> 16)) : "memory");
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const int tok = tok_first + p_tok;
        {   // tokens beyond the tile compute on stale bytes and store nothing: the lanes of a warp stay together
          const uint32_t src = buf + p_tok * L::kPitch + p_blk * 32;
          uint4 graw[2], uraw[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(graw[i].x), "=r"(graw[i].y), "=r"(graw[i].z), "=r"(graw[i].w)
                         : "r"(src + i * 16) : "memory");
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(uraw[i].x), "=r"(uraw[i].y), "=r"(uraw[i].z), "=r"(uraw[i].w)
                         : "r"(src + 128 + i * 16) : "memory");
          }
          float act[16];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw[i]);
            const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 gt = __bfloat1622float2(gh[e]);
              const float2 up = __bfloat1622float2(uh[e]);
              act[i * 8 + e * 2] = silu_mul(gt.x, up.x);
              act[i * 8 + e * 2 + 1] = silu_mul(gt.y, up.y);
            }
          }
          uint2 q2;
          uint32_t sfb;
          quantize_16(act, gs, q2, sfb);
          const uint32_t sfw = gather_scale_word(sfb);   // valid in the lane of block 0
          const size_t orow = row0 + tok;
          const int col = col0 + p_blk * 16;
          if (tok < tn) {
            *reinterpret_cast<uint2*>(p.out_q + orow * (width >> 1) + (col >> 1)) = q2;
            if (p_blk == 0)
              *reinterpret_cast<uint32_t*>(p.out_sf + tiled_sf_word((int)orow, col0 >> 6, width >> 6)) = sfw;
          }
        }
      }
      if (warp == 0) MSC_STAMP(0, tl, 1);   // debug builds: end of this tile's epilogue
    }
  }

  tc_fence_before_sync();
  __syncthreads();
#ifdef MSC_DEBUG
  if (p.trace && threadIdx.x == 0) p.trace[(size_t)gridDim.x * 48 + blockIdx.x * 2 + 1] = clock64();
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

template <int KIND, int STAGES, bool SWIGLU>
static int launch_swap(const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = SwapSmem<KIND, STAGES, SWIGLU>;
  auto kern = gemm_swap_kernel<KIND, STAGES, SWIGLU>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc = pdl_launch_config(grid, L::kThreads, L::kAlloc, stream, attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, maps[0], maps[1], maps[2], maps[3], maps[4], p));
  return MSC_OK;
}

int launch_swap_gemm(int kind, const void* a_q, const void* b_q, long long rows_total, long long k_bytes,
                     const GemmParams& p, int max_ctas, cudaStream_t stream) {
  const int chunk_rows = (kind == KIND_NVFP4) ? 16 : 4;   // 128-byte rows of a stage's scale chunks
  if (kind != KIND_NVFP4 && p.out_q)
    return fail(MSC_ERR_UNSUPPORTED, "the fused SwiGLU epilogue is built for NVFP4");
  if (p.n % 256) return fail(MSC_ERR_BAD_ARG, "the tokens-on-N kernel needs n %% 256 == 0, got n=%d", p.n);
  if (!p.group_rows || !p.group_offsets)
    return fail(MSC_ERR_BAD_ARG, "the tokens-on-N kernel takes row-concatenated groups");
  if (p.row_dest) return fail(MSC_ERR_UNSUPPORTED, "the tokens-on-N kernel has no row-scatter epilogue");
  CUtensorMap maps[5];
  int rc = make_tmap_bytes_2d(&maps[0], b_q, (uint64_t)p.l * p.n, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&maps[1], a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&maps[2], a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 32);
  if (rc) return rc;
  rc = make_tmap_sf_2d(&maps[3], p.sfb, (uint64_t)p.l * (p.n / 128) * p.sf_chunks * 4, chunk_rows);
  if (rc) return rc;
  const uint64_t row_tiles = (uint64_t)(rows_total + 127) / 128;
  rc = make_tmap_sf_2d(&maps[4], p.sfa, row_tiles * p.sf_chunks * 4, chunk_rows);
  if (rc) return rc;
  const long long max_tiles = ((rows_total + 255) / 256 + p.l) * (long long)(p.n / 256);
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  if (pairs > max_tiles) pairs = (int)max_tiles;
  const int grid = 2 * pairs;
  if (p.out_q) return launch_swap<KIND_NVFP4, 4, true>(maps, p, grid, stream);
  if (kind == KIND_NVFP4) return launch_swap<KIND_NVFP4, 4, false>(maps, p, grid, stream);
  return launch_swap<KIND_MXFP8, 4, false>(maps, p, grid, stream);
}

// ---- w1 with gate and up rows interleaved in blocks of 64 ------------------------------------
// dst row 128 i + j is gate row 64 i + j for j < 64 and up row n + 64 i + (j - 64) otherwise
// (n = n2 / 2); packed values move 16 bytes per thread, scale words one per thread.
__global__ void __launch_bounds__(256)
swiglu_interleave_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                         uint8_t* __restrict__ oq, uint8_t* __restrict__ osf, int l, int n2, int kh,
                         int kwords) {
  const int n = n2 >> 1;
  const int vecs = kh >> 4;                       // 16-byte pieces of a packed row
  const int per_row = vecs + kwords;              // work items of one row
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long rowi = item / per_row;
  if (rowi >= (long long)l * n2) return;
  const int w = (int)(item - rowi * per_row);
  const int g = (int)(rowi / n2), dr = (int)(rowi - (long long)g * n2);
  const int blk = dr >> 7, j = dr & 127;
  const int sr = j < 64 ? blk * 64 + j : n + blk * 64 + (j - 64);
  if (w < vecs) {
    reinterpret_cast<uint4*>(oq + ((size_t)g * n2 + dr) * kh)[w] =
        __ldg(reinterpret_cast<const uint4*>(q + ((size_t)g * n2 + sr) * kh) + w);
  } else {
    const int kw = w - vecs;
    const size_t gbase = (size_t)g * (n2 >> 7) * kwords * 512;
    *reinterpret_cast<uint32_t*>(osf + gbase + tiled_sf_word(dr, kw, kwords)) =
        __ldg(reinterpret_cast<const uint32_t*>(sf + gbase + tiled_sf_word(sr, kw, kwords)));
  }
}

}  // namespace msc

extern "C" int msc_swiglu_interleave_w1(const void* w1_q, const void* w1_sf, void* out_q, void* out_sf,
                                        int l, int n2, int k, void* stream) {
  using namespace msc;
  if (!w1_q || !w1_sf || !out_q || !out_sf) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (w1_q == out_q || w1_sf == out_sf) return fail(MSC_ERR_BAD_ARG, "the interleaved copy cannot be made in place");
  if (l <= 0 || n2 <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (n2 % 256) return fail(MSC_ERR_BAD_ARG, "n2=%d (gate + up rows) must be a multiple of 256", n2);
  if (k % 64) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 64", k);
  if (reinterpret_cast<uintptr_t>(w1_q) % 16 || reinterpret_cast<uintptr_t>(out_q) % 16 ||
      reinterpret_cast<uintptr_t>(w1_sf) % 4 || reinterpret_cast<uintptr_t>(out_sf) % 4)
    return fail(MSC_ERR_BAD_ARG, "packed weights must be 16-byte aligned, scales 4-byte aligned");
  const int kh = k / 2, kwords = k / 64;
  const long long items = (long long)l * n2 * (kh / 16 + kwords);
  const long long blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  swiglu_interleave_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(w1_q), static_cast<const uint8_t*>(w1_sf), static_cast<uint8_t*>(out_q),
      static_cast<uint8_t*>(out_sf), l, n2, kh, kwords);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}
