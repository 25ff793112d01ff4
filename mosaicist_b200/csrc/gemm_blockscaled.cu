// Block-scaled grouped GEMM for sm_100a: NVFP4 (e2m1 x e2m1, ue4m3 scale per 16) and
// MXFP8 (e4m3 x e4m3, ue8m0 scale per 32), fp32 accumulation in TMEM, bf16 output.
//
// One persistent CTA per SM, three roles:
//   epilogue warps (4 for 128-wide tiles, 8 for 256-wide): tcgen05.ld a 32-row x 128-column
//              block of the accumulator, scale, round to bf16, TMA-store through shared memory
//   MMA warp:  one elected lane stages scale factors into TMEM (tcgen05.cp) and issues
//              tcgen05.mma for each K step of the tile
//   producer warp: one elected lane issues TMA loads for the operand ring
// The accumulator is double-buffered in TMEM (when two fit) so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Both operand kinds move the same bytes: a K stage is 128 bytes of K per row (256 e2m1 or
// 128 e4m3 elements), loaded as a [128 or TILE_N rows] x 128 B box with the 128-byte swizzle,
// and consumed by four MMAs that each advance 32 bytes along K.  What differs is the scale
// bookkeeping: NVFP4 uses one 512-byte scale chunk (32 x 16 B: 128 rows x 4 scales) per MMA,
// MXFP8 one chunk per stage with the MMA picking its byte through the descriptor's
// scale-factor id.
//
// Arithmetic follows masked_grouped_gemm_reference
// (experiments/flashinfer-megamoe-sm100a/nvfp4.py:68-78): products of e2m1/e4m3 values and
// their block scales accumulate in fp32, alpha is applied in fp32, one rounding to bf16.
#include "gemm_common.cuh"

namespace msc {

#ifdef MSC_DEBUG
unsigned long long* g_trace = nullptr;
int g_debug_flags = 0;
#endif

template <int TILE_N, int STAGES>
struct Smem {
  static constexpr int kHeader = 1024;
  static constexpr int kA = 128 * 128;
  static constexpr int kB = TILE_N * 128;
  static constexpr int kSub = TILE_N / 128;
  static constexpr int kSfa = 4 * 512;
  static constexpr int kSfb = 4 * 512 * kSub;
  static constexpr int kOffA = kHeader;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffSfa = kOffB + STAGES * kB;
  static constexpr int kOffSfb = kOffSfa + STAGES * kSfa;
  static constexpr int kEpiWarps = (TILE_N == 256) ? 8 : 4;  // one 128-column slab per warp
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
  static constexpr int kOffC = kOffSfb + STAGES * kSfb;  // epilogue staging, 32 KB in all
  static constexpr int kCPerWarp = 32768 / kEpiWarps;    // two 4 KB boxes (4 warps) or one (8)
  static constexpr int kC = 32768;
  static constexpr int kTotal = kOffC + kC;
  static constexpr int kAlloc = kTotal + 1024;  // slack to realign the base to 1024 B
  static_assert(kAlloc <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

template <int KIND, int TILE_N, int STAGES>
__global__ void __launch_bounds__(Smem<TILE_N, STAGES>::kThreads, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using L = Smem<TILE_N, STAGES>;
  constexpr int kSub = L::kSub;
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr int kAccBufs = (TILE_N == 128) ? 2 : 1;
  constexpr int kSfaCols = 16;             // 4 MMAs x 4 columns (NVFP4); MXFP8 uses 4
  constexpr int kSfbCols = 16 * kSub;
  constexpr int kSlotCols = kSfaCols + kSfbCols;
  constexpr int kSfCol0 = kAccBufs * TILE_N;
  constexpr int kSfSlots = (512 - kSfCol0) / kSlotCols >= 4 ? 4 : (512 - kSfCol0) / kSlotCols;
  static_assert(kSfSlots >= 1, "no TMEM left for scale factors");
  constexpr int kChunksPerStage = (KIND == KIND_NVFP4) ? 4 : 1;
  constexpr uint32_t kIdescBase =
      (KIND == KIND_NVFP4)
          ? ((1u << 7) | (1u << 10) | (uint32_t(TILE_N >> 3) << 17) | (8u << 24))
          : ((uint32_t(TILE_N >> 3) << 17) | (1u << 23) | (8u << 24));

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);

  // header: barriers, TMEM base pointer, abort flag
  const uint32_t bar_full = sbase;                        // STAGES x 8
  const uint32_t bar_empty = sbase + 8 * STAGES;          // STAGES x 8
  const uint32_t bar_acc_full = sbase + 16 * STAGES;      // 2 x 8
  const uint32_t bar_acc_empty = bar_acc_full + 16;       // 2 x 8
  const uint32_t bar_drain = bar_acc_empty + 16;          // 1 x 8
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + 512);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + 516);

  // broadcast from lane 0 so the compiler knows the role index is warp-uniform and keeps the
  // role bodies (and the operands of their asynchronous instructions) on the uniform path
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int ntiles = p.n / TILE_N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, L::kEpiWarps);
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  // set-up done; wait for the previous kernel in the stream before touching global memory
  // (a no-op unless launched with programmatic stream serialization) and let the next one in
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

  // The producer and MMA warps run their loops with all 32 lanes converged and issue each
  // asynchronous instruction from one elected lane: operands then stay warp-uniform, which
  // is what keeps the issue cost of TMA / tcgen05 instructions low.
  if (warp == kProducerWarp) {
    // ------------------------------ producer ------------------------------------
    TileCursor cur;
    int it = 0, tl = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok; t += gridDim.x, ++tl) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      const int row0 = cur.off + mt * 128;
      const int brow0 = cur.g * p.n + nt * TILE_N;
      const uint8_t* sfa_src = p.sfa + (size_t)(row0 >> 7) * p.sf_chunks * 512;
      const uint8_t* sfb_src =
          p.sfb + ((size_t)cur.g * (p.n >> 7) + (size_t)nt * kSub) * p.sf_chunks * 512;
      MSC_STAMP(0, tl, 0);
      for (int kb = 0; kb < p.k_stages; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (lane == 0) MSC_FINE(0);
        ok = warp_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        if (lane == 0) MSC_FINE(1);
        const int c0 = kb * kChunksPerStage;
        const int nch = min(kChunksPerStage, p.sf_chunks - c0);
        const uint32_t full = bar_full + 8 * s;
        if (elect_one()) {
          if (MSC_FLAG(8)) {
            mbar_arrive(full);
          } else {
            mbar_arrive_expect_tx(full, L::kA + L::kB + (1 + kSub) * nch * 512);
            tma_load_2d(sbase + L::kOffA + s * L::kA, &tmap_a, full, kb * 128, row0);
            tma_load_2d(sbase + L::kOffB + s * L::kB, &tmap_b, full, kb * 128, brow0);
            bulk_load_1d(sbase + L::kOffSfa + s * L::kSfa, sfa_src + (size_t)c0 * 512, nch * 512,
                         full);
#pragma unroll
            for (int sub = 0; sub < kSub; ++sub)
              bulk_load_1d(sbase + L::kOffSfb + s * L::kSfb + sub * 2048,
                           sfb_src + ((size_t)sub * p.sf_chunks + c0) * 512, nch * 512, full);
          }
          MSC_FINE(2);
        }
        __syncwarp();
        if (lane == 0) MSC_FINE(3);
      }
      MSC_STAMP(0, tl, 1);
    }
    if (*abort_flag && lane == 0) {
      // wait (bounded) for the loads still in flight so none lands after the CTA exits
      for (int j = max(0, it - STAGES); j < it; ++j)
        mbar_wait_drain(bar_full + 8 * (j % STAGES), (j / STAGES) & 1);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ----------------------------------
    // The tensor pipe takes instructions through a shallow queue, so it idles whenever this
    // warp spends long between MMAs.  The loop is therefore software-pipelined: the wait for
    // the NEXT stage's operands and the issue of its scale copies sit between the second and
    // third MMA of the CURRENT stage, where two queued MMAs cover their latency.  Stage
    // index, parity and descriptor words are stepped, never divided.
    TileCursor cur;
    int tl = 0;
    uint32_t s = 0, ph = 0, slot = 0;
    bool ok = true;
    const uint64_t adesc0 = operand_desc_sw128(sbase + L::kOffA);
    const uint64_t bdesc0 = operand_desc_sw128(sbase + L::kOffB);
    const uint64_t sfa_d0 = scale_desc(sbase + L::kOffSfa);
    const uint64_t sfb_d0 = scale_desc(sbase + L::kOffSfb);
    // descriptor low words count 16-byte units: +32 per 512-byte scale chunk, +128 per
    // 2048-byte sub-tile block, +2 per 32 bytes of K inside the swizzled operand tile
    auto copy_scales = [&](uint32_t st, uint32_t sl, int nch) {
      const uint32_t sfa_t = tmem_base + kSfCol0 + sl * kSlotCols;
      const uint32_t sfb_t = sfa_t + kSfaCols;
      const uint64_t sfa_d = sfa_d0 + st * (L::kSfa >> 4);
      const uint64_t sfb_d = sfb_d0 + st * (L::kSfb >> 4);
      if (MSC_FLAG(2)) return;
#pragma unroll
      for (int c = 0; c < kChunksPerStage; ++c) {
        if (c < nch) {
          tc_cp_32x128b_warpx4(sfa_t + 4 * c, sfa_d + 32 * c);
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub)
            tc_cp_32x128b_warpx4(sfb_t + 4 * kSub * c + 4 * sub, sfb_d + 128 * sub + 32 * c);
        }
      }
    };
    auto mma = [&](uint32_t acc, uint32_t st, uint32_t sl, int j, uint32_t accumulate) {
      const uint32_t sfa_t = tmem_base + kSfCol0 + sl * kSlotCols;
      const uint32_t sfb_t = sfa_t + kSfaCols;
      const uint64_t adesc = adesc0 + st * (L::kA >> 4) + 2 * j;
      const uint64_t bdesc = bdesc0 + st * (L::kB >> 4) + 2 * j;
      if (MSC_FLAG(4)) return;
      if (KIND == KIND_NVFP4) {
        tc_mma_nvfp4(acc, adesc, bdesc, kIdescBase, sfa_t + 4 * j, sfb_t + 4 * kSub * j, accumulate);
      } else {
        const uint32_t idesc = kIdescBase | (uint32_t(j) << 29) | (uint32_t(j) << 4);
        tc_mma_mxf8(acc, adesc, bdesc, idesc, sfa_t, sfb_t, accumulate);
      }
    };
    const int nch_first = min(kChunksPerStage, p.sf_chunks);
    bool primed = false;  // scale copies of the stage about to be consumed already issued
    for (int t = blockIdx.x; ok; t += gridDim.x, ++tl) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      TileCursor peek = cur;
      int mt2, nt2;
      const bool more_tiles = peek.seek(p, ntiles, t + gridDim.x, mt2, nt2);
      if (!primed) {
        ok = warp_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3);
        if (!ok) break;
        tc_fence_after_sync();
        if (elect_one()) copy_scales(s, slot, nch_first);
        primed = true;
      }
      const int buf = tl % kAccBufs;
      const uint32_t aph = (tl / kAccBufs) & 1;
      ok = warp_wait(bar_acc_empty + 8 * buf, aph ^ 1u, abort_flag, p.status, 2);
      if (!ok) break;
      tc_fence_after_sync();
      MSC_STAMP(1, tl, 0);
      const uint32_t acc = tmem_base + buf * TILE_N;
      for (int kb = 0; kb < p.k_stages; ++kb) {
        if (lane == 0) MSC_FINE(8);
        const int nch = min(kChunksPerStage, p.sf_chunks - kb * kChunksPerStage);
        const int nmma = (KIND == KIND_NVFP4) ? nch : 4;
        const bool last_kb = kb + 1 == p.k_stages;
        const bool has_next = !last_kb || more_tiles;
        const int nch_next =
            last_kb ? nch_first : min(kChunksPerStage, p.sf_chunks - (kb + 1) * kChunksPerStage);
        const uint32_t s_next = (s + 1 == STAGES) ? 0u : s + 1;
        const uint32_t ph_next = (s + 1 == STAGES) ? ph ^ 1u : ph;
        const uint32_t slot_next = (slot + 1 == kSfSlots) ? 0u : slot + 1;
        if (elect_one()) {
          mma(acc, s, slot, 0, kb > 0 ? 1u : 0u);
          if (nmma > 1) mma(acc, s, slot, 1, 1u);
        }
        if (lane == 0) MSC_FINE(9);
        if (has_next) {
          const bool ready = mbar_test(bar_full + 8 * s_next, ph_next);
          if (!__all_sync(0xffffffffu, ready)) {
            ok = warp_wait(bar_full + 8 * s_next, ph_next, abort_flag, p.status, 3);
            if (!ok) break;
          }
          tc_fence_after_sync();
        }
        if (lane == 0) MSC_FINE(10);
        if (elect_one()) {
          if (has_next) copy_scales(s_next, slot_next, nch_next);
          MSC_FINE(11);
          if (nmma > 2) mma(acc, s, slot, 2, 1u);
          if (nmma > 3) mma(acc, s, slot, 3, 1u);
          MSC_FINE(12);
          tc_commit(bar_empty + 8 * s);  // frees the smem stage once these MMAs have read it
          MSC_FINE(13);
        }
        if (lane == 0) MSC_FINE(15);
        s = s_next;
        ph = ph_next;
        slot = slot_next;
      }
      if (ok && elect_one()) tc_commit(bar_acc_full + 8 * buf);
      MSC_STAMP(1, tl, 1);
    }
    __syncwarp();
    if (*abort_flag && lane == 0) {
      tc_commit(bar_drain);
      mbar_wait_drain(bar_drain, 0);
    }
  } else {
    // ------------------------------ epilogue ------------------------------------
    // Warp w owns TMEM lane quadrant w % 4 (32 accumulator rows) and the 128-column slab
    // w / 4 of the tile.  It pulls its 32 x 128 fp32 block into registers in one go and
    // hands the accumulator back to the MMA warp as soon as those loads land; then, 64
    // columns at a time: scale, round to bf16, park the rows in its shared-memory staging
    // box in the 128-byte-swizzled layout and let one lane issue a TMA store of the box.
    // A warp whose 32 rows are not all valid (the ragged end of a group) writes its valid
    // rows with plain 16-byte stores instead, so rows past masked_m are never touched.
    TileCursor cur;
    int tl = 0;
    const int quad = warp & 3;
    const int slab = warp >> 2;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t stage_c = sbase + L::kOffC + warp * L::kCPerWarp;
    constexpr bool kTwoBoxes = (L::kCPerWarp == 8192);
    for (int t = blockIdx.x;; t += gridDim.x, ++tl) {
      int mt, nt;
      if (!cur.seek(p, ntiles, t, mt, nt)) break;
      const int buf = tl % kAccBufs;
      const uint32_t aph = (tl / kAccBufs) & 1;
      // one lane per warp waits; the others park on the warp vote instead of polling
      bool ok = true;
      if (lane == 0) ok = mbar_wait_bounded(bar_acc_full + 8 * buf, aph, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 0) MSC_STAMP(2, tl, 0);
      const int row_warp = mt * 128 + quad * 32;
      const bool valid = row_warp + lane < cur.rows;
      const bool whole_warp = row_warp + 32 <= cur.rows;
      const size_t out_row = (size_t)cur.off + row_warp + lane;
      float scale = p.alpha ? __ldg(p.alpha + cur.g) : 1.0f;
      if (p.row_scale && valid) scale *= __ldg(p.row_scale + out_row);

      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld_32x32b_x32(tmem_base + lane_base + buf * TILE_N + slab * 128 + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      if (warp == 0) MSC_STAMP(2, tl, 1);
      if (MSC_FLAG(1)) continue;

      const int col0 = nt * TILE_N + slab * 128;
      if (whole_warp) {
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const uint32_t box = stage_c + (kTwoBoxes ? sub * 4096 : 0);
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
              // row = lane; 16-byte chunk j of the 128-byte row sits at j ^ (row & 7)
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
    if (lane == 0) bulk_wait_group_read0();  // staging area must outlive the stores that read it
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
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------- host side -------------------------------------------

template <int KIND, int TILE_N, int STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                  const GemmParams& p, int grid, cudaStream_t stream) {
  using L = Smem<TILE_N, STAGES>;
  auto kern = gemm_blockscaled_kernel<KIND, TILE_N, STAGES>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc = pdl_launch_config(grid, L::kThreads, L::kAlloc, stream, attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
  return MSC_OK;
}

template <int KIND, int TILE_N>
static int pick_stages(int stages, const CUtensorMap& ta, const CUtensorMap& tb,
                       const CUtensorMap& tc, const GemmParams& p, int grid, cudaStream_t stream) {
  constexpr int kMax = (TILE_N == 128) ? 5 : 3;  // what fits beside the 32 KB staging area
  if (stages <= 0 || stages > kMax) stages = kMax;
  switch (stages) {
    case 2: return launch<KIND, TILE_N, 2>(ta, tb, tc, p, grid, stream);
    case 3: return launch<KIND, TILE_N, 3>(ta, tb, tc, p, grid, stream);
    case 4:
      if constexpr (TILE_N == 128) return launch<KIND, TILE_N, 4>(ta, tb, tc, p, grid, stream);
      break;
    case 5:
      if constexpr (TILE_N == 128) return launch<KIND, TILE_N, 5>(ta, tb, tc, p, grid, stream);
      break;
    default: break;
  }
  return fail(MSC_ERR_UNSUPPORTED, "stages=%d is not built for tile_n=%d", stages, TILE_N);
}

// Shared body of the three entry points.  k_bytes: bytes of K per row; chunk_elems: K
// elements one 512-byte scale chunk covers.
static int grouped_gemm(int kind, const void* a_q, const void* a_sf, const void* b_q,
                        const void* b_sf, const float* alpha, const int32_t* group_offsets,
                        const int32_t* group_rows, const float* row_scale, void* out, int l,
                        long long rows_total, int m_stride, int n, int k,
                        const msc_gemm_cfg* cfg_in, void* stream_v) {
  msc_gemm_cfg cfg = {};
  if (cfg_in) cfg = *cfg_in;
  if (!a_q || !a_sf || !b_q || !b_sf || !out) return fail(MSC_ERR_BAD_ARG, "NULL operand pointer");
  if (l <= 0 || rows_total <= 0 || n <= 0 || k <= 0)
    return fail(MSC_ERR_BAD_ARG, "l, rows, n, k must be positive");
  const int tile_n = cfg.tile_n ? cfg.tile_n : 128;
  if (tile_n != 128 && tile_n != 256)
    return fail(MSC_ERR_UNSUPPORTED, "tile_n must be 128 or 256, got %d", tile_n);
  if (n % tile_n) return fail(MSC_ERR_BAD_ARG, "n=%d must be a multiple of tile_n=%d", n, tile_n);
  const int chunk_elems = (kind == KIND_NVFP4) ? 64 : 128;
  if (k % chunk_elems)
    return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of %d", k, chunk_elems);
  if (cfg.cta_pair < 0 || cfg.cta_pair > 3)
    return fail(MSC_ERR_BAD_ARG, "cta_pair must be 0 (auto), 1 (pair), 2 (single CTA) or 3 (pair, tokens on N)");
  if (cfg.cta_pair == 3 && (!group_offsets || !group_rows))
    return fail(MSC_ERR_UNSUPPORTED, "cta_pair=3 (tokens on N) is built for row-concatenated groups");
  if (cfg.epilogue != MSC_EPI_PLAIN && cfg.epilogue != MSC_EPI_ROW_SCALE)
    return fail(MSC_ERR_UNSUPPORTED, "unknown epilogue %d", cfg.epilogue);
  if (cfg.epilogue == MSC_EPI_ROW_SCALE && !row_scale)
    return fail(MSC_ERR_BAD_ARG, "MSC_EPI_ROW_SCALE needs row_scale");
  if (reinterpret_cast<uintptr_t>(a_sf) % 16 || reinterpret_cast<uintptr_t>(b_sf) % 16 ||
      reinterpret_cast<uintptr_t>(out) % 16)
    return fail(MSC_ERR_BAD_ARG, "scale and output pointers must be 16-byte aligned");
  const long long k_bytes = (kind == KIND_NVFP4) ? k / 2 : k;

  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");

  CUtensorMap ta, tb, tc;
  int rc = make_tmap_bytes_2d(&ta, a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&tb, b_q, (uint64_t)l * n, (uint64_t)k_bytes, (uint32_t)tile_n);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tc, out, (uint64_t)rows_total, (uint64_t)n, 32);
  if (rc) return rc;

  GemmParams p;
  p.sfa = static_cast<const uint8_t*>(a_sf);
  p.sfb = static_cast<const uint8_t*>(b_sf);
  p.alpha = alpha;
  p.row_scale = (cfg.epilogue == MSC_EPI_ROW_SCALE) ? row_scale : nullptr;
  p.group_rows = group_rows;
  p.group_offsets = group_offsets;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.l = l;
  p.m_stride = m_stride;
  p.rows_total = (int)rows_total;
  p.n = n;
  p.k_stages = (int)((k_bytes + 127) / 128);
  p.sf_chunks = k / chunk_elems;
  p.raster = cfg.raster ? 1 : 0;
  p.out_q = nullptr;
  p.out_sf = nullptr;
  p.out_gs = nullptr;
  p.row_dest = nullptr;
  p.scatter_count = p.scatter_rows = 0;
  for (auto& b : p.scatter_base) b = nullptr;
#ifdef MSC_DEBUG
  p.trace = g_trace;
  p.debug_flags = g_debug_flags;
#endif

  // 0 = choose.  Row-concatenated groups of a few hundred rows with a long contraction go to the
  // tokens-on-N kernel: a group's tail costs it a slightly wider tile instead of a second one,
  // and from 1 KB of K per row on its transposing epilogue fits under the K loop (measured on
  // 256 groups of 256 +- 16 rows: -10 % at k_bytes = 1 KB, -7 % at 3.5 KB; -3 % on the Zipf
  // MXFP8 benchmark; groups of exactly 256 rows pay 4 - 6 %).
  const bool swap_auto = cfg.cta_pair == 0 && cfg.tile_n == 0 && group_offsets && group_rows && n % 256 == 0 &&
                         k_bytes >= 1024 && rows_total / l <= 640;
  if (cfg.cta_pair == 3 || swap_auto)
    return launch_swap_gemm(kind, a_q, b_q, rows_total, k_bytes, p, cfg.max_ctas, static_cast<cudaStream_t>(stream_v));
  // 0 = choose: pairs pay off when whole 256-row tiles are common and n allows 256-wide tiles
  bool pair = cfg.cta_pair == 1;
  if (cfg.cta_pair == 0 && cfg.tile_n == 0)
    pair = (n % 256 == 0) && ((m_stride > 0 ? m_stride : rows_total / l) >= 256);
  if (pair)
    return launch_pair_gemm(kind, a_q, b_q, rows_total, k_bytes, p, cfg.stages, cfg.max_ctas,
                            static_cast<cudaStream_t>(stream_v), cfg.sf_warps == 1);

  const long long max_tiles = ((rows_total + 127) / 128 + l) * (long long)(n / tile_n);
  int grid = cfg.max_ctas > 0 ? cfg.max_ctas : num_sms();
  if (grid <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  if (grid > max_tiles) grid = (int)max_tiles;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  if (kind == KIND_NVFP4) {
    if (tile_n == 128) return pick_stages<KIND_NVFP4, 128>(cfg.stages, ta, tb, tc, p, grid, stream);
    return pick_stages<KIND_NVFP4, 256>(cfg.stages, ta, tb, tc, p, grid, stream);
  }
  if (tile_n == 128) return pick_stages<KIND_MXFP8, 128>(cfg.stages, ta, tb, tc, p, grid, stream);
  return pick_stages<KIND_MXFP8, 256>(cfg.stages, ta, tb, tc, p, grid, stream);
}

}  // namespace msc

extern "C" {

#ifdef MSC_DEBUG
// Debug builds only: device buffer for per-tile clock stamps and pipeline-stage skip flags.
int msc_debug_config(void* trace, int flags) {
  msc::g_trace = static_cast<unsigned long long*>(trace);
  msc::g_debug_flags = flags;
  return MSC_OK;
}
#endif

int msc_grouped_gemm_nvfp4(const void* a_q, const void* a_sf, const void* b_q, const void* b_sf,
                           const float* alpha, const int32_t* masked_m, void* out, int l, int m,
                           int n, int k, const msc_gemm_cfg* cfg, void* stream) {
  if (m <= 0 || m % 128) return msc::fail(MSC_ERR_BAD_ARG, "m=%d must be a positive multiple of 128", m);
  if (cfg && cfg->epilogue != MSC_EPI_PLAIN)
    return msc::fail(MSC_ERR_UNSUPPORTED, "the masked form takes MSC_EPI_PLAIN only");
  return msc::grouped_gemm(msc::KIND_NVFP4, a_q, a_sf, b_q, b_sf, alpha, nullptr, masked_m, nullptr,
                           out, l, (long long)l * m, m, n, k, cfg, stream);
}

int msc_grouped_gemm_nvfp4_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                  const void* b_sf, const float* alpha,
                                  const int32_t* group_offsets, const int32_t* group_rows,
                                  const float* row_scale, void* out, int l, int rows_total, int n,
                                  int k, const msc_gemm_cfg* cfg, void* stream) {
  if (!group_offsets || !group_rows)
    return msc::fail(MSC_ERR_BAD_ARG, "group_offsets and group_rows are required");
  return msc::grouped_gemm(msc::KIND_NVFP4, a_q, a_sf, b_q, b_sf, alpha, group_offsets, group_rows,
                           row_scale, out, l, rows_total, 0, n, k, cfg, stream);
}

int msc_grouped_gemm_nvfp4_swiglu_ragged(const void* a_q, const void* a_sf, const void* w1_q,
                                         const void* w1_sf, const float* alpha,
                                         const int32_t* group_offsets, const int32_t* group_rows,
                                         const float* out_global_scale, void* d_q, void* d_sf, int l,
                                         int rows_total, int n2, int k, const msc_gemm_cfg* cfg,
                                         void* stream) {
  using namespace msc;
  if (!a_q || !a_sf || !w1_q || !w1_sf || !group_offsets || !group_rows || !out_global_scale || !d_q || !d_sf)
    return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (l <= 0 || rows_total <= 0 || n2 <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (n2 % 256) return fail(MSC_ERR_BAD_ARG, "n2=%d (gate + up rows) must be a multiple of 256", n2);
  if (k % 64) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 64", k);
  if (reinterpret_cast<uintptr_t>(d_q) % 16 || reinterpret_cast<uintptr_t>(d_sf) % 4)
    return fail(MSC_ERR_BAD_ARG, "d_q must be 16-byte aligned, d_sf 4-byte aligned");
  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");
  GemmParams p;
  p.sfa = static_cast<const uint8_t*>(a_sf);
  p.sfb = static_cast<const uint8_t*>(w1_sf);
  p.alpha = alpha;
  p.row_scale = nullptr;
  p.group_rows = group_rows;
  p.group_offsets = group_offsets;
  p.out = nullptr;
  p.status = status;
  p.l = l;
  p.m_stride = 0;
  p.rows_total = rows_total;
  p.n = n2;
  p.k_stages = (k / 2 + 127) / 128;
  p.sf_chunks = k / 64;
  p.raster = 0;
  p.out_q = static_cast<uint8_t*>(d_q);
  p.out_sf = static_cast<uint8_t*>(d_sf);
  p.out_gs = out_global_scale;
  p.row_dest = nullptr;
  p.scatter_count = p.scatter_rows = 0;
  for (auto& b : p.scatter_base) b = nullptr;
#ifdef MSC_DEBUG
  p.trace = g_trace;
  p.debug_flags = g_debug_flags;
#endif
  if (cfg && cfg->cta_pair == 3)   // tokens on N: w1 comes interleaved (msc_swiglu_interleave_w1)
    return launch_swap_gemm(KIND_NVFP4, a_q, w1_q, rows_total, k / 2, p, cfg->max_ctas, static_cast<cudaStream_t>(stream));
  return launch_pair_gemm(KIND_NVFP4, a_q, w1_q, rows_total, k / 2, p, cfg ? cfg->stages : 0,
                          cfg ? cfg->max_ctas : 0, static_cast<cudaStream_t>(stream), false);
}

int msc_grouped_gemm_nvfp4_scatter_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                          const void* b_sf, const float* alpha,
                                          const int32_t* group_offsets, const int32_t* group_rows,
                                          const float* row_scale, const int32_t* row_dest,
                                          void* const* dest_bases, int dest_count, int dest_rows,
                                          int l, int rows_total, int n, int k,
                                          const msc_gemm_cfg* cfg, void* stream) {
  using namespace msc;
  if (!a_q || !a_sf || !b_q || !b_sf || !group_offsets || !group_rows || !row_dest || !dest_bases)
    return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (dest_count < 1 || dest_count > 16)
    return fail(MSC_ERR_UNSUPPORTED, "dest_count=%d must be in [1, 16]", dest_count);
  if (dest_rows < 1 || dest_rows > 0x04000000)
    return fail(MSC_ERR_BAD_ARG, "dest_rows=%d must be in [1, 2^26]", dest_rows);
  if (l <= 0 || rows_total <= 0 || n <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (n % 256) return fail(MSC_ERR_BAD_ARG, "n=%d must be a multiple of 256", n);
  if (k % 64) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 64", k);
  if (reinterpret_cast<uintptr_t>(a_sf) % 16 || reinterpret_cast<uintptr_t>(b_sf) % 16)
    return fail(MSC_ERR_BAD_ARG, "scale pointers must be 16-byte aligned");
  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");
  GemmParams p;
  p.sfa = static_cast<const uint8_t*>(a_sf);
  p.sfb = static_cast<const uint8_t*>(b_sf);
  p.alpha = alpha;
  p.row_scale = row_scale;
  p.group_rows = group_rows;
  p.group_offsets = group_offsets;
  p.out = nullptr;
  p.status = status;
  p.l = l;
  p.m_stride = 0;
  p.rows_total = rows_total;
  p.n = n;
  p.k_stages = (k / 2 + 127) / 128;
  p.sf_chunks = k / 64;
  p.raster = 0;
  p.out_q = nullptr;
  p.out_sf = nullptr;
  p.out_gs = nullptr;
  p.row_dest = row_dest;
  p.scatter_count = dest_count;
  p.scatter_rows = dest_rows;
  for (int i = 0; i < 16; ++i) {
    p.scatter_base[i] = i < dest_count ? static_cast<uint8_t*>(dest_bases[i]) : nullptr;
    if (i < dest_count && (!dest_bases[i] || reinterpret_cast<uintptr_t>(dest_bases[i]) % 16))
      return fail(MSC_ERR_BAD_ARG, "destination %d must be a 16-byte aligned device pointer", i);
  }
#ifdef MSC_DEBUG
  p.trace = g_trace;
  p.debug_flags = g_debug_flags;
#endif
  return launch_pair_gemm(KIND_NVFP4, a_q, b_q, rows_total, k / 2, p, 4, cfg ? cfg->max_ctas : 0,
                          static_cast<cudaStream_t>(stream), false);
}

int msc_grouped_gemm_mxfp8_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                  const void* b_sf, const float* alpha,
                                  const int32_t* group_offsets, const int32_t* group_rows,
                                  const float* row_scale, void* out, int l, int rows_total, int n,
                                  int k, const msc_gemm_cfg* cfg, void* stream) {
  if (!group_offsets || !group_rows)
    return msc::fail(MSC_ERR_BAD_ARG, "group_offsets and group_rows are required");
  return msc::grouped_gemm(msc::KIND_MXFP8, a_q, a_sf, b_q, b_sf, alpha, group_offsets, group_rows,
                           row_scale, out, l, rows_total, 0, n, k, cfg, stream);
}

}  // extern "C"
