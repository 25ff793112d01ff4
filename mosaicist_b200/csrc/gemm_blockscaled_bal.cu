// Block-scaled NVFP4 grouped GEMM on CTA pairs with a balanced schedule and two accumulators.
//
// The kernel of gemm_blockscaled_pair.cu gives every CTA pair whole 256 x 256 tiles.  At the
// headline shape (8 groups x 512 x 2048, k = 2048) that is 128 tiles on 74 pairs: 20 pairs get
// one tile, the others two, and the pair with two waits for the first tile's accumulator to
// drain before it starts the second.  This kernel cuts the work at a finer grain:
//
//   * the output is measured in UNITS of 256 rows x 64 columns; the units of all groups, in
//     (group, row tile, column) order, are dealt out in equal contiguous runs, one per pair
//     (7 units = 448 columns at the headline shape: 73 pairs busy to the same degree);
//   * a run is cut into tiles of 64, 128, 192 or 256 columns (one tcgen05.mma N each).  A tile
//     may start on an odd multiple of 64 columns: its B scales are then fetched from the
//     128-row chunk it starts in and the MMA reads them two tensor-memory columns further on
//     (a column holds the scales of 32 rows);
//   * tensor memory holds TWO accumulators (columns 0-255 and 256-447) and one 48-column
//     staging area for a K stage's scale factors (columns 448-495), reused every stage: the
//     copies and the MMAs that read them are issued by one thread, in order.  While the
//     epilogue warps drain one accumulator the MMA warp fills the other.
//
// Roles, barriers, operand layout and arithmetic are those of the pair kernel: 8 epilogue
// warps, one MMA warp (leader CTA only), one TMA producer warp per CTA; no load is multicast.
// Results are bit-identical to the other kernels (same products, same fp32 accumulation order
// along K, same rounding).
#include "gemm_common.cuh"

namespace msc {

template <int STAGES>
struct BalSmem {
  static constexpr int kHeader = 1024;
  static constexpr int kA = 128 * 128;
  static constexpr int kB = 128 * 128;       // up to 128 of the tile's (up to 256) B rows
  static constexpr int kSfa = 4 * 512;
  static constexpr int kSfb = 2 * 4 * 512;   // the two 128-row scale chunks a tile can touch
  static constexpr int kOffA = kHeader;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffSfa = kOffB + STAGES * kB;
  static constexpr int kOffSfb = kOffSfa + STAGES * kSfa;
  static constexpr int kOffC = kOffSfb + STAGES * kSfb;
  static constexpr int kEpiWarps = 8;
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
  static constexpr int kCBox = 32 * 64;      // 32 rows x 32 bf16 columns, 64-byte swizzle
  static constexpr int kCPerWarp = 2 * kCBox;
  static constexpr int kTotal = kOffC + kEpiWarps * kCPerWarp;
  static constexpr int kAlloc = kTotal + 1024;
  static_assert(kAlloc <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

constexpr int kBalAcc1Col = 256;   // second accumulator: 192 columns
constexpr int kBalSfCol = 448;     // scale staging: 16 columns of A scales, 32 of B scales

// One tile of a pair's run.
struct BalTile {
  int g, mt;        // group, 256-row tile inside it
  int rows, off;    // the group's row count and first row
  int n0, w;        // first column, width in units of 64 columns (1..4)
  int slot;         // accumulator: 0 (columns 0-255) or 1 (columns 256-447, at most 192 wide)
};

// Walks a pair's run of units, tile by tile.  Every role warp of both CTAs runs the same walk
// and arrives at the same tiles.
struct BalWalker {
  int u = 0, u_end = 0, units_n = 1;
  int prev_slot = -1;
  int g = 0, slab_base = 0, mtiles = 0, rows = 0, off = 0;
  bool primed = false;

  // rows and first row of group g, cut to what the buffers hold (as TileCursor does)
  static __device__ __forceinline__ void group_extent(const GemmParams& p, int g, int& rows, int& off) {
    rows = p.group_rows ? __ldg(p.group_rows + g) : p.m_stride;
    if (rows < 0) rows = 0;
    if (p.m_stride > 0 && rows > p.m_stride) rows = p.m_stride;
    off = p.group_offsets ? __ldg(p.group_offsets + g) : g * p.m_stride;
    if (off < 0 || off >= p.rows_total) rows = 0;
    else if (rows > p.rows_total - off) rows = p.rows_total - off;
  }

  __device__ __forceinline__ void init(const GemmParams& p, int pair, int npairs) {
    const int lane = threadIdx.x & 31;
    int slabs = 0;
    for (int i = lane; i < p.l; i += 32) {
      int r, o;
      group_extent(p, i, r, o);
      slabs += (r + 255) >> 8;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) slabs += __shfl_xor_sync(0xffffffffu, slabs, d);
    units_n = p.n >> 6;
    const long long total = (long long)slabs * units_n;
    const long long q = (total + npairs - 1) / npairs;
    const long long first = q * pair;
    u = (int)(first < total ? first : total);
    u_end = (int)(first + q < total ? first + q : total);
  }

  __device__ __forceinline__ bool next(const GemmParams& p, BalTile& t) {
    if (u >= u_end) return false;
    const int slab = u / units_n;
    const int nu = u - slab * units_n;
    while (true) {
      if (!primed) {
        int r = 0, o = 0;
        if ((threadIdx.x & 31) == 0) group_extent(p, g, r, o);
        rows = __shfl_sync(0xffffffffu, r, 0);
        off = __shfl_sync(0xffffffffu, o, 0);
        mtiles = (rows + 255) >> 8;
        primed = true;
      }
      if (slab < slab_base + mtiles) break;
      slab_base += mtiles;
      ++g;
      primed = false;
    }
    const int left = min(u_end - u, units_n - nu);   // units left in this run and this row tile
    const bool odd = nu & 1;
    // accumulator 0 holds up to 4 units, accumulator 1 up to 3; a tile that starts on an odd
    // unit spans at most 3 (its scales must fit the two chunks fetched per stage).  Tiles
    // alternate between the accumulators so that one drains while the other fills.
    int cap = odd ? 3 : 4;
    if (prev_slot == 0) cap = min(cap, 3);
    int w;
    if (left <= cap) w = left;
    else if (cap == 4) w = (left == 5) ? 3 : 4;      // 5 = 3 + 2 rather than 4 + 1
    else w = (left == 4) ? 2 : 3;                    // 4 = 2 + 2 rather than 3 + 1
    t.g = g;
    t.mt = slab - slab_base;
    t.rows = rows;
    t.off = off;
    t.n0 = nu << 6;
    t.w = w;
    t.slot = (w == 4) ? 0 : (prev_slot == 1 ? 0 : 1);
    prev_slot = t.slot;
    u += w;
    return true;
  }
};

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BalSmem<STAGES>::kThreads, 1)
gemm_bal_kernel(const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_sfa,
                const __grid_constant__ CUtensorMap tmap_sfb,
                const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using L = BalSmem<STAGES>;
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr int kSfaCols = 16;
  constexpr uint32_t kSfBoxBytes = 4 * 512;
  // instruction descriptor without N: e2m1 x e2m1, ue4m3 scales, M = 256 over the pair
  constexpr uint32_t kIdescBase = (1u << 7) | (1u << 10) | (16u << 24);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);

  const uint32_t bar_full = sbase;                      // STAGES x 8 (used in the leader)
  const uint32_t bar_empty = sbase + 8 * STAGES;        // STAGES x 8
  const uint32_t bar_acc_full = sbase + 16 * STAGES;    // 2 x 8
  const uint32_t bar_acc_empty = bar_acc_full + 16;     // 2 x 8 (used in the leader)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + 512);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + 516);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);
      mbar_init(bar_acc_empty + 8 * a, 2 * L::kEpiWarps);
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
  // set-up is done: from here on global memory is touched (the group table first), so wait for
  // the previous kernel in the stream and let the next one begin its own set-up
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
    BalWalker walk;
    walk.init(p, pair, npairs);
    BalTile t;
    uint32_t bits = 0;  // per-stage use parity
    uint32_t s = 0;
    bool ok = true;
    int tl = 0;
    while (ok && walk.next(p, t)) {
      const int row0 = t.off + (2 * t.mt + (int)rank) * 128;
      const int brows = 32 * t.w;                                  // this CTA's half of the tile's B rows
      const int brow0 = t.g * p.n + t.n0 + (int)rank * brows;
      const int sfa_row = (row0 >> 7) * p.sf_chunks * 4;
      const int sfb_row = (t.g * (p.n >> 7) + (t.n0 >> 7)) * p.sf_chunks * 4;
      const int sfb_row1 = sfb_row + p.sf_chunks * 4;
      const uint32_t stage_bytes = 2u * (L::kA + (uint32_t)brows * 128u + 3u * kSfBoxBytes);
      MSC_STAMP(0, tl, 0);
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_empty + 8 * s, ((bits >> s) & 1u) ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t full = bar_full + 8 * s;
        const int c4 = kb * 16;
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(full, stage_bytes);
          tma_load_2d_pair(sbase + L::kOffA + s * L::kA, &tmap_a, full, kb * 128, row0);
          for (int i = 0; i < t.w; ++i)
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB + i * 4096, &tmap_b, full, kb * 128,
                             brow0 + 32 * i);
          tma_load_2d_pair(sbase + L::kOffSfa + s * L::kSfa, &tmap_sfa, full, 0, sfa_row + c4);
          tma_load_2d_pair(sbase + L::kOffSfb + s * L::kSfb, &tmap_sfb, full, 0, sfb_row + c4);
          tma_load_2d_pair(sbase + L::kOffSfb + s * L::kSfb + 2048, &tmap_sfb, full, 0, sfb_row1 + c4);
        }
        __syncwarp();
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
      MSC_STAMP(0, tl, 1);
      ++tl;
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer (leader only) --------------------
    if (leader) {
      BalWalker walk;
      walk.init(p, pair, npairs);
      BalTile t;
      uint32_t bits = 0, acc_uses = 0;   // acc_uses bit a: parity of the times accumulator a was filled
      uint32_t s = 0;
      int tl = 0;
      bool ok = true;
      const uint64_t adesc0 = operand_desc_sw128(sbase + L::kOffA);
      const uint64_t bdesc0 = operand_desc_sw128(sbase + L::kOffB);
      const uint64_t sfa_d0 = scale_desc(sbase + L::kOffSfa);
      const uint64_t sfb_d0 = scale_desc(sbase + L::kOffSfb);
      const uint32_t sfa_t = tmem_base + kBalSfCol;
      const uint32_t sfb_t0 = sfa_t + kSfaCols;
      while (ok && walk.next(p, t)) {
        const uint32_t a = (uint32_t)t.slot;
        ok = warp_wait(bar_acc_empty + 8 * a, ((acc_uses >> a) & 1u) ^ 1u, abort_flag, p.status, 2);
        if (!ok) break;
        acc_uses ^= 1u << a;
        tc_fence_after_sync();
        MSC_STAMP(1, tl, 0);
        const uint32_t acc = tmem_base + (a ? kBalAcc1Col : 0);
        const uint32_t idesc = kIdescBase | (uint32_t(t.w * 8) << 17);      // N = 64 w
        const bool odd = (t.n0 & 64) != 0;
        const uint32_t sfb_t = sfb_t0 + (odd ? 2u : 0u);                    // skip the chunk's first 64 rows
        const bool two_chunks = (odd ? 64 : 0) + 64 * t.w > 128;
        for (int kb = 0; kb < p.k_stages && ok; ++kb) {
          ok = warp_wait(bar_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 3);
          if (!ok) break;
          bits ^= 1u << s;
          tc_fence_after_sync();
          const int nch = min(4, p.sf_chunks - kb * 4);
          // descriptor low words count 16-byte units: +32 per 512-byte scale chunk, +128 per
          // 2048-byte block of 128 B rows, +2 per 32 bytes of K in the operand tile
          const uint64_t sfa_d = sfa_d0 + s * (L::kSfa >> 4);
          const uint64_t sfb_d = sfb_d0 + s * (L::kSfb >> 4);
          const uint64_t adesc = adesc0 + s * (L::kA >> 4);
          const uint64_t bdesc = bdesc0 + s * (L::kB >> 4);
          if (elect_one()) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              if (c < nch) {
                tc_cp_32x128b_warpx4_pair(sfa_t + 4 * c, sfa_d + 32 * c);
                tc_cp_32x128b_warpx4_pair(sfb_t0 + 8 * c, sfb_d + 32 * c);
                if (two_chunks) tc_cp_32x128b_warpx4_pair(sfb_t0 + 8 * c + 4, sfb_d + 128 + 32 * c);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < nch) {
                const uint32_t accumulate = (j > 0 || kb > 0) ? 1u : 0u;
                tc_mma_nvfp4_pair(acc, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t + 4 * j, sfb_t + 8 * j,
                                  accumulate);
              }
            }
            tc_commit_pair(bar_empty + 8 * s, 3);  // frees this stage in both CTAs
          }
          __syncwarp();
          s = (s + 1 == STAGES) ? 0u : s + 1;
        }
        if (ok && elect_one()) tc_commit_pair(bar_acc_full + 8 * a, 3);
        __syncwarp();
        MSC_STAMP(1, tl, 1);
        ++tl;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------
    // warp e drains lane quadrant e % 4; of the tile's 2 w chunks of 32 columns the warps of
    // half e / 4 take chunks [half * w, half * w + w)
    BalWalker walk;
    walk.init(p, pair, npairs);
    BalTile t;
    uint32_t acc_uses = 0;
    int tl = 0;
    const int quad = warp & 3;
    const int half = warp >> 2;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t box0 = sbase + L::kOffC + warp * L::kCPerWarp;
    while (walk.next(p, t)) {
      const uint32_t a = (uint32_t)t.slot;
      bool ok = true;
      if (lane == 0) ok = mbar_wait_bounded(bar_acc_full + 8 * a, (acc_uses >> a) & 1u, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      acc_uses ^= 1u << a;
      tc_fence_after_sync();
      if (warp == 0) MSC_STAMP(2, tl, 0);
      const int row_warp = (2 * t.mt + (int)rank) * 128 + quad * 32;
      const bool valid = row_warp + lane < t.rows;
      const bool whole_warp = row_warp + 32 <= t.rows;
      const size_t out_row = (size_t)t.off + row_warp + lane;
      float scale = p.alpha ? __ldg(p.alpha + t.g) : 1.0f;
      if (p.row_scale && valid) scale *= __ldg(p.row_scale + out_row);

      const int w = t.w;
      const uint32_t acc = tmem_base + lane_base + (a ? kBalAcc1Col : 0) + half * w * 32;
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c < w) tmem_ld_32x32b_x32(acc + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster((bar_acc_empty + 8 * a) & kLeaderMask);
      if (warp == 0) MSC_STAMP(2, tl, 1);
      ++tl;
      if (MSC_FLAG(1)) continue;

      const int col0 = t.n0 + half * w * 32;
      if (whole_warp) {
        if (lane == 0) bulk_wait_group_read0();  // the previous tile's stores have left the boxes
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < w) {
            const uint32_t box = box0 + (c & 1) * L::kCBox;
            if (c >= 2) {   // the box is reused: its earlier store (two groups back) has been read
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              __syncwarp();
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t wd[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
                const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
                __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                wd[e] = *reinterpret_cast<uint32_t*>(&pr);
              }
              // 64-byte swizzle: the 16-byte unit index is XORed with bits 7-8 of the address
              const uint32_t addr = box + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(wd[0]),
                           "r"(wd[1]), "r"(wd[2]), "r"(wd[3]) : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, box, col0 + c * 32, t.off + row_warp);
              bulk_commit_group();
            }
          }
        }
      } else if (valid) {
        __nv_bfloat16* dst = p.out + out_row * p.n + col0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < w) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t wd[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
                const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
                __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                wd[e] = *reinterpret_cast<uint32_t*>(&pr);
              }
              d4[q] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
            }
          }
        }
      }
    }
    if (lane == 0) bulk_wait_group_read0();
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

template <int STAGES>
static int launch_bal(const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = BalSmem<STAGES>;
  auto kern = gemm_bal_kernel<STAGES>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc = pdl_launch_config(grid, L::kThreads, L::kAlloc, stream, attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, maps[0], maps[1], maps[2], maps[3], maps[4], p));
  return MSC_OK;
}

int launch_bal_gemm(const void* a_q, const void* b_q, long long rows_total, long long k_bytes,
                    const GemmParams& p, int stages, int max_ctas, cudaStream_t stream) {
  if (p.n % 64) return fail(MSC_ERR_BAD_ARG, "the balanced CTA-pair kernel needs n %% 64 == 0, got n=%d", p.n);
  if (p.n % 128)
    return fail(MSC_ERR_BAD_ARG, "the scale tiling covers 128 rows of B per chunk: n=%d must be a multiple of 128", p.n);
  CUtensorMap maps[5];
  int rc = make_tmap_bytes_2d(&maps[0], a_q, (uint64_t)rows_total, (uint64_t)k_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_bytes_2d(&maps[1], b_q, (uint64_t)p.l * p.n, (uint64_t)k_bytes, 32);
  if (rc) return rc;
  const uint64_t row_tiles = (uint64_t)(rows_total + 127) / 128;
  rc = make_tmap_sf_2d(&maps[2], p.sfa, row_tiles * p.sf_chunks * 4, 16);
  if (rc) return rc;
  rc = make_tmap_sf_2d(&maps[3], p.sfb, (uint64_t)p.l * (p.n / 128) * p.sf_chunks * 4, 16);
  if (rc) return rc;
  rc = make_tmap_bf16_narrow_2d(&maps[4], p.out, (uint64_t)rows_total, (uint64_t)p.n, 32);
  if (rc) return rc;

  const long long max_units = ((rows_total + 255) / 256 + p.l) * (long long)(p.n / 64);
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  if (pairs > max_units) pairs = (int)max_units;
  const int grid = 2 * pairs;
  if (stages <= 0 || stages > 5) stages = 5;
  if (stages < 2) stages = 2;
  switch (stages) {
    case 2: return launch_bal<2>(maps, p, grid, stream);
    case 3: return launch_bal<3>(maps, p, grid, stream);
    case 4: return launch_bal<4>(maps, p, grid, stream);
    default: return launch_bal<5>(maps, p, grid, stream);
  }
}

}  // namespace msc
