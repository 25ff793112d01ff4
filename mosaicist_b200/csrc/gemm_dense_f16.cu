// Dense 16-bit GEMM for sm_100a: C(M,N) = A(M,K) * B(K,N), A and B fp16 (or bf16) row-major,
// fp32 accumulation in TMEM, C in the input type.  This is the reference's dense benchmark
// problem (experiments/hopper_gemm/gen_inputs.py:26-27: B stored (K, N) row-major;
// ref_cutedsl.py:50-74: 128x256 CTA tile, 2x1 cluster, oracle a.double() @ b.double()).
//
// CTA pairs (tcgen05 cta_group::2) compute 256 x 256 tiles: each CTA owns 128 rows of A
// (K-major boxes of 64 K-elements) and 128 of the tile's 256 columns of B.  B is used as
// stored — its contiguous axis is N, so its shared-memory tiles are "MN-major": two boxes
// of 64 columns x 64 K rows per CTA and stage, addressed through the descriptor's leading
// byte offset.  Each CTA fetches its own boxes (no multicast).  Without scale factors the
// 512 TMEM columns hold two 256-column accumulators, so the epilogue of one tile overlaps
// the main loop of the next.  Edges: TMA zero-fills loads and clips stores outside the
// matrices, so M, N and K only need 16-byte alignment, not tile multiples.
//
// TALL form (grouped only, the default there): a tile is 512 rows x 256 columns, two 256-row
// blocks of one group that share the B stage.  Both MMAs of a K step read the same weights, so a
// group of 257 - 512 rows streams (and, with int4 weights, expands) its weights once instead of
// twice; a tile whose second block holds no rows of the group neither loads nor multiplies it.
//
// WIDE form (dense only, the default for matrices of at least 512 columns): the two
// accumulators belong to ONE 256 x 512 tile, each K step is two MMAs that share the A stage.
// A 256 x 256 tile moves 64 KB per 64-element K stage for 512 tensor-pipe cycles, 62 bytes per
// clock and SM, which is what an SM can pull out of L2 when all of them do: that form is
// bounded by the L2 -> SM fabric at about 90 % of the tensor peak.  The wide tile moves 96 KB
// per 1024 cycles (47 B/clk), so the tensor pipe is the limit again; the price is that a tile's
// drain is no longer hidden behind the next tile's main loop (1-2 % at K = 8192).
//
// The same kernel has a grouped form (GROUPED = true): A is a row-concatenated batch of groups
// (group g owns rows [group_offsets[g], + group_rows[g]), offsets multiples of 128), B is
// (groups, n, k) with K contiguous ("NT", what a weight matrix per group looks like), C is
// (rows_total, n) bf16 scaled by alpha[g]; rows outside every group are never written.  It is
// the second half of the mixed-dtype grouped GEMM: int4 weights are expanded to bf16 by
// int4_dequant_kernel (convert to bf16, multiply by the group scale in bf16 — the order the
// reference prescribes, ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-81) and then
// multiplied here with fp32 accumulation (problems.py:84-87).
#include "gemm_common.cuh"

#include <cuda_fp16.h>

namespace msc {

struct DenseParams {
  int m_tiles, n_tiles;   // 256 x 256 pair tiles (dense form)
  int k_stages;           // ceil(K / 64)
  int band;               // m-tiles per raster band
  int is_bf16;
  int* status;
  const __nv_bfloat16* scales;   // int4 form: (groups, n, k / group_size)
  int group_size;
  GemmParams g;           // grouped form: group_rows / group_offsets / alpha / out / l / n
};

template <int STAGES, bool INT4 = false, bool WIDE = false, bool TALL = false>
struct DenseSmem {
  static constexpr int kHeader = 1024;
  static constexpr int kABlock = 128 * 128;  // 128 rows x 64 K-elements
  static constexpr int kA = TALL ? 2 * kABlock : kABlock;   // tall tiles: this CTA's rows of both row blocks
  static constexpr int kBHalf = 2 * 64 * 128;             // two boxes of 64 K rows x 64 columns
  static constexpr int kB = WIDE ? 2 * kBHalf : kBHalf;   // wide tiles: this CTA's share of both column blocks
  static constexpr int kP = INT4 ? 128 * 32 : 0;   // packed int4: 128 weight rows x 64 K-elements
  static constexpr int kOffA = kHeader;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffP = kOffB + STAGES * kB;
  static constexpr int kOffC = kOffP + STAGES * kP;
  static constexpr int kEpiWarps = 8;
  static constexpr int kConvWarps = INT4 ? 8 : 0;  // warps expanding int4 to bf16 in shared memory
  static constexpr int kThreads = (kEpiWarps + 2 + kConvWarps) * 32;
  static constexpr int kCPerWarp = 4096;
  static constexpr int kTotal = kOffC + kEpiWarps * kCPerWarp;
  static constexpr int kAlloc = kTotal + 1024;
  static_assert(kAlloc <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

__device__ __forceinline__ void dense_tile(const DenseParams& p, int t, int& mt, int& nt) {
  // bands of `band` m-tiles, n-tile slowest inside a band: the tiles in flight at one time
  // cover a near-square patch of C, so A and B panels are shared through L2
  const int per_band = p.band * p.n_tiles;
  const int b = t / per_band;
  const int u = t - b * per_band;
  const int rows = min(p.band, p.m_tiles - b * p.band);
  nt = u / rows;
  mt = b * p.band + (u - nt * rows);
}

template <int STAGES, bool GROUPED, bool INT4 = false, bool WIDE = false, bool TALL = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DenseSmem<STAGES, INT4, WIDE, TALL>::kThreads, 1)
gemm_dense_f16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const DenseParams p) {
  using L = DenseSmem<STAGES, INT4, WIDE, TALL>;
  static_assert(!INT4 || GROUPED, "int4 weights come with the grouped form");
  static_assert(!WIDE || !GROUPED, "wide tiles are built for the dense form");
  static_assert(!TALL || GROUPED, "tall tiles are built for the grouped form");
  constexpr int kTileCols = WIDE ? 512 : 256;
  constexpr int kTileRows = TALL ? 512 : 256;
  constexpr int kMShift = TALL ? 9 : 8;
  constexpr bool kOneAcc = WIDE || TALL;     // a tile fills both accumulators: no double buffering
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr int kFirstConvWarp = L::kEpiWarps + 2;
  // bytes TMA brings per CTA and stage onto the leader's full barrier: with int4 weights only A
  // (the packed weights land on each CTA's own barrier and reach the MMA through the converters)
  constexpr uint32_t kStageBytes = INT4 ? L::kABlock : L::kABlock + L::kB;   // with one row block

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const uint32_t bar_full = sbase;                    // leader's are used
  const uint32_t bar_empty = sbase + 8 * STAGES;
  const uint32_t bar_acc_full = sbase + 16 * STAGES;  // 2 x 8
  const uint32_t bar_acc_empty = bar_acc_full + 16;   // 2 x 8, leader's are used
  const uint32_t bar_packed = bar_acc_empty + 16;     // STAGES x 8: this CTA's packed weights landed
  const uint32_t bar_conv = bar_packed + 8 * STAGES;  // STAGES x 8 (leader's): bf16 weights written
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + 512);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + 516);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int total_tiles = p.m_tiles * p.n_tiles;
  // instruction descriptor: fp32 accumulate, A K-major, B MN-major (dense) or K-major
  // (grouped), M = 256, N = 256
  const uint32_t idesc = (1u << 4) | (p.is_bf16 ? ((1u << 7) | (1u << 10)) : 0u) |
                         (GROUPED ? 0u : (1u << 16)) | (uint32_t(256 >> 3) << 17) |
                         (uint32_t(256 >> 4) << 24);
  const int ntiles_g = GROUPED ? p.g.n / 256 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 2 * L::kEpiWarps);
    }
    if (INT4) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(bar_packed + 8 * s, 1);
        mbar_init(bar_conv + 8 * s, 2 * L::kConvWarps);
      }
    }
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  grid_dependency_wait();    // set-up may overlap the previous kernel; its data is read after this
  grid_launch_dependents();

  if (warp == kProducerWarp) {
    // ------------------------------ producer (both CTAs) ------------------------
    uint32_t bits = 0, s = 0;
    bool ok = true;
    TileCursor cur;
    cur.mshift = kMShift;
    for (int t = pair; ok; t += npairs) {
      int mt, nt, row0, col0;
      if (GROUPED) {
        if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
        row0 = cur.off + mt * kTileRows + (int)rank * 128;          // rows of A
        col0 = cur.g * p.g.n + nt * 256 + (int)rank * 128;          // rows of B (K-major)
      } else {
        if (t >= total_tiles) break;
        dense_tile(p, t, mt, nt);
        row0 = (2 * mt + (int)rank) * 128;                          // rows of A
        col0 = (nt * kTileCols + (int)rank * 128) * 2;              // byte column of B
      }
      // tall tiles: the second row block is fetched only if it holds rows of the group
      const bool has1 = TALL && mt * kTileRows + 256 < cur.rows;
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_empty + 8 * s, ((bits >> s) & 1u) ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t full = bar_full + 8 * s;
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(full, 2 * (kStageBytes + (has1 ? (uint32_t)L::kABlock : 0u)));
          tma_load_2d_pair(sbase + L::kOffA + s * L::kA, &tmap_a, full, kb * 128, row0);
          if (has1)
            tma_load_2d_pair(sbase + L::kOffA + s * L::kA + L::kABlock, &tmap_a, full, kb * 128, row0 + 256);
          if (INT4) {
            const uint32_t packed = bar_packed + 8 * s;
            mbar_arrive_expect_tx(packed, L::kP);
            tma_load_2d(sbase + L::kOffP + s * L::kP, &tmap_b, packed, kb * 32, col0);
          } else if (GROUPED) {
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB, &tmap_b, full, kb * 128, col0);
          } else {
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB, &tmap_b, full, col0, kb * 64);
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB + 8192, &tmap_b, full, col0 + 128, kb * 64);
            if (WIDE) {   // this CTA's 128 columns of the tile's second 256-column block
              tma_load_2d_pair(sbase + L::kOffB + s * L::kB + L::kBHalf, &tmap_b, full, col0 + 512, kb * 64);
              tma_load_2d_pair(sbase + L::kOffB + s * L::kB + L::kBHalf + 8192, &tmap_b, full, col0 + 640,
                               kb * 64);
            }
          }
        }
        __syncwarp();
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer (leader only) --------------------
    if (leader) {
      uint32_t bits = 0, s = 0;
      int tl = 0;
      bool ok = true;
      const uint64_t adesc0 = operand_desc_sw128(sbase + L::kOffA);
      const uint64_t bdesc0 = GROUPED ? operand_desc_sw128(sbase + L::kOffB)
                                      : operand_desc_mn_sw128(sbase + L::kOffB, 8192u);
      constexpr int kBStep = GROUPED ? 2 : 128;
      TileCursor cur;
      cur.mshift = kMShift;
      for (int t = pair; ok; t += npairs, ++tl) {
        bool has1 = false;
        if (GROUPED) {
          int mt, nt;
          if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
          has1 = TALL && mt * kTileRows + 256 < cur.rows;
        } else if (t >= total_tiles) {
          break;
        }
        // a wide or tall tile fills both accumulators: it uses barrier pair 0 every time
        const int buf = kOneAcc ? 0 : (tl & 1);
        const uint32_t use = kOneAcc ? (uint32_t)tl : (uint32_t)(tl >> 1);
        ok = warp_wait(bar_acc_empty + 8 * buf, (use & 1u) ^ 1u, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + buf * 256;
        for (int kb = 0; kb < p.k_stages; ++kb) {
          ok = warp_wait(bar_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 3);
          if (ok && INT4) ok = warp_wait(bar_conv + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 5);
          if (!ok) break;
          bits ^= 1u << s;
          tc_fence_after_sync();
          // A advances 32 bytes of K per MMA inside its swizzled rows (+2 in 16-byte units);
          // an MN-major B advances 16 K rows = 2048 bytes (+128), a K-major B like A
          const uint64_t adesc = adesc0 + s * (L::kA >> 4);
          const uint64_t bdesc = bdesc0 + s * (L::kB >> 4);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              tc_mma_f16_pair(acc, adesc + 2 * j, bdesc + kBStep * j, idesc, (kb | j) ? 1u : 0u);
              if (WIDE)
                tc_mma_f16_pair(acc + 256, adesc + 2 * j, bdesc + (L::kBHalf >> 4) + kBStep * j, idesc,
                                (kb | j) ? 1u : 0u);
              if (has1)   // the tile's second row block against the same B stage
                tc_mma_f16_pair(acc + 256, adesc + (L::kABlock >> 4) + 2 * j, bdesc + kBStep * j, idesc,
                                (kb | j) ? 1u : 0u);
            }
            tc_commit_pair(bar_empty + 8 * s, 3);
          }
          __syncwarp();
          s = (s + 1 == STAGES) ? 0u : s + 1;
        }
        if (ok && elect_one()) tc_commit_pair(bar_acc_full + 8 * buf, 3);
        __syncwarp();
      }
    }
  } else if (INT4 && warp >= kFirstConvWarp) {
    // ------------------------------ int4 -> bf16 converters (both CTAs) ---------
    // Two threads share weight row r of this CTA's 128: per stage each reads 16 of the row's 32
    // packed bytes (32 K-elements), forms bf16(q) * scale in bf16 (the reference's order,
    // problems.py:75-81) and writes four of the eight 16-byte chunks of the row in the K-major,
    // 128-byte-swizzled operand tile the MMA reads (chunk j of row r sits at chunk j ^ (r & 7)).
    // An int4 value q becomes bf16 exactly: the nibble with its sign bit flipped is q + 8, OR-ed
    // into the mantissa of 128.0 it reads 136 + q, and subtracting 136 is exact.  The nibbles
    // of a word are expanded as (n0,n4) (n1,n5) (n2,n6) (n3,n7) - one mask per pair - and
    // byte-permuted back into K order afterwards.
    const int ct = (warp - kFirstConvWarp) * 32 + lane;
    const int r = ct >> 1, half = ct & 1;
    const int groups_k = p.k_stages * 64 / p.group_size;
    const int stages_per_group = p.group_size >> 6;
    uint32_t bits = 0, s = 0;
    bool ok = true;
    TileCursor cur;
    cur.mshift = kMShift;
    const __nv_bfloat162 k136 = __float2bfloat162_rn(136.0f);
    for (int t = pair; ok; t += npairs) {
      int mt, nt;
      if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
      const __nv_bfloat16* srow =
          p.scales + ((size_t)cur.g * p.g.n + nt * 256 + (int)rank * 128 + r) * groups_k;
      __nv_bfloat16 sc = __ldg(srow);
      for (int kb = 0; kb < p.k_stages; ++kb) {
        const int kg = kb / stages_per_group;
        // the next group's scale is requested before this stage's data is waited for
        __nv_bfloat16 sc_next = sc;
        if (kb + 1 < p.k_stages && (kb + 1) % stages_per_group == 0) sc_next = __ldg(srow + kg + 1);
        ok = warp_wait(bar_packed + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 6);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t src = sbase + L::kOffP + s * L::kP + r * 32 + half * 16;
        const uint32_t dst = sbase + L::kOffB + s * L::kB + r * 128;
        const __nv_bfloat162 sc2 = __halves2bfloat162(sc, sc);
        uint32_t w[4];
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(src) : "memory");
#pragma unroll
        for (int jl = 0; jl < 4; ++jl) {
          const uint32_t x = w[jl] ^ 0x88888888u;
          uint32_t e[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t m = ((x >> (4 * i)) & 0x000F000Fu) | 0x43004300u;   // (n_i, n_{i+4})
            __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&m), k136);
            v = __hmul2(v, sc2);
            e[i] = *reinterpret_cast<uint32_t*>(&v);
          }
          const uint32_t o0 = __byte_perm(e[0], e[1], 0x5410);   // (n0, n1)
          const uint32_t o1 = __byte_perm(e[2], e[3], 0x5410);   // (n2, n3)
          const uint32_t o2 = __byte_perm(e[0], e[1], 0x7632);   // (n4, n5)
          const uint32_t o3 = __byte_perm(e[2], e[3], 0x7632);   // (n6, n7)
          const int j = half * 4 + jl;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                       ::"r"(dst + ((j ^ (r & 7)) << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
        }
        fence_proxy_async_smem();   // the tensor core reads these bytes through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster((bar_conv + 8 * s) & kLeaderMask);
        sc = sc_next;
        s = (s + 1 == STAGES) ? 0u : s + 1;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------
    // warp w: TMEM lane quadrant w % 4, 128-column slab w / 4; 64 columns at a time through a
    // swizzled 4 KB staging box and a TMA store, which also clips the matrix edges
    int tl = 0;
    const int quad = warp & 3;
    const int slab = warp >> 2;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t box = sbase + L::kOffC + warp * L::kCPerWarp;
    TileCursor cur;
    cur.mshift = kMShift;
    for (int t = pair;; t += npairs, ++tl) {
      int mt, nt;
      if (GROUPED) {
        if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
      } else {
        if (t >= total_tiles) break;
        dense_tile(p, t, mt, nt);
      }
      const int buf = kOneAcc ? 0 : (tl & 1);
      const uint32_t use = kOneAcc ? (uint32_t)tl : (uint32_t)(tl >> 1);
      bool ok = true;
      if (lane == 0)
        ok = mbar_wait_bounded(bar_acc_full + 8 * buf, use & 1u, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      // tall tiles: row block 0 sits in accumulator columns 0-255, block 1 (if the group reaches
      // it) in 256-511; the accumulators are handed back after the last block has been read
      const int nblk = (TALL && mt * kTileRows + 256 < cur.rows) ? 2 : 1;
      for (int blk = 0; blk < nblk; ++blk) {
      const int acc_col = TALL ? blk * 256 : buf * 256;
      const int row_in = mt * kTileRows + blk * 256 + (int)rank * 128 + quad * 32;   // row inside the group / matrix
      const int row0 = (GROUPED ? cur.off : 0) + row_in;
      // wide tiles: slab w / 4 drains one whole 256-column accumulator, 128 columns per pass
      const int colb = WIDE ? (nt * 512 + slab * 256) * 2 : (nt * 256 + slab * 128) * 2;   // byte column
      const float scale = (GROUPED && p.g.alpha) ? __ldg(p.g.alpha + cur.g) : 1.0f;
      const bool ragged = GROUPED && row_in + 32 > cur.rows;
      // The warp's 128 columns are drained in one pass, or in two 64-column passes where the
      // converter warps leave fewer registers per thread; the accumulator is handed back after
      // the last read either way (there are two accumulators, the next tile is not waiting).
      constexpr int kPasses = (INT4 || WIDE) ? 2 : 1;
      constexpr int kCh = WIDE ? 4 : 4 / kPasses;          // 32-column chunks per pass
      constexpr int kSubs = WIDE ? 2 : 2 / kPasses;        // 64-column store boxes per pass
      constexpr int kSlabCols = WIDE ? 256 : 128;          // accumulator columns one warp drains
#pragma unroll
      for (int pass = 0; pass < kPasses; ++pass) {
        uint32_t v[kCh][32];
#pragma unroll
        for (int c = 0; c < kCh; ++c)
          tmem_ld_32x32b_x32(tmem_base + lane_base + acc_col + slab * kSlabCols + (pass * kCh + c) * 32, v[c]);
        tmem_ld_wait();
        if (pass == kPasses - 1 && blk == nblk - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster((bar_acc_empty + 8 * buf) & kLeaderMask);
        }
        if (ragged) {
          // ragged end of a group: plain stores of the valid rows only
          if (row_in + lane < cur.rows) {
            __nv_bfloat16* dst = p.g.out + (size_t)(row0 + lane) * p.g.n + (colb >> 1) + pass * kCh * 32;
#pragma unroll
            for (int c = 0; c < kCh; ++c) {
              uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(v[c][q * 8 + 2 * e]) * scale,
                                                            __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale);
                  w[e] = *reinterpret_cast<uint32_t*>(&pr);
                }
                d4[q] = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
          }
          continue;
        }
#pragma unroll
        for (int s2 = 0; s2 < kSubs; ++s2) {
          const int sub = pass * kSubs + s2;
          if (lane == 0) bulk_wait_group_read0();
          __syncwarp();
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = s2 * 2 + cc;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[c][q * 8 + 2 * e]) * scale;
                const float hi = __uint_as_float(v[c][q * 8 + 2 * e + 1]) * scale;
                if (p.is_bf16) {
                  __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                  w[e] = *reinterpret_cast<uint32_t*>(&pr);
                } else {
                  __half2 pr = __floats2half2_rn(lo, hi);
                  w[e] = *reinterpret_cast<uint32_t*>(&pr);
                }
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
            tma_store_2d(&tmap_c, box, colb + sub * 128, row0);
            bulk_commit_group();
          }
        }
      }
      }   // row blocks
    }
    if (lane == 0) bulk_wait_group_read0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Expands int4 weights to bf16: out[g, n, k] = bf16( bf16(q[g, n, k]) * scale[g, n, k / group] ),
// q in [-8, 7] two per byte (element 2i in the low nibble).  One thread per 16 elements.
__global__ void __launch_bounds__(256)
int4_dequant_kernel(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scales,
                    __nv_bfloat16* __restrict__ out, long long rows, int k, int group) {
  const int units = k >> 4;
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = unit / units;
  const int u = (int)(unit - row * units);
  if (row >= rows) return;
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(q + row * (k >> 1)) + u);
  const __nv_bfloat16 sc = scales[row * (k / group) + (u * 16) / group];
  uint32_t words[2] = {raw.x, raw.y};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t byte = (words[i >> 2] >> (8 * (i & 3))) & 0xFFu;
    const int lo = (int)(byte & 0xF), hi = (int)(byte >> 4);
    const __nv_bfloat16 a = __hmul(__int2bfloat16_rn(lo >= 8 ? lo - 16 : lo), sc);
    const __nv_bfloat16 b = __hmul(__int2bfloat16_rn(hi >= 8 ? hi - 16 : hi), sc);
    __nv_bfloat162 pr = __halves2bfloat162(a, b);
    o[i] = *reinterpret_cast<uint32_t*>(&pr);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + row * k + u * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace msc

extern "C" int msc_int4_dequant_bf16(const void* q, const void* scales, void* out, int groups, int n,
                                     int k, int group_size, void* stream) {
  using namespace msc;
  if (!q || !scales || !out) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (groups <= 0 || n <= 0 || k <= 0 || group_size <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (k % 16 || group_size % 16 || k % group_size)
    return fail(MSC_ERR_BAD_ARG, "k and group_size must be multiples of 16 and group_size must divide k");
  const long long rows = (long long)groups * n;
  const long long blocks = (rows * (k / 16) + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  int4_dequant_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), static_cast<const __nv_bfloat16*>(scales),
      static_cast<__nv_bfloat16*>(out), rows, k, group_size);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

extern "C" int msc_grouped_gemm_bf16_ragged(const void* a, const void* b, const float* alpha,
                                            const int32_t* group_offsets, const int32_t* group_rows,
                                            void* out, int l, int rows_total, int n, int k,
                                            int max_ctas, void* stream) {
  using namespace msc;
  if (!a || !b || !out || !group_offsets || !group_rows) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (l <= 0 || rows_total <= 0 || n <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (n % 256) return fail(MSC_ERR_BAD_ARG, "n=%d must be a multiple of 256", n);
  if (k % 8) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 8", k);
  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");
  CUtensorMap ta, tb, tc;
  int rc = make_tmap_pitched_2d(&ta, a, (uint64_t)rows_total, (uint64_t)k * 2, (uint64_t)k * 2, 128);
  if (rc) return rc;
  rc = make_tmap_pitched_2d(&tb, b, (uint64_t)l * n, (uint64_t)k * 2, (uint64_t)k * 2, 128);
  if (rc) return rc;
  rc = make_tmap_pitched_2d(&tc, out, (uint64_t)rows_total, (uint64_t)n * 2, (uint64_t)n * 2, 32);
  if (rc) return rc;
  DenseParams p;
  p.m_tiles = p.n_tiles = 0;
  p.k_stages = (k + 63) / 64;
  p.band = 8;
  p.is_bf16 = 1;
  p.status = status;
  p.scales = nullptr;
  p.group_size = 0;
  p.g = GemmParams{};
  p.g.alpha = alpha;
  p.g.group_rows = group_rows;
  p.g.group_offsets = group_offsets;
  p.g.out = static_cast<__nv_bfloat16*>(out);
  p.g.l = l;
  p.g.m_stride = 0;
  p.g.rows_total = rows_total;
  p.g.n = n;
  p.g.raster = 0;
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  // 256-row tiles with two accumulators in turn: with bf16 weights the tall form (one weight
  // stage for two row blocks) measured slower here, 0.638 ms against 0.605 ms on 64 groups of
  // 64 - 512 rows, because its drain is not hidden; it pays where the weights are expanded
  const long long tiles = ((long long)(rows_total + 255) / 256 + l) * (n / 256);
  if (pairs > tiles) pairs = (int)tiles;
  constexpr int kStages = 6;
  using L = DenseSmem<kStages>;
  auto kern = gemm_dense_f16_kernel<kStages, true>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc =
      pdl_launch_config(2 * pairs, L::kThreads, L::kAlloc, static_cast<cudaStream_t>(stream), attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
  return MSC_OK;
}

extern "C" int msc_grouped_gemm_bf16_int4_ragged(const void* a, const void* b_q, const void* scales,
                                                 const float* alpha, const int32_t* group_offsets,
                                                 const int32_t* group_rows, void* out, int l,
                                                 int rows_total, int n, int k, int group_size,
                                                 int max_ctas, void* stream) {
  using namespace msc;
  if (!a || !b_q || !scales || !out || !group_offsets || !group_rows)
    return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (l <= 0 || rows_total <= 0 || n <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (n % 256) return fail(MSC_ERR_BAD_ARG, "n=%d must be a multiple of 256", n);
  if (k % 64) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 64", k);
  if (group_size <= 0 || group_size % 64 || k % group_size)
    return fail(MSC_ERR_UNSUPPORTED,
                "group_size=%d must be a multiple of 64 that divides k (use msc_int4_dequant_bf16 + "
                "msc_grouped_gemm_bf16_ragged otherwise)", group_size);
  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");
  CUtensorMap ta, tb, tc;
  int rc = make_tmap_pitched_2d(&ta, a, (uint64_t)rows_total, (uint64_t)k * 2, (uint64_t)k * 2, 128);
  if (rc) return rc;
  rc = make_tmap_narrow_2d(&tb, b_q, (uint64_t)l * n, (uint64_t)k / 2, 128);
  if (rc) return rc;
  rc = make_tmap_pitched_2d(&tc, out, (uint64_t)rows_total, (uint64_t)n * 2, (uint64_t)n * 2, 32);
  if (rc) return rc;
  DenseParams p;
  p.m_tiles = p.n_tiles = 0;
  p.k_stages = k / 64;
  p.band = 8;
  p.is_bf16 = 1;
  p.status = status;
  p.scales = static_cast<const __nv_bfloat16*>(scales);
  p.group_size = group_size;
  p.g = GemmParams{};
  p.g.alpha = alpha;
  p.g.group_rows = group_rows;
  p.g.group_offsets = group_offsets;
  p.g.out = static_cast<__nv_bfloat16*>(out);
  p.g.l = l;
  p.g.m_stride = 0;
  p.g.rows_total = rows_total;
  p.g.n = n;
  p.g.raster = 0;
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  const long long tiles = ((long long)(rows_total + 511) / 512 + l) * (n / 256);
  if (pairs > tiles) pairs = (int)tiles;
  constexpr int kStages = 3;
  using L = DenseSmem<kStages, true, false, true>;
  auto kern = gemm_dense_f16_kernel<kStages, true, true, false, true>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc =
      pdl_launch_config(2 * pairs, L::kThreads, L::kAlloc, static_cast<cudaStream_t>(stream), attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
  return MSC_OK;
}

extern "C" int msc_gemm_f16(const void* a, const void* b, void* c, int m, int n, int k, int lda,
                            int ldb, int ldc, int dtype, int max_ctas, void* stream) {
  using namespace msc;
  if (!a || !b || !c) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "m, n, k must be positive");
  if (dtype != 0 && dtype != 1) return fail(MSC_ERR_UNSUPPORTED, "dtype must be 0 (fp16) or 1 (bf16)");
  if (lda < k || ldb < n || ldc < n) return fail(MSC_ERR_BAD_ARG, "leading dimension smaller than the row");
  if ((k | n | lda | ldb | ldc) % 8)
    return fail(MSC_ERR_BAD_ARG, "k, n and the leading dimensions must be multiples of 8 (16 bytes)");
  int* status = status_word();
  if (!status) return fail(MSC_ERR_CUDA, "status word unavailable on this device");
  CUtensorMap ta, tb, tc;
  int rc = make_tmap_pitched_2d(&ta, a, (uint64_t)m, (uint64_t)k * 2, (uint64_t)lda * 2, 128);
  if (rc) return rc;
  rc = make_tmap_pitched_2d(&tb, b, (uint64_t)k, (uint64_t)n * 2, (uint64_t)ldb * 2, 64);
  if (rc) return rc;
  rc = make_tmap_pitched_2d(&tc, c, (uint64_t)m, (uint64_t)n * 2, (uint64_t)ldc * 2, 32);
  if (rc) return rc;
  DenseParams p;
  p.m_tiles = (m + 255) / 256;
  p.n_tiles = (n + 255) / 256;
  p.k_stages = (k + 63) / 64;
  p.band = 8;
  p.is_bf16 = dtype;
  p.status = status;
  p.scales = nullptr;
  p.group_size = 0;
  p.g = GemmParams{};
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  // 256 x 512 tiles when there are enough of them to keep every pair busy for a few rounds;
  // otherwise 256 x 256 tiles, which split a small problem into more pieces.  A negative
  // max_ctas keeps its magnitude as the grid size and forces the 256 x 256 form.
  const bool force_narrow = max_ctas < 0;
  if (force_narrow) pairs = (-max_ctas) / 2 > 0 ? (-max_ctas) / 2 : num_sms() / 2;
  const long long wide_tiles = (long long)p.m_tiles * ((n + 511) / 512);
  cudaLaunchAttribute attr[1];
  if (!force_narrow && wide_tiles >= 2LL * pairs) {
    p.n_tiles = (n + 511) / 512;
    p.band = 16;   // 8192^3: 0.721 / 0.707 / 0.700 / 0.711 ms with bands of 4 / 8 / 16 / 32 row tiles
    if (pairs > wide_tiles) pairs = (int)wide_tiles;
    constexpr int kStages = 4;
    using L = DenseSmem<kStages, false, true>;
    auto kern = gemm_dense_f16_kernel<kStages, false, false, true>;
    if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
    cudaLaunchConfig_t lc =
        pdl_launch_config(2 * pairs, L::kThreads, L::kAlloc, static_cast<cudaStream_t>(stream), attr);
    MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
    return MSC_OK;
  }
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  if (pairs > tiles) pairs = (int)tiles;
  constexpr int kStages = 6;
  using L = DenseSmem<kStages>;
  auto kern = gemm_dense_f16_kernel<kStages, false>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kAlloc)) return rc;
  cudaLaunchConfig_t lc =
      pdl_launch_config(2 * pairs, L::kThreads, L::kAlloc, static_cast<cudaStream_t>(stream), attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
  return MSC_OK;
}
