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
  GemmParams g;           // grouped form: group_rows / group_offsets / alpha / out / l / n
};

template <int STAGES>
struct DenseSmem {
  static constexpr int kHeader = 1024;
  static constexpr int kA = 128 * 128;       // 128 rows x 64 K-elements
  static constexpr int kB = 2 * 64 * 128;    // two boxes of 64 K rows x 64 columns
  static constexpr int kOffA = kHeader;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffC = kOffB + STAGES * kB;
  static constexpr int kEpiWarps = 8;
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
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

template <int STAGES, bool GROUPED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DenseSmem<STAGES>::kThreads, 1)
gemm_dense_f16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const DenseParams p) {
  using L = DenseSmem<STAGES>;
  constexpr int kMmaWarp = L::kEpiWarps;
  constexpr int kProducerWarp = L::kEpiWarps + 1;
  constexpr uint32_t kStageBytes = L::kA + L::kB;  // per CTA

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const uint32_t bar_full = sbase;                    // leader's are used
  const uint32_t bar_empty = sbase + 8 * STAGES;
  const uint32_t bar_acc_full = sbase + 16 * STAGES;  // 2 x 8
  const uint32_t bar_acc_empty = bar_acc_full + 16;   // 2 x 8, leader's are used
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
    cur.mshift = 8;
    for (int t = pair; ok; t += npairs) {
      int mt, nt, row0, col0;
      if (GROUPED) {
        if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
        row0 = cur.off + (2 * mt + (int)rank) * 128;                // rows of A
        col0 = cur.g * p.g.n + nt * 256 + (int)rank * 128;          // rows of B (K-major)
      } else {
        if (t >= total_tiles) break;
        dense_tile(p, t, mt, nt);
        row0 = (2 * mt + (int)rank) * 128;                          // rows of A
        col0 = (nt * 256 + (int)rank * 128) * 2;                    // byte column of B
      }
      for (int kb = 0; kb < p.k_stages; ++kb) {
        ok = warp_wait(bar_empty + 8 * s, ((bits >> s) & 1u) ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        bits ^= 1u << s;
        const uint32_t full = bar_full + 8 * s;
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(full, 2 * kStageBytes);
          tma_load_2d_pair(sbase + L::kOffA + s * L::kA, &tmap_a, full, kb * 128, row0);
          if (GROUPED) {
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB, &tmap_b, full, kb * 128, col0);
          } else {
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB, &tmap_b, full, col0, kb * 64);
            tma_load_2d_pair(sbase + L::kOffB + s * L::kB + 8192, &tmap_b, full, col0 + 128, kb * 64);
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
      cur.mshift = 8;
      for (int t = pair; ok; t += npairs, ++tl) {
        if (GROUPED) {
          int mt, nt;
          if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
        } else if (t >= total_tiles) {
          break;
        }
        const int buf = tl & 1;
        ok = warp_wait(bar_acc_empty + 8 * buf, ((uint32_t)(tl >> 1) & 1u) ^ 1u, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + buf * 256;
        for (int kb = 0; kb < p.k_stages; ++kb) {
          ok = warp_wait(bar_full + 8 * s, (bits >> s) & 1u, abort_flag, p.status, 3);
          if (!ok) break;
          bits ^= 1u << s;
          tc_fence_after_sync();
          // A advances 32 bytes of K per MMA inside its swizzled rows (+2 in 16-byte units);
          // an MN-major B advances 16 K rows = 2048 bytes (+128), a K-major B like A
          const uint64_t adesc = adesc0 + s * (L::kA >> 4);
          const uint64_t bdesc = bdesc0 + s * (L::kB >> 4);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_mma_f16_pair(acc, adesc + 2 * j, bdesc + kBStep * j, idesc, (kb | j) ? 1u : 0u);
            tc_commit_pair(bar_empty + 8 * s, 3);
          }
          __syncwarp();
          s = (s + 1 == STAGES) ? 0u : s + 1;
        }
        if (ok && elect_one()) tc_commit_pair(bar_acc_full + 8 * buf, 3);
        __syncwarp();
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
    cur.mshift = 8;
    for (int t = pair;; t += npairs, ++tl) {
      int mt, nt;
      if (GROUPED) {
        if (!cur.seek(p.g, ntiles_g, t, mt, nt)) break;
      } else {
        if (t >= total_tiles) break;
        dense_tile(p, t, mt, nt);
      }
      const int buf = tl & 1;
      bool ok = true;
      if (lane == 0)
        ok = mbar_wait_bounded(bar_acc_full + 8 * buf, (uint32_t)(tl >> 1) & 1u, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld_32x32b_x32(tmem_base + lane_base + buf * 256 + slab * 128 + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster((bar_acc_empty + 8 * buf) & kLeaderMask);

      const int row_in = (2 * mt + (int)rank) * 128 + quad * 32;   // row inside the group / matrix
      const int row0 = (GROUPED ? cur.off : 0) + row_in;
      const int colb = (nt * 256 + slab * 128) * 2;   // byte column
      float scale = 1.0f;
      if (GROUPED) {
        scale = p.g.alpha ? __ldg(p.g.alpha + cur.g) : 1.0f;
        if (row_in + 32 > cur.rows) {
          // ragged end of a group: plain stores of the valid rows only
          if (row_in + lane < cur.rows) {
            __nv_bfloat16* dst = p.g.out + (size_t)(row0 + lane) * p.g.n + (colb >> 1);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
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
      }
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        if (lane == 0) bulk_wait_group_read0();
        __syncwarp();
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
  p.g = GemmParams{};
  p.g.alpha = alpha;
  p.g.group_rows = group_rows;
  p.g.group_offsets = group_offsets;
  p.g.out = static_cast<__nv_bfloat16*>(out);
  p.g.l = l;
  p.g.m_stride = 0;
  p.g.n = n;
  p.g.raster = 0;
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  const long long tiles = ((long long)(rows_total + 255) / 256 + l) * (n / 256);
  if (pairs > tiles) pairs = (int)tiles;
  constexpr int kStages = 6;
  using L = DenseSmem<kStages>;
  auto kern = gemm_dense_f16_kernel<kStages, true>;
  static bool configured[64] = {false};
  int dev = 0;
  MSC_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MSC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    configured[dev & 63] = true;
  }
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
  p.g = GemmParams{};
  int pairs = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs <= 0) return fail(MSC_ERR_CUDA, "could not query the SM count");
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  if (pairs > tiles) pairs = (int)tiles;
  constexpr int kStages = 6;
  using L = DenseSmem<kStages>;
  auto kern = gemm_dense_f16_kernel<kStages, false>;
  static bool configured[64] = {false};
  int dev = 0;
  MSC_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MSC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    configured[dev & 63] = true;
  }
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t lc =
      pdl_launch_config(2 * pairs, L::kThreads, L::kAlloc, static_cast<cudaStream_t>(stream), attr);
  MSC_CUDA_OK(cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p));
  return MSC_OK;
}
