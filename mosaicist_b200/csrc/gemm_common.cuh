// Pieces shared by the block-scaled GEMM kernels: launch parameters, the tile walker and the
// debug-build trace hooks.
#pragma once

#include "host_common.h"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace msc {

enum : int { KIND_NVFP4 = 0, KIND_MXFP8 = 1 };

struct GemmParams {
  const uint8_t* sfa;        // [row_tiles][sf_chunks][512]
  const uint8_t* sfb;        // [l][n/128][sf_chunks][512]
  const float* alpha;        // [l] or null
  const float* row_scale;    // [rows_total] or null
  const int* group_rows;     // [l] or null (= m_stride)
  const int* group_offsets;  // [l] or null (= g * m_stride)
  __nv_bfloat16* out;        // [rows_total][n]
  int* status;
  int l, m_stride, n;
  int rows_total;            // rows of a_q / out: no group may reach beyond them
  int k_stages;              // ceil(k_bytes / 128)
  int sf_chunks;             // scale chunks along K per 128-row tile
  int raster;
  // fused SwiGLU + requantise epilogue (B holds gate rows then up rows, n = 2 x width):
  uint8_t* out_q;            // (rows_total, n/4) packed e2m1 of silu(gate) * up
  uint8_t* out_sf;           // its e4m3 scales, tiled (rows_total/128, n/128, 32, 16)
  const float* out_gs;       // [l] global scale of the activation
  // row-scatter epilogue: row r goes to scatter_base[code >> 26] + (code & 0x3ffffff) * n bf16,
  // code = row_dest[r]; negative codes are skipped
  const int* row_dest;       // [rows_total] or null
  uint8_t* scatter_base[16]; // unused entries are null: rows coded for them are skipped
  int scatter_count;         // destinations in use; codes naming another one are refused
  int scatter_rows;          // rows every destination holds; codes beyond them are refused
#ifdef MSC_DEBUG
  unsigned long long* trace;  // [cta][8 tiles][3 roles][2] clock64 stamps, then [cta][2] at the end
  int debug_flags;            // 1: skip global stores, 2: skip scale loads/copies, 4: skip MMAs
#endif
};

#ifdef MSC_DEBUG
extern unsigned long long* g_trace;
extern int g_debug_flags;
#define MSC_STAMP(role, tl, which)                                                        \
  do {                                                                                    \
    if (p.trace && (tl) < 8 && (threadIdx.x & 31) == 0)                                                            \
      p.trace[(((size_t)blockIdx.x * 8 + (tl)) * 3 + (role)) * 2 + (which)] = clock64();  \
  } while (0)
#define MSC_FLAG(bit) (p.debug_flags & (bit))
// fine stamps: [cta][32] after the per-CTA begin/end pairs; taken for tile 1, K stage 4
#define MSC_FINE(slot)                                                                     \
  do {                                                                                     \
    if (p.trace && tl == 1 && kb == 4)                                                     \
      p.trace[(size_t)gridDim.x * 50 + (size_t)blockIdx.x * 32 + (slot)] = clock64();      \
  } while (0)
#else
#define MSC_FINE(slot) do {} while (0)
#define MSC_STAMP(role, tl, which) do {} while (0)
#define MSC_FLAG(bit) false
#endif

// Walks the flattened (group, m-tile, n-tile) space in increasing tile id.
struct TileCursor {
  int g = 0, base = 0, mtiles = 0, rows = 0, off = 0;
  int mshift = 7;  // log2 of the rows one tile covers: 7 for one CTA, 8 for a CTA pair
  bool primed = false;
  __device__ __forceinline__ bool seek(const GemmParams& p, int ntiles, int t, int& mt, int& nt) {
    while (true) {
      if (!primed) {
        if (g >= p.l) return false;
        // every lane reads the same word; the broadcast tells the compiler so
        rows = p.group_rows ? __shfl_sync(0xffffffffu, __ldg(p.group_rows + g), 0) : p.m_stride;
        if (rows < 0) rows = 0;
        if (p.m_stride > 0 && rows > p.m_stride) rows = p.m_stride;
        off = p.group_offsets ? __shfl_sync(0xffffffffu, __ldg(p.group_offsets + g), 0)
                              : g * p.m_stride;
        // a group table that reaches beyond the buffers (an overflowing expert-parallel step,
        // a stale table after a timed-out wait) is cut to what the buffers hold
        if (off < 0 || off >= p.rows_total) rows = 0;
        else if (rows > p.rows_total - off) rows = p.rows_total - off;
        mtiles = (rows + (1 << mshift) - 1) >> mshift;
        primed = true;
      }
      const int tiles = mtiles * ntiles;
      if (t < base + tiles) break;
      base += tiles;
      ++g;
      primed = false;
    }
    const int u = t - base;
    if (p.raster == 0) {
      mt = u / ntiles;
      nt = u - mt * ntiles;
    } else {
      nt = u / mtiles;
      mt = u - nt * mtiles;
    }
    return true;
  }
};

// Launcher of the CTA-pair kernel (gemm_blockscaled_pair.cu).
int launch_pair_gemm(int kind, const void* a_q, const void* b_q, long long rows_total, long long k_bytes,
                     const GemmParams& p, int stages, int max_ctas, cudaStream_t stream,
                     bool sf_by_warps);

// Launcher of the tokens-on-N kernel (gemm_blockscaled_swap.cu): row-concatenated groups.
int launch_swap_gemm(int kind, const void* a_q, const void* b_q, long long rows_total, long long k_bytes,
                     const GemmParams& p, int max_ctas, cudaStream_t stream);

}  // namespace msc
