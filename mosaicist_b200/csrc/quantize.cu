// NVFP4 quantisation kernels (HBM-bound): activations -> packed e2m1 + one e4m3 scale per
// 16 K-elements, with the scales written either row-major or directly in the 128-row MMA
// tiling the GEMM reads; SiLU(gate)*up fused in front of the same quantiser; and the
// stand-alone scale re-tiling kernel.
//
// Arithmetic follows quantize_nvfp4 (experiments/flashinfer-megamoe-sm100a/nvfp4.py:39-57):
//   sf   = e4m3( clip(amax / 6 * gs, 0, 448) )        per block of 16
//   step = f32(sf) / gs
//   q    = e2m1_rne( clip(x / step, -6, 6) )           (0 when step == 0)
// every operation in IEEE fp32 (explicit _rn intrinsics, so no contraction or approximate
// division can change a rounding).  One thread owns one block of 16 elements (32 B of bf16
// in, 8 B of e2m1 out); four neighbouring lanes pool their scale bytes into one aligned
// 32-bit word, which is a unit of both scale layouts.
#include "host_common.h"
#include "quantize_common.cuh"

namespace msc {

struct QuantParams {
  const void* x;            // (rows_total, k) or, with silu, (rows_total, 2k)
  const float* gs;          // (l) per-group global scale
  const int* group_rows;    // (l) or null
  const int* group_offsets; // (l) or null
  uint8_t* q;               // (rows_total, k/2)
  uint8_t* sf;
  int l, m_stride, k;
  long long rows_total;
  int tiled, silu, f32_in;
};

// Group of a row in the ragged layout: offsets ascend (empty groups share the offset of the
// group after them), so the owner is the last group whose offset is <= row.
__device__ __forceinline__ int group_of_row(const QuantParams& p, long long row, bool& valid) {
  if (!p.group_offsets) {
    const int g = (int)(row / p.m_stride);
    const int r = (int)(row - (long long)g * p.m_stride);
    valid = !p.group_rows || r < __ldg(p.group_rows + g);
    return g;
  }
  int lo = 0, hi = p.l - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (__ldg(p.group_offsets + mid) <= row) lo = mid; else hi = mid - 1;
  }
  const long long off = __ldg(p.group_offsets + lo);
  valid = row >= off && row < off + __ldg(p.group_rows + lo);
  return lo;
}

// One thread per block of 16 elements: a warp reads 1 KB of one row with two fully used
// 16-byte loads per lane and writes 256 contiguous bytes of e2m1; four neighbouring lanes
// pool their scale bytes into one aligned 32-bit store.
__global__ void __launch_bounds__(256) nvfp4_quantize_kernel(const QuantParams p) {
  const int kblocks = p.k >> 4;
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = unit / kblocks;
  const int kb = (int)(unit - row * kblocks);
  // whole warps stay alive for the shuffle below; k % 64 == 0 keeps a row's lanes in fours
  bool valid = row < p.rows_total;
  int g = 0;
  if (valid) g = group_of_row(p, row, valid);
  float v[16];
  uint2 q8 = make_uint2(0, 0);
  uint32_t sfb = 0;
  if (valid) {
    const float gs = __ldg(p.gs + g);
    if (p.silu) {
      // row holds [gate (k) | up (k)] in bf16; activation stays fp32 (nvfp4.py:81-88)
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.x) + row * 2 * p.k + kb * 16;
      float gt[16], up[16];
      load16_bf16(base, gt);
      load16_bf16(base + p.k, up);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        v[i] = silu_mul(gt[i], up[i]);
      }
    } else if (p.f32_in) {
      const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + row * p.k + kb * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 f = __ldg(src + i);
        v[i * 4] = f.x; v[i * 4 + 1] = f.y; v[i * 4 + 2] = f.z; v[i * 4 + 3] = f.w;
      }
    } else {
      load16_bf16(static_cast<const __nv_bfloat16*>(p.x) + row * p.k + kb * 16, v);
    }
    quantize_16(v, gs, q8, sfb);
    *reinterpret_cast<uint2*>(p.q + row * (p.k >> 1) + kb * 8) = q8;
  }
  const uint32_t word = gather_scale_word(sfb);
  if (valid && (kb & 3) == 0) {
    const int kw = kb >> 2, kwords = kblocks >> 2;
    if (p.tiled)
      *reinterpret_cast<uint32_t*>(p.sf + tiled_sf_word((int)row, kw, kwords)) = word;
    else
      *reinterpret_cast<uint32_t*>(p.sf + row * (p.k >> 4) + kw * 4) = word;
  }
}

// (groups, mn, kwords*4) row-major scale bytes -> (groups, ceil(mn/128), kwords, 32, 16),
// padding rows zero.  One thread per 32-bit word of the output.
__global__ void __launch_bounds__(256)
sf_swizzle_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int groups, int mn,
                  int kwords) {
  const int tiles = (mn + 127) >> 7;
  const long long total = (long long)groups * tiles * kwords * 128;
  const long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= total) return;
  // w enumerates [g][t][c][b][a]: consecutive threads write consecutive words
  const int a = (int)(w & 3);
  const int b = (int)((w >> 2) & 31);
  long long rest = w >> 7;
  const int c = (int)(rest % kwords);
  rest /= kwords;
  const int t = (int)(rest % tiles);
  const int g = (int)(rest / tiles);
  const int row = t * 128 + a * 32 + b;
  uint32_t val = 0;
  if (row < mn)
    val = __ldg(reinterpret_cast<const uint32_t*>(src + ((size_t)g * mn + row) * kwords * 4) + c);
  reinterpret_cast<uint32_t*>(dst)[w] = val;
}

// The same re-tiling through shared memory: a CTA takes 32 bytes (8 words) of each of a tile's
// 128 rows - two lanes read one full sector of a row - and writes eight 512-byte chunks of the
// tiling with one 16-byte store per thread.  The tile's rows sit at a 9-word pitch, so the
// column reads of the second phase fall in 32 different banks.  With rows_used (device, one
// group only) tiles at or beyond that row are left alone.  Needs kwords % 4 == 0 and 16-byte
// aligned pointers.
__global__ void __launch_bounds__(256)
sf_swizzle_tile_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int groups, int mn,
                       int kwords, const int* __restrict__ rows_used) {
  __shared__ uint32_t tile[128 * 9];
  const int tiles = (mn + 127) >> 7;
  const int cgroups = (kwords + 7) >> 3;
  const int cg = blockIdx.x % cgroups;
  const int rest = blockIdx.x / cgroups;
  const int t = rest % tiles, g = rest / tiles;
  if (rows_used && t * 128 >= __ldg(rows_used)) return;   // uniform over the CTA
  {
    const int row_l = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int row = t * 128 + row_l, c0 = cg * 8 + half * 4;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < mn && c0 < kwords)
      v = __ldg(reinterpret_cast<const uint4*>(src + ((size_t)g * mn + row) * kwords * 4 + (size_t)c0 * 4));
    uint32_t* d = tile + row_l * 9 + half * 4;
    d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
  }
  __syncthreads();
  const int cc = threadIdx.x >> 5, b = threadIdx.x & 31;
  const int c = cg * 8 + cc;
  if (c < kwords) {
    const uint4 o = make_uint4(tile[b * 9 + cc], tile[(32 + b) * 9 + cc], tile[(64 + b) * 9 + cc],
                               tile[(96 + b) * 9 + cc]);
    *reinterpret_cast<uint4*>(dst + ((((size_t)g * tiles + t) * kwords + c) * 32 + b) * 16) = o;
  }
}

int launch_sf_swizzle(const void* sf_rowmajor, void* sf_tiled, int groups, int mn, int kwords,
                      const int* rows_used, cudaStream_t stream) {
  const long long tiles = (mn + 127) / 128;
  const bool by_tiles = kwords % 4 == 0 && reinterpret_cast<uintptr_t>(sf_rowmajor) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(sf_tiled) % 16 == 0;
  if (by_tiles) {
    const long long blocks = (long long)groups * tiles * ((kwords + 7) / 8);
    if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
    sf_swizzle_tile_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const uint8_t*>(sf_rowmajor), static_cast<uint8_t*>(sf_tiled), groups, mn, kwords,
        groups == 1 ? rows_used : nullptr);
  } else {
    const long long total = (long long)groups * tiles * kwords * 128;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
    sf_swizzle_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const uint8_t*>(sf_rowmajor), static_cast<uint8_t*>(sf_tiled), groups, mn, kwords);
  }
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

static int quantize_common(const void* x, int x_dtype, const float* gs, const int32_t* group_offsets,
                           const int32_t* group_rows, void* q, void* sf, int sf_layout, int l,
                           long long rows_total, int m_stride, int k, int silu, void* stream) {
  if (!x || !gs || !q || !sf) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (l <= 0 || rows_total <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (k % 64) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 64", k);
  if (x_dtype != 0 && x_dtype != 1) return fail(MSC_ERR_UNSUPPORTED, "x_dtype must be 0 (bf16) or 1 (f32)");
  if (silu && x_dtype != 0) return fail(MSC_ERR_UNSUPPORTED, "the fused SiLU form takes bf16 input");
  if (sf_layout != 0 && sf_layout != 1) return fail(MSC_ERR_BAD_ARG, "sf_layout must be 0 or 1");
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(q) % 16 ||
      reinterpret_cast<uintptr_t>(sf) % 4)
    return fail(MSC_ERR_BAD_ARG, "x and q must be 16-byte aligned, sf 4-byte aligned");
  QuantParams p;
  p.x = x; p.gs = gs; p.group_rows = group_rows; p.group_offsets = group_offsets;
  p.q = static_cast<uint8_t*>(q); p.sf = static_cast<uint8_t*>(sf);
  p.l = l; p.m_stride = m_stride; p.k = k; p.rows_total = rows_total;
  p.tiled = sf_layout; p.silu = silu; p.f32_in = x_dtype;
  const long long units = rows_total * (k / 16);
  const int threads = 256;
  const long long blocks = (units + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  nvfp4_quantize_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

}  // namespace msc

extern "C" {

int msc_nvfp4_quantize(const void* x, int x_dtype, const float* global_scale,
                       const int32_t* masked_m, void* q, void* sf, int sf_layout, int l, int m,
                       int k, void* stream) {
  if (m <= 0) return msc::fail(MSC_ERR_BAD_ARG, "m must be positive");
  if (sf_layout == 1 && m % 128)
    return msc::fail(MSC_ERR_BAD_ARG, "tiled scales need m %% 128 == 0 in the masked layout");
  return msc::quantize_common(x, x_dtype, global_scale, nullptr, masked_m, q, sf, sf_layout, l,
                              (long long)l * m, m, k, 0, stream);
}

int msc_nvfp4_silu_mul_quantize(const void* gateup, const float* global_scale,
                                const int32_t* masked_m, void* q, void* sf, int sf_layout, int l,
                                int m, int n, void* stream) {
  if (m <= 0) return msc::fail(MSC_ERR_BAD_ARG, "m must be positive");
  if (sf_layout == 1 && m % 128)
    return msc::fail(MSC_ERR_BAD_ARG, "tiled scales need m %% 128 == 0 in the masked layout");
  return msc::quantize_common(gateup, 0, global_scale, nullptr, masked_m, q, sf, sf_layout, l,
                              (long long)l * m, m, n, 1, stream);
}

int msc_nvfp4_quantize_ragged(const void* x, int x_dtype, const float* global_scale,
                              const int32_t* group_offsets, const int32_t* group_rows, void* q,
                              void* sf, int l, int rows_total, int k, int silu, void* stream) {
  if (!group_offsets || !group_rows)
    return msc::fail(MSC_ERR_BAD_ARG, "group_offsets and group_rows are required");
  return msc::quantize_common(x, x_dtype, global_scale, group_offsets, group_rows, q, sf, 1, l,
                              rows_total, 0, k, silu, stream);
}

int msc_sf_swizzle(const void* sf_rowmajor, void* sf_tiled, int groups, int mn, int k_scales,
                   void* stream) {
  if (!sf_rowmajor || !sf_tiled) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (groups <= 0 || mn <= 0 || k_scales <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (k_scales % 4) return msc::fail(MSC_ERR_BAD_ARG, "k_scales=%d must be a multiple of 4", k_scales);
  if (reinterpret_cast<uintptr_t>(sf_rowmajor) % 4 || reinterpret_cast<uintptr_t>(sf_tiled) % 4)
    return msc::fail(MSC_ERR_BAD_ARG, "scale pointers must be 4-byte aligned");
  return msc::launch_sf_swizzle(sf_rowmajor, sf_tiled, groups, mn, k_scales / 4, nullptr,
                                static_cast<cudaStream_t>(stream));
}

}  // extern "C"
