// MXFP8 quantisation and the per-group global scale of NVFP4 (both HBM-bound).
//
// MXFP8 (OCP Microscaling): e4m3 values with one power-of-two scale (ue8m0: a biased exponent
// byte, 2^(b - 127)) per 32 K-elements.  Structure of the reference's block-scaled FP8
// quantiser (experiments/flashinfer-megamoe-sm90a/quant.py:47-75: scale from the block
// maximum, q = x / scale clipped to the e4m3 range) with the MX scale rule:
//   scale = 2^e,  e = the smallest integer with blockmax <= 448 * 2^e, clamped to [-127, 127]
//   q     = e4m3_rne( clip(x / scale, -448, 448) )
// e is found from the bits of blockmax (blockmax = m 2^E, 1 <= m < 2, 448 = 1.75 * 2^8:
// e = E - 8 + (m > 1.75)), so no logarithm or division can round it the wrong way; x / 2^e is
// exact.  A block of zeros (or of values below 2^-126) gets the smallest scale, byte 0.
//
// One thread owns 8 consecutive elements (32 B of fp32 or 16 B of bf16 in, 8 B out), four
// neighbouring lanes share a block's maximum through two shuffles, sixteen lanes pool four
// scale bytes into one aligned 32-bit word, which is a unit of both scale layouts (row-major
// and the 128-row MMA tiling the GEMM reads).
//
// Global scale (experiments/flashinfer-megamoe-sm100a/nvfp4.py:29-36): gs[g] = numerator /
// max|x| over group g, a maximum of 0 counted as 1.  |x| as fp32 bit patterns orders like
// unsigned integers, so the groups' maxima are reduced with atomicMax into the output array
// itself and a second, one-block kernel turns them into the quotient in place.
#include "host_common.h"
#include "quantize_common.cuh"

namespace msc {

struct MxQuantParams {
  const void* x;             // (rows, k)
  uint8_t* q;                // (rows, k) e4m3
  uint8_t* sf;               // ue8m0: row-major (rows, k/32) or tiled (ceil(rows/128), k/128, 32, 16)
  const int* group_rows;     // (l) or null: only rows inside a group are quantised
  const int* group_offsets;  // (l) ascending, with group_rows
  long long rows;
  int k, l, tiled, f32_in;
};

__device__ __forceinline__ bool mx_row_live(const MxQuantParams& p, long long row) {
  if (!p.group_offsets) return true;
  int lo = 0, hi = p.l - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (__ldg(p.group_offsets + mid) <= row) lo = mid; else hi = mid - 1;
  }
  const long long off = __ldg(p.group_offsets + lo);
  return row >= off && row < off + __ldg(p.group_rows + lo);
}

// Biased exponent byte of the block scale for a block maximum `amax` >= 0.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  const int E = (int)(bits >> 23) - 127;                       // -127 for zero and subnormals
  int e = E - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);     // mantissa above 1.75
  e = max(-127, min(127, e));
  return (uint32_t)(e + 127);
}

// Four 8-element segments per thread, `stride` threads apart: all four loads are issued before
// anything is computed (the kernel is bound by the latency of HBM, not by arithmetic), and the
// lanes of a warp still cover consecutive segments in every round, so loads and stores coalesce
// and the 4- and 16-lane groups of one scale block / scale word stay together.
constexpr int kMxRounds = 4;

__global__ void __launch_bounds__(256) mxfp8_quantize_kernel(const MxQuantParams p, long long stride) {
  const int per_row = p.k >> 3;                                 // segments per row
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long row[kMxRounds];
  int seg[kMxRounds];
  bool live[kMxRounds];
  uint4 raw[kMxRounds][2];
#pragma unroll
  for (int r = 0; r < kMxRounds; ++r) {
    const long long unit = first + r * stride;
    row[r] = unit / per_row;
    seg[r] = (int)(unit - row[r] * per_row);                    // 8-element segment inside the row
    // whole warps stay alive for the shuffles; k % 128 == 0 keeps 16-lane groups inside a row
    live[r] = row[r] < p.rows;
    if (live[r]) live[r] = mx_row_live(p, row[r]);
    raw[r][0] = raw[r][1] = make_uint4(0u, 0u, 0u, 0u);
    if (live[r]) {
      if (p.f32_in) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const float*>(p.x) + row[r] * p.k + seg[r] * 8);
        raw[r][0] = __ldg(src);
        raw[r][1] = __ldg(src + 1);
      } else {
        raw[r][0] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.x) + row[r] * p.k + seg[r] * 8));
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kMxRounds; ++r) {
    float v[8];
    if (p.f32_in) {
      const float* f0 = reinterpret_cast<const float*>(&raw[r][0]);
      const float* f1 = reinterpret_cast<const float*>(&raw[r][1]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = f0[i];
        v[4 + i] = f1[i];
      }
    } else {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r][0]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t sfb = mx_scale_byte(amax);
    if (live[r]) {
      // 1 / scale = 2^(127 - byte) is a normal fp32 number for every byte the rule can produce
      // (byte <= 247), so x / scale is one exact multiplication (or one rounding into the fp32
      // subnormals, far below e4m3's reach); the saturating conversion is the clip to +-448
      // followed by round-to-nearest-even, two values per instruction
      const float inv = __uint_as_float((254u - sfb) << 23);
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] * inv, v[4 * h + 1] * inv),
                                                     __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] * inv, v[4 * h + 3] * inv),
                                                     __NV_SATFINITE, __NV_E4M3);
        w[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(p.q + row[r] * p.k + seg[r] * 8) = make_uint2(w[0], w[1]);
    }
    // lanes 0, 4, 8, 12 (and 16 ... 28) hold the scale bytes of four consecutive blocks
    uint32_t word = sfb;
    word |= __shfl_down_sync(0xffffffffu, sfb, 4) << 8;
    word |= __shfl_down_sync(0xffffffffu, sfb, 8) << 16;
    word |= __shfl_down_sync(0xffffffffu, sfb, 12) << 24;
    if (live[r] && (threadIdx.x & 15) == 0) {
      const int kw = seg[r] >> 4, kwords = p.k >> 7;
      if (p.tiled)
        *reinterpret_cast<uint32_t*>(p.sf + tiled_sf_word((int)row[r], kw, kwords)) = word;
      else
        *reinterpret_cast<uint32_t*>(p.sf + row[r] * (p.k >> 5) + kw * 4) = word;
    }
  }
}

// max |x| per group into out[g] (as fp32 bit patterns, which order like unsigned integers).
__global__ void __launch_bounds__(256)
amax_groups_kernel(const void* __restrict__ x, int f32_in, long long per_group, unsigned int* __restrict__ out) {
  const int g = blockIdx.y;
  const long long vecs = per_group >> 3;                        // 8 elements per step
  float m = 0.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    if (f32_in) {
      const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(x) + g * per_group) + 2 * i;
      const float4 a = __ldg(src), b = __ldg(src + 1);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
      m = fmaxf(m, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
    } else {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + g * per_group) + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  __shared__ float warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, warp_max[i]);
    atomicMax(out + g, __float_as_uint(m));
  }
}

__global__ void amax_to_scale_kernel(float* __restrict__ inout, int l, float numerator) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= l) return;
  const float amax = inout[g];
  inout[g] = __fdiv_rn(numerator, amax == 0.0f ? 1.0f : amax);
}

static int mx_quantize(const void* x, int x_dtype, void* q, void* sf, int sf_layout, long long rows, int k,
                       const int32_t* group_offsets, const int32_t* group_rows, int l, void* stream) {
  if (!x || !q || !sf) return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (rows <= 0 || k <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (k % 128) return fail(MSC_ERR_BAD_ARG, "k=%d must be a multiple of 128", k);
  if (x_dtype != 0 && x_dtype != 1) return fail(MSC_ERR_UNSUPPORTED, "x_dtype must be 0 (bf16) or 1 (f32)");
  if (sf_layout != 0 && sf_layout != 1) return fail(MSC_ERR_BAD_ARG, "sf_layout must be 0 or 1");
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(q) % 8 ||
      reinterpret_cast<uintptr_t>(sf) % 4)
    return fail(MSC_ERR_BAD_ARG, "x must be 16-byte aligned, q 8-byte aligned, sf 4-byte aligned");
  MxQuantParams p;
  p.x = x; p.q = static_cast<uint8_t*>(q); p.sf = static_cast<uint8_t*>(sf);
  p.group_rows = group_rows; p.group_offsets = group_offsets;
  p.rows = rows; p.k = k; p.l = l; p.tiled = sf_layout; p.f32_in = x_dtype;
  const long long units = rows * (k / 8);
  // a quarter of the segments per round, rounded up to whole blocks
  const long long blocks = (units + 256LL * kMxRounds - 1) / (256LL * kMxRounds);
  if (blocks > 0x7fffffffLL) return fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  mxfp8_quantize_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, blocks * 256LL);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

}  // namespace msc

extern "C" {

int msc_mxfp8_quantize(const void* x, int x_dtype, void* q, void* sf, int sf_layout, int rows, int k,
                       void* stream) {
  return msc::mx_quantize(x, x_dtype, q, sf, sf_layout, rows, k, nullptr, nullptr, 0, stream);
}

int msc_mxfp8_quantize_ragged(const void* x, int x_dtype, const int32_t* group_offsets,
                              const int32_t* group_rows, void* q, void* sf, int l, int rows_total, int k,
                              void* stream) {
  if (!group_offsets || !group_rows || l <= 0)
    return msc::fail(MSC_ERR_BAD_ARG, "group_offsets, group_rows and l > 0 are required");
  return msc::mx_quantize(x, x_dtype, q, sf, 1, rows_total, k, group_offsets, group_rows, l, stream);
}

int msc_amax_global_scale(const void* x, int x_dtype, int l, long long elems_per_group, float numerator,
                          float* global_scale, void* stream) {
  if (!x || !global_scale) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (l <= 0 || elems_per_group <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (elems_per_group % 8) return msc::fail(MSC_ERR_BAD_ARG, "elems_per_group must be a multiple of 8");
  if (l > 65535) return msc::fail(MSC_ERR_UNSUPPORTED, "l=%d exceeds 65535 groups", l);
  if (x_dtype != 0 && x_dtype != 1) return msc::fail(MSC_ERR_UNSUPPORTED, "x_dtype must be 0 (bf16) or 1 (f32)");
  if (reinterpret_cast<uintptr_t>(x) % 16) return msc::fail(MSC_ERR_BAD_ARG, "x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MSC_CUDA_OK(cudaMemsetAsync(global_scale, 0, sizeof(float) * l, st));
  // enough blocks per group to fill the machine a few times over, never more than the group has work for
  const long long vecs = elems_per_group / 8;
  long long per_group = (vecs + 256 * 8 - 1) / (256 * 8);
  const long long want = (long long)msc::num_sms() * 8 / l + 1;
  if (per_group > want) per_group = want;
  if (per_group < 1) per_group = 1;
  msc::amax_groups_kernel<<<dim3((unsigned)per_group, (unsigned)l), 256, 0, st>>>(
      x, x_dtype, elems_per_group, reinterpret_cast<unsigned int*>(global_scale));
  MSC_CUDA_OK(cudaGetLastError());
  msc::amax_to_scale_kernel<<<(l + 255) / 256, 256, 0, st>>>(global_scale, l, numerator);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

}  // extern "C"
