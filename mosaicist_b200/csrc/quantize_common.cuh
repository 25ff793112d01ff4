// Device helpers of the NVFP4 quantiser shared by the stand-alone quantise kernels and the
// MoE dispatch kernel: the arithmetic of quantize_nvfp4
// (experiments/flashinfer-megamoe-sm100a/nvfp4.py:39-57) on 64 values at a time, and the
// address of a scale word in the 128-row MMA tiling (nvfp4.py:121-131).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace msc {

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(__half(h));
}

// Offset of scale (row, kblock/4 word) in the tiled layout (row_tiles, kwords, 32, 16):
// row = 128 t + 32 a + b  ->  [t, c, b, 4 a + d], d = kblock % 4.
__device__ __forceinline__ size_t tiled_sf_word(int row, int kword, int kwords) {
  const int t = row >> 7, a = (row >> 5) & 3, b = row & 31;
  return (((size_t)t * kwords + kword) * 32 + b) * 16 + 4 * a;
}

// Quantises 64 fp32 values held as v[64] into 32 bytes + 4 scale bytes.
__device__ __forceinline__ void quantize_64(const float* v, float gs, uint32_t* q8, uint32_t& sf4) {
  sf4 = 0;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[blk * 16 + i]));
    float s = __fmul_rn(__fdiv_rn(amax, 6.0f), gs);
    s = fminf(fmaxf(s, 0.0f), 448.0f);
    const uint8_t sfb = (uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
    const float step = __fdiv_rn(e4m3_to_float(sfb), gs);
    // a dead block (step == 0) keeps the sign of x: x / 1 * 0 = +-0, as the reference computes
    const float live = (step > 0.0f) ? 1.0f : 0.0f;
    const float safe = (step == 0.0f) ? 1.0f : step;
    sf4 |= (uint32_t)sfb << (8 * blk);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      uint32_t word = 0;
#pragma unroll
      for (int pr = 0; pr < 4; ++pr) {
        const int i = blk * 16 + w * 8 + pr * 2;
        float x0 = __fmul_rn(__fdiv_rn(v[i], safe), live);
        float x1 = __fmul_rn(__fdiv_rn(v[i + 1], safe), live);
        x0 = fminf(fmaxf(x0, -6.0f), 6.0f);
        x1 = fminf(fmaxf(x1, -6.0f), 6.0f);
        const __nv_fp4x2_storage_t b2 =
            __nv_cvt_float2_to_fp4x2(make_float2(x0, x1), __NV_E2M1, cudaRoundNearest);
        word |= (uint32_t)b2 << (8 * pr);
      }
      q8[blk * 2 + w] = word;
    }
  }
}

// Loads 64 consecutive bf16 values (128 bytes, 16-byte aligned) as fp32.
__device__ __forceinline__ void load64_bf16(const __nv_bfloat16* src, float* v) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 raw = __ldg(s4 + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      v[i * 8 + j * 2] = f.x;
      v[i * 8 + j * 2 + 1] = f.y;
    }
  }
}

}  // namespace msc
