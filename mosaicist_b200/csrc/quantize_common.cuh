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

// silu(gate) * up = gate / (1 + 2^(-gate log2 e)) * up in fp32 (nvfp4.py:81-88), with the
// approximate exponential and reciprocal the reference's own kernel uses
// (quantize_kernels.py:50-69): the result only feeds the e2m1 / e4m3 quantiser, a few ulp are
// far below its steps, and the accurate expf + IEEE reciprocal cost five times the
// instructions.  Every kernel that activates goes through this one function, so the fused and
// the stand-alone paths keep producing the same bytes.
__device__ __forceinline__ float silu_mul(float gate, float up) {
  float e, s;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(gate, -1.4426950408889634f)));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(__fadd_rn(1.0f, e)));
  return __fmul_rn(__fmul_rn(s, gate), up);
}

// a / b rounded to nearest, given rb = RN(1 / b): one multiply and two fused multiply-adds
// (q = RN(a rb); r = a - q b exactly; q' = RN(q + r rb)), which is the correctly rounded
// quotient whenever rb is the correctly rounded reciprocal and nothing overflows; the block
// quantiser divides 16 values by the same step, so the reciprocal is shared.
template <bool GUARD = true>
__device__ __forceinline__ float div_rn_shared_rcp(float a, float b, float rb) {
  const float q = __fmul_rn(a, rb);
  const float r = __fmaf_rn(-q, b, a);
  const float qc = __fmaf_rn(r, rb, q);
  // keep +-inf instead of inf - inf; a block whose largest quotient is finite needs no guard
  // (a NaN element comes out NaN either way)
  return (!GUARD || fabsf(q) <= 3.0e38f) ? qc : q;
}

// 16 values / step -> 8 bytes of e2m1.  The reference's clip to [-6, 6] is what the saturating
// conversion does to finite and infinite values alike, so it is not repeated here.
template <bool GUARD>
__device__ __forceinline__ void pack_block(const float* v, float safe, float rsafe, uint32_t* w) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t word = 0;
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
      const int i = h * 8 + pr * 2;
      const float x0 = div_rn_shared_rcp<GUARD>(v[i], safe, rsafe);
      const float x1 = div_rn_shared_rcp<GUARD>(v[i + 1], safe, rsafe);
      const __nv_fp4x2_storage_t b2 =
          __nv_cvt_float2_to_fp4x2(make_float2(x0, x1), __NV_E2M1, cudaRoundNearest);
      word |= (uint32_t)b2 << (8 * pr);
    }
    w[h] = word;
  }
}

// Quantises one block of 16 fp32 values into 8 bytes of e2m1 and its e4m3 scale byte.
__device__ __forceinline__ void quantize_16(const float* v, float gs, uint2& q8, uint32_t& sfb) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  float s = __fmul_rn(__fdiv_rn(amax, 6.0f), gs);
  s = fminf(fmaxf(s, 0.0f), 448.0f);
  sfb = (uint32_t)(uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
  const float step = __fdiv_rn(e4m3_to_float((uint8_t)sfb), gs);
  // A dead block (step == 0) must yield x / 1 * 0 = +-0 with the sign of x, as the reference
  // computes: with divisor 1 and "reciprocal" 0 the shared-reciprocal division returns exactly
  // that (q = x * 0, remainder x, correction x * 0 + q), so no separate multiply is needed.
  const bool dead = step == 0.0f;
  const float safe = dead ? 1.0f : step;
  const float rsafe = dead ? 0.0f : __frcp_rn(step);
  // the largest quotient of the block bounds all of them: only a block where it overflows (an
  // infinite element, a step that underflowed) takes the per-element overflow guard
  uint32_t w[2];
  if (__fmul_rn(amax, rsafe) <= 3.0e38f) pack_block<false>(v, safe, rsafe, w);
  else pack_block<true>(v, safe, rsafe, w);
  q8 = make_uint2(w[0], w[1]);
}

// The four lanes that own the four blocks of one 64-element unit (lane & 3 = block index)
// assemble their scale bytes into one 32-bit word, valid in the lane with (lane & 3) == 0.
__device__ __forceinline__ uint32_t gather_scale_word(uint32_t sfb) {
  uint32_t w = sfb;
  w |= __shfl_down_sync(0xffffffffu, sfb, 1) << 8;
  w |= __shfl_down_sync(0xffffffffu, sfb, 2) << 16;
  w |= __shfl_down_sync(0xffffffffu, sfb, 3) << 24;
  return w;
}

// Loads 16 consecutive bf16 values (32 bytes, 16-byte aligned) as fp32.
__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* src, float* v) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
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
