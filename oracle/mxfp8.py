"""MXFP8 block-scaled arithmetic on numpy + ml_dtypes (test infrastructure, not product).

PARITY UNPINNED: the reference tree has no MXFP8 (e4m3 values, one ue8m0 scale per 32
K-elements) code and no golden vectors for it.  The nearest reference arithmetic is the
Hopper analog's block-scaled FP8 quantiser (experiments/flashinfer-megamoe-sm90a/
quant.py:47-75: e4m3 values, e4m3 scale per 128, `q = x / scale` clipped to the e4m3
range, dequant `q * scale`); this file keeps that structure and substitutes the OCP MX
scale rule the benchmark configuration names: scale = 2^ceil(log2(blockmax / 448)), i.e. the
smallest power of two with blockmax / scale <= 448, stored as ue8m0 (biased exponent byte,
2^(b - 127)).
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

BLOCK = 32
E4M3 = ml_dtypes.float8_e4m3fn
E4M3_MAX = 448.0


def ue8m0_to_float(b: np.ndarray) -> np.ndarray:
    return np.ldexp(1.0, np.asarray(b, np.int32) - 127)


def quantize_mxfp8(x: np.ndarray):
    """(..., k) f32 -> (q e4m3 (..., k), sf ue8m0 bytes (..., k // 32))."""
    x = np.asarray(x, np.float32)
    k = x.shape[-1]
    if k % BLOCK:
        raise ValueError(f"K={k} must be a multiple of {BLOCK}")
    xb = x.reshape(*x.shape[:-1], k // BLOCK, BLOCK)
    amax = np.max(np.abs(xb), axis=-1)
    # the smallest integer e with amax <= 448 * 2^e, found exactly: amax = m 2^E with
    # 0.5 <= m < 1 (frexp), 448 = 0.875 * 2^9, so e = E - 9 + (m > 0.875); a logarithm in
    # floating point would misplace block maxima within an ulp of 448 * 2^e
    m, E = np.frexp(amax)
    e = np.where(amax > 0, E - 9 + (m > 0.875), -127)
    e = np.clip(e, -127, 127).astype(np.int32)
    scale = np.ldexp(np.float32(1.0), e)
    q = np.clip(xb / scale[..., None], -E4M3_MAX, E4M3_MAX).astype(E4M3)
    return q.reshape(x.shape), (e + 127).astype(np.uint8)


def dequantize_mxfp8(q: np.ndarray, sf: np.ndarray) -> np.ndarray:
    return np.asarray(q, np.float64) * np.repeat(ue8m0_to_float(sf), BLOCK, axis=-1)


def ragged_grouped_gemm_f64(a_q, a_sf, b_q, b_sf, offsets, rows, alpha=None, row_scale=None):
    """float64 oracle over row-concatenated groups: out[off_g + r] = alpha_g * w_r *
    dequant(A)[off_g + r] @ dequant(B)[g].T for r < rows[g]; other rows are zero."""
    a = dequantize_mxfp8(a_q, a_sf)
    out = np.zeros((a.shape[0], b_q.shape[1]), np.float64)
    for g, (o, r) in enumerate(zip(offsets, rows)):
        if r <= 0:
            continue
        y = a[o:o + r] @ dequantize_mxfp8(b_q[g], b_sf[g]).T
        if alpha is not None:
            y = y * float(alpha[g])
        if row_scale is not None:
            y = y * np.asarray(row_scale[o:o + r], np.float64)[:, None]
        out[o:o + r] = y
    return out


def exact_operands(rng: np.random.Generator, rows: int, k: int):
    """Small integers with power-of-two block scales: the whole GEMM is exact in fp32."""
    q = rng.integers(-4, 5, size=(rows, k)).astype(np.float32).astype(E4M3)
    sf = (rng.integers(-2, 3, size=(rows, k // BLOCK)) + 127).astype(np.uint8)
    return q, sf
