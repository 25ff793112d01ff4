"""Byte-level decoders for the narrow formats the library consumes, and the NVFP4 quantiser
stated on numpy.

Used by the capture modules' `reference()` hooks (the float64 opinion Mosaicist's numerics
gate asks every module for, src/mosaicist/capture.py:254-264) and by host-side input
preparation.  Nothing here runs on the hot path and no operator falls back to it.
"""

from __future__ import annotations

import numpy as np

_E2M1_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
E2M1_LUT = np.concatenate([_E2M1_MAG, -_E2M1_MAG])           # code -> value (bit 3 = sign)


def _e4m3_lut() -> np.ndarray:
    out = np.empty(256, np.float64)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e, m = (b >> 3) & 0xF, b & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = sign * v
    return out


E4M3_LUT = _e4m3_lut()
UE8M0_LUT = np.ldexp(1.0, np.arange(256) - 127)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """uint8 (..., k/2), element 2i in the low nibble -> float64 (..., k)."""
    p = np.asarray(packed, np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), np.float64)
    out[..., 0::2] = E2M1_LUT[p & 0xF]
    out[..., 1::2] = E2M1_LUT[p >> 4]
    return out


def from_mma_scale_layout(tiled: np.ndarray, mn: int) -> np.ndarray:
    """(tiles, kwords, 32, 16) -> (mn, 4 * kwords): [t, c, b, 4a + d] is row 128t + 32a + b,
    column 4c + d (the inverse of experiments/flashinfer-megamoe-sm100a/nvfp4.py:121-131)."""
    t, c = tiled.shape[0], tiled.shape[1]
    return (np.asarray(tiled).reshape(t, c, 32, 4, 4).transpose(0, 3, 2, 1, 4)
            .reshape(t * 128, c * 4)[:mn])


def dequant_nvfp4(q_packed: np.ndarray, sf_tiled: np.ndarray) -> np.ndarray:
    """(rows, k/2) packed e2m1 + tiled e4m3 scales -> float64 (rows, k) = q * sf."""
    q = unpack_e2m1(q_packed)
    rows = q.shape[0]
    sf = E4M3_LUT[from_mma_scale_layout(np.asarray(sf_tiled, np.uint8), rows)]
    return q * np.repeat(sf, 16, axis=-1)


def quantize_nvfp4_values(x: np.ndarray, global_scale) -> tuple[np.ndarray, np.ndarray]:
    """NVFP4 quantisation of (groups, rows, k) values as the layer defines it
    (experiments/flashinfer-megamoe-sm100a/nvfp4.py:39-57), in float32 with the narrow casts
    from ml_dtypes: sf = e4m3(clip(blockmax / 6 * gs, 0, 448)), step = f32(sf) / gs,
    q = e2m1_rne(clip(x / step, -6, 6)), a block whose step is zero quantises to zero.
    Returns the VALUES, not bytes: q (groups, rows, k) and sf (groups, rows, k/16) as float64,
    so that q * repeat(sf, 16) is the dequantised operand a float64 reference multiplies."""
    import ml_dtypes

    f32 = np.float32
    g, r, k = x.shape
    xf = np.asarray(x, f32).reshape(g, r, k // 16, 16)
    gs = np.asarray(global_scale, f32).reshape(g, 1, 1)
    sf = np.clip(np.max(np.abs(xf), axis=-1) / f32(6.0) * gs, f32(0.0), f32(448.0)).astype(ml_dtypes.float8_e4m3fn)
    step = sf.astype(f32) / gs
    safe = np.where(step == 0.0, f32(1.0), step)
    live = (step > 0.0).astype(f32)
    q = np.clip(xf / safe[..., None] * live[..., None], f32(-6.0), f32(6.0)).astype(ml_dtypes.float4_e2m1fn)
    return q.astype(np.float64).reshape(g, r, k), sf.astype(np.float64)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float64 / float32 values rounded to the nearest bfloat16 (ties to even), as float32."""
    import ml_dtypes

    return np.asarray(x, np.float32).astype(ml_dtypes.bfloat16).astype(np.float32)
