"""Byte-level decoders for the narrow formats the library consumes, on numpy.

Used by the capture modules' `reference()` hooks (the float64 opinion Mosaicist's numerics
gate asks every module for, src/mosaicist/capture.py:254-264) and by host-side input
preparation.  Nothing here runs on the hot path.
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
