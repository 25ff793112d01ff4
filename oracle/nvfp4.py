"""NVFP4 arithmetic restated on numpy + ml_dtypes (test infrastructure, not product).

Restates, function by function, the reference's plain-JAX arithmetic model of the
block-scaled grouped GEMM and the MoE layer built on it
(experiments/flashinfer-megamoe-sm100a/nvfp4.py) and the float64 oracle of the
candidate module (experiments/loop/cand_pallas_gemm.py:54-63).  JAX is not
installable where this runs, so the same formulas are written against numpy; the
narrow float casts come from ml_dtypes, the package JAX itself uses for them.

Pinning: tests/golden/make_golden.py executes the reference's own nvfp4.py on top of
a numpy-backed stand-in for the few jax.numpy calls it makes and stores the results;
tests/test_oracle_golden.py checks this module against those stored vectors and
against the five known-answer checks of the reference's test_nvfp4.py.
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

SF_VEC_SIZE = 16          # nvfp4.py:21
FP4_MAX = 6.0             # nvfp4.py:23
SF_MAX = 448.0            # nvfp4.py:25
FP4 = ml_dtypes.float4_e2m1fn
E4M3 = ml_dtypes.float8_e4m3fn
BF16 = ml_dtypes.bfloat16

_f32 = np.float32


def global_scale_for(x: np.ndarray) -> np.ndarray:
    """Per-group `(6 * 448) / amax`, amax == 0 -> 1.  nvfp4.py:29-36."""
    amax = np.max(np.abs(x.astype(_f32)), axis=(-2, -1))
    return (_f32(FP4_MAX * SF_MAX) / np.where(amax == 0, _f32(1.0), amax)).astype(_f32)


def quantize_nvfp4(x: np.ndarray, global_scale: np.ndarray):
    """(l, m, k) -> (q e2m1 (l, m, k), sf e4m3 (l, m, k // 16)), row-major scales.

    nvfp4.py:39-57: the block scale is clipped to [0, 448] *before* the e4m3 cast
    (ml_dtypes' e4m3fn does not saturate), the represented step is f32(sf) / gs, a
    zero step quantizes the block to zero, and values are clipped to +-6 before the
    round-to-nearest-even e2m1 cast.
    """
    l, m, k = x.shape
    if k % SF_VEC_SIZE:
        raise ValueError(f"K={k} must be a multiple of SF_VEC_SIZE={SF_VEC_SIZE}")
    xf = x.astype(_f32).reshape(l, m, k // SF_VEC_SIZE, SF_VEC_SIZE)
    amax = np.max(np.abs(xf), axis=-1)
    gs = np.asarray(global_scale, _f32).reshape(l, 1, 1)
    sf = np.clip(amax / _f32(FP4_MAX) * gs, _f32(0.0), _f32(SF_MAX)).astype(E4M3)
    step = sf.astype(_f32) / gs
    safe = np.where(step == 0.0, _f32(1.0), step)
    live = np.where(step > 0.0, _f32(1.0), _f32(0.0))
    q = np.clip(xf / safe[..., None] * live[..., None], _f32(-FP4_MAX), _f32(FP4_MAX))
    return q.astype(FP4).reshape(l, m, k), sf


def dequantize_nvfp4(q: np.ndarray, sf: np.ndarray, global_scale: np.ndarray) -> np.ndarray:
    """Inverse of quantize_nvfp4 in fp32.  nvfp4.py:60-65."""
    l, m, k = q.shape
    step = sf.astype(_f32) / np.asarray(global_scale, _f32).reshape(l, 1, 1)
    qf = q.astype(_f32).reshape(l, m, k // SF_VEC_SIZE, SF_VEC_SIZE)
    return (qf * step[..., None]).reshape(l, m, k)


def masked_grouped_gemm_reference(a_q, a_sf, a_gs, b_q, b_sf, b_gs, alpha, masked_m,
                                  out_dtype=BF16) -> np.ndarray:
    """out[l,m,n] = alpha[l] * dequant(A)[l] @ dequant(B)[l].T in fp32, rows >= masked_m
    zeroed, then cast.  nvfp4.py:68-78."""
    a = dequantize_nvfp4(a_q, a_sf, a_gs)
    b = dequantize_nvfp4(b_q, b_sf, b_gs)
    out = np.matmul(a, np.swapaxes(b, -1, -2)) * np.asarray(alpha, _f32).reshape(-1, 1, 1)
    rows = np.arange(out.shape[1])[None, :, None]
    out = np.where(rows < np.asarray(masked_m).reshape(-1, 1, 1), out, _f32(0.0))
    return out.astype(out_dtype)


def grouped_gemm_f64(a_q, a_sf, b_q, b_sf, alpha=None, masked_m=None) -> np.ndarray:
    """float64 oracle: q * repeat(sf, 16), contracted in double precision, no global
    scale.  experiments/loop/cand_pallas_gemm.py:54-63; alpha and masking are the
    extensions masked_grouped_gemm_reference (nvfp4.py:68-78) applies."""
    a = np.asarray(a_q, np.float64) * np.repeat(np.asarray(a_sf, np.float64), SF_VEC_SIZE, axis=-1)
    b = np.asarray(b_q, np.float64) * np.repeat(np.asarray(b_sf, np.float64), SF_VEC_SIZE, axis=-1)
    out = np.matmul(a, np.swapaxes(b, -1, -2))
    if alpha is not None:
        out = out * np.asarray(alpha, np.float64).reshape(-1, 1, 1)
    if masked_m is not None:
        rows = np.arange(out.shape[1])[None, :, None]
        out = np.where(rows < np.asarray(masked_m).reshape(-1, 1, 1), out, 0.0)
    return out


def sigmoid(x: np.ndarray) -> np.ndarray:
    x = x.astype(_f32)
    return (_f32(1.0) / (_f32(1.0) + np.exp(-x))).astype(_f32)


def silu_mul(gateup: np.ndarray) -> np.ndarray:
    """(l, m, 2n) -> (l, m, n) fp32, gate half first, never rounded to bf16.
    nvfp4.py:81-88."""
    gate, up = np.split(gateup.astype(_f32), 2, axis=-1)
    return sigmoid(gate) * gate * up


def moe_reference(hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha,
                  masked_m, input_global_scale, a2_global_scale) -> np.ndarray:
    """quantize -> GEMM1 (bf16 gateup) -> silu_mul -> quantize -> GEMM2.  nvfp4.py:91-108."""
    a_q, a_sf = quantize_nvfp4(hidden, input_global_scale)
    gateup = masked_grouped_gemm_reference(a_q, a_sf, input_global_scale, w1_q, w1_sf, w1_gs,
                                           w1_alpha, masked_m, BF16)
    d_q, d_sf = quantize_nvfp4(silu_mul(gateup), a2_global_scale)
    return masked_grouped_gemm_reference(d_q, d_sf, a2_global_scale, w2_q, w2_sf, w2_gs,
                                         w2_alpha, masked_m, BF16)


def to_mma_scale_layout(sf: np.ndarray) -> np.ndarray:
    """(mn, k_scales) -> (ceil(mn/128), k_scales // 4, 32, 16): row 128t+32a+b, column
    4c+d lands at [t, c, b, 4a+d].  nvfp4.py:121-131."""
    mn, ks = sf.shape
    pad_mn = (mn + 127) // 128 * 128
    if ks % 4:
        raise ValueError(f"k_scales={ks} must be a multiple of 4")
    padded = np.zeros((pad_mn, ks), sf.dtype)
    padded[:mn] = sf
    return (padded.reshape(pad_mn // 128, 4, 32, ks // 4, 4)
            .transpose(0, 3, 2, 1, 4)
            .reshape(pad_mn // 128, ks // 4, 32, 16))


def from_mma_scale_layout(tiled: np.ndarray, mn: int) -> np.ndarray:
    """Inverse of to_mma_scale_layout, dropping padding rows.  nvfp4.py:134-139."""
    mn_tiles, k_tiles, _, _ = tiled.shape
    return (tiled.reshape(mn_tiles, k_tiles, 32, 4, 4)
            .transpose(0, 3, 2, 1, 4)
            .reshape(mn_tiles * 128, k_tiles * 4)[:mn])


def retile(sf: np.ndarray) -> np.ndarray:
    """to_mma_scale_layout over the leading group axis (the reference's jax.vmap,
    moe.py:44)."""
    return np.stack([to_mma_scale_layout(s) for s in sf])


# --- byte-level views the C-ABI consumes ------------------------------------------

def pack_e2m1(q: np.ndarray) -> np.ndarray:
    """e2m1 (..., k) -> uint8 (..., k // 2), element 2i in the low nibble."""
    codes = np.asarray(q, FP4).view(np.uint8) & 0xF
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """Inverse of pack_e2m1."""
    p = np.asarray(packed, np.uint8)
    codes = np.stack([p & 0xF, p >> 4], axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    return codes.astype(np.uint8).view(FP4)


def e4m3_bytes(sf: np.ndarray) -> np.ndarray:
    return np.asarray(sf, E4M3).view(np.uint8)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as float32."""
    return np.asarray(x, _f32).astype(BF16).astype(_f32)


# --- inputs the reference's tests and candidate modules use -----------------------

_EXACT_VALUES = np.array([-4., -3., -2., -1., 0., 1., 2., 3., 4., 6.], _f32)


def exact_operands(rng: np.random.Generator, l: int, rows: int, k: int):
    """Operands that make the whole GEMM exact in fp32 (small integers on the e2m1 grid,
    power-of-two scales 2^[-2, 2]), so kernel and reference must agree bit for bit.
    test_kernels.py:28-36 (values and ranges; the random stream is numpy's, not JAX's)."""
    q = rng.choice(_EXACT_VALUES, size=(l, rows, k)).astype(FP4)
    sf = np.exp2(rng.integers(-2, 3, size=(l, rows, k // SF_VEC_SIZE)).astype(_f32)).astype(E4M3)
    return q, sf


def tolerance_ok(out: np.ndarray, ref64: np.ndarray):
    """|err| <= 2^-7 |ref| + 1e-3 rms(ref), elementwise.  Returns (ok, worst_ratio)."""
    ref64 = np.asarray(ref64, np.float64)
    err = np.abs(np.asarray(out, np.float64) - ref64)
    rms = float(np.sqrt(np.mean(ref64 ** 2))) if ref64.size else 0.0
    bound = 2.0 ** -7 * np.abs(ref64) + 1e-3 * rms
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(bound > 0, err / bound, np.where(err > 0, np.inf, 0.0))
    return bool(np.all(err <= bound)), float(ratio.max()) if ratio.size else 0.0
