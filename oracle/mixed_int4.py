"""bf16 x int4 mixed-dtype grouped GEMM on numpy (test infrastructure, not product).

Follows ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-87: dequant(B)[n, k] =
MmaType(Bq[n, k]) * scale[n, k // c] with the multiply carried out in the MMA type (bf16),
D_g = alpha_g * A_g @ dequant(B_g)^T accumulated in fp32.  The reference checks its fp8
variants against this formula bit for bit on small-integer inputs (check_matrix.py:12-22); it
never ported int4 (README.md:95); its problems.py is plain torch and runs on the CPU, so
tests/golden/make_golden.py executes its `dequant` and `reference` on int4-valued weights and
tests/test_oracle_golden.py pins this file against those vectors (int4_golden.npz).
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16


def pack_int4(q: np.ndarray) -> np.ndarray:
    """int8 values in [-8, 7], (..., k) -> uint8 (..., k/2), element 2i in the low nibble."""
    u = (np.asarray(q, np.int8).astype(np.int16) & 0xF).astype(np.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


def dequant(q: np.ndarray, scales: np.ndarray, group: int) -> np.ndarray:
    """(..., k) int + (..., k/group) bf16 -> bf16, multiply rounded to bf16 (problems.py:75-81)."""
    b = np.asarray(q, np.float32).astype(BF16)
    s = np.repeat(np.asarray(scales, BF16), group, axis=-1)
    return (b.astype(np.float32) * s.astype(np.float32)).astype(BF16)


def ragged_gemm_f64(a_bf16, b_deq, offsets, rows, alpha=None) -> np.ndarray:
    a = np.asarray(a_bf16, np.float64)
    out = np.zeros((a.shape[0], b_deq.shape[1]), np.float64)
    for g, (o, r) in enumerate(zip(offsets, rows)):
        if r > 0:
            y = a[o:o + r] @ np.asarray(b_deq[g], np.float64).T
            out[o:o + r] = y * (1.0 if alpha is None else float(alpha[g]))
    return out
