"""The reference's numerics gate restated (test infrastructure, not product).

Follows src/mosaicist/verify/formats.py:33-110 (value-based ULP arithmetic on
float64 arrays) and src/mosaicist/verify/numerics.py:81-136 (quantile gate with
delta = 0.10, tau = 1 ulp, quantiles 0.5 / 0.99 / 1.0, NaN/Inf pattern equality).
The reference package cannot travel to the GPU machine, so the parity tests use
this restatement; tests/golden/gate_golden.json holds outputs of the reference's
own functions on seeded inputs and tests/test_oracle_golden.py checks this file
against them.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

# name -> (explicit mantissa bits, exponent of smallest normal, largest finite, has inf)
_FORMATS = {
    "float32": (23, -126, float(np.finfo(np.float32).max), True),
    "float16": (10, -14, 65504.0, True),
    "bfloat16": (7, -126, float.fromhex("0x1.fep127"), True),
    "float8_e4m3fn": (3, -6, 448.0, False),
    "float8_e5m2": (2, -14, 57344.0, True),
}
_SHORT = {"f32": "float32", "f16": "float16", "half": "float16", "bf16": "bfloat16",
          "e4m3": "float8_e4m3fn", "e5m2": "float8_e5m2"}


def _fmt(name: str):
    full = _SHORT.get(name, name)
    if full not in _FORMATS:
        raise KeyError(f"unknown float format {name!r}")
    return full, _FORMATS[full]


def _binade(mag: np.ndarray, emin: int) -> np.ndarray:
    """floor(log2 |x|), clamped below at emin (subnormals and zero use emin)."""
    _, e = np.frexp(mag)
    e = e.astype(np.int64) - 1
    e[mag == 0] = emin
    return np.maximum(e, emin)


def ulp(x, fmt: str) -> np.ndarray:
    """Spacing of the format in the binade that holds |x|.  formats.py:68-72."""
    _, (mant, emin, _, _) = _fmt(fmt)
    mag = np.abs(np.asarray(x, np.float64))
    return np.ldexp(1.0, _binade(mag, emin) - mant)


def round_to_format(x, fmt: str) -> np.ndarray:
    """Round-to-nearest-even into the format, as float64; overflow -> inf, or the
    largest finite value for formats without inf.  formats.py:75-91."""
    _, (mant, emin, big, has_inf) = _fmt(fmt)
    x = np.asarray(x, np.float64)
    step = ulp(x, fmt)
    with np.errstate(invalid="ignore", over="ignore"):
        r = np.rint(x / step) * step
    fin = np.isfinite(x)
    too_big = fin & (np.abs(r) > big)
    r = np.where(too_big, np.copysign(np.inf if has_inf else big, x), r)
    return np.where(fin, r, x)


def ordinal(x, fmt: str) -> np.ndarray:
    """Signed index of each representable value in the format's ordered value set
    (+0 and -0 are both 0).  formats.py:94-110."""
    _, (mant, emin, _, _) = _fmt(fmt)
    x = np.asarray(x, np.float64)
    mag = np.abs(x)
    e = _binade(mag, emin)
    step = np.ldexp(1.0, e - mant)
    is_normal = mag >= 2.0 ** emin
    base = np.where(is_normal, np.ldexp(1.0, e), 0.0)
    inside = np.rint((mag - base) / step).astype(np.int64)
    idx = np.where(is_normal, (e - emin + 1) * (1 << mant) + inside, inside)
    return np.where(np.signbit(x) & (mag > 0), -idx, idx)


@dataclass
class GateReport:
    passed: bool
    fmt: str
    n: int
    rows: list = field(default_factory=list)        # (q, ref_err, cand_err, bound, ok)
    bitwise_equal_fraction: float = 0.0
    max_ulp_ref_vs_cand: int = 0
    special_mismatch: int = 0
    failures: list = field(default_factory=list)


def compare_outputs(ref, cand, oracle, fmt: str, quantiles=(0.5, 0.99, 1.0),
                    delta: float = 0.10, tau_ulp: float = 1.0) -> GateReport:
    """Q_q(e_cand) <= (1 + delta) Q_q(e_ref) + tau for each quantile, with e the error
    against the float64 oracle in ULPs of `fmt`; the NaN/Inf pattern of ref and cand must
    match.  numerics.py:81-136."""
    full, _ = _fmt(fmt)
    ref = np.asarray(ref, np.float64)
    cand = np.asarray(cand, np.float64)
    oracle = np.asarray(oracle, np.float64)
    if not (ref.shape == cand.shape == oracle.shape):
        return GateReport(False, full, int(cand.size), failures=[
            f"shape mismatch: ref {ref.shape}, cand {cand.shape}, oracle {oracle.shape}"])
    rep = GateReport(True, full, int(cand.size))

    def inf_sign(a):
        return np.where(np.isinf(a), np.sign(a), 0)

    special = (np.isnan(ref) != np.isnan(cand)) | (inf_sign(ref) != inf_sign(cand))
    rep.special_mismatch = int(special.sum())
    if rep.special_mismatch:
        rep.failures.append(f"NaN/Inf pattern differs at {rep.special_mismatch} positions")

    same = ((ref == cand) & (np.signbit(ref) == np.signbit(cand))) | (np.isnan(ref) & np.isnan(cand))
    rep.bitwise_equal_fraction = float(same.mean()) if same.size else 1.0

    ok = np.isfinite(ref) & np.isfinite(cand) & np.isfinite(oracle)
    if ok.any():
        u = ulp(oracle, fmt)
        with np.errstate(invalid="ignore"):
            e_ref = (np.abs(ref - oracle) / u)[ok]
            e_cand = (np.abs(cand - oracle) / u)[ok]
        for q in quantiles:
            qr, qc = float(np.quantile(e_ref, q)), float(np.quantile(e_cand, q))
            bound = (1 + delta) * qr + tau_ulp
            rep.rows.append((q, qr, qc, bound, qc <= bound))
            if qc > bound:
                rep.failures.append(f"q{q:g} error {qc:.3g} ulp exceeds bound {bound:.3g}")
        rep.max_ulp_ref_vs_cand = int(np.abs(ordinal(ref[ok], fmt) - ordinal(cand[ok], fmt)).max())
    rep.passed = not rep.failures
    return rep


def gate_bf16(cand, oracle) -> GateReport:
    """Gate a bf16 output against the float64 oracle with the oracle's own bf16 rounding
    standing in as the reference arm — the reference's practice when no second kernel
    shares the inputs (experiments/loop/gen_v0_check.py:36-44)."""
    return compare_outputs(round_to_format(oracle, "bf16"), cand, oracle, "bf16")
