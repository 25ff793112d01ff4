"""Pins the CPU oracle: against vectors produced by the reference's own code
(tests/golden/make_golden.py) and against the known-answer checks of the reference's
experiments/flashinfer-megamoe-sm100a/test_nvfp4.py."""

import json
import pathlib

import ml_dtypes
import numpy as np
import pytest

from oracle import gate, nvfp4 as O

GOLD = pathlib.Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def g():
    return np.load(GOLD / "nvfp4_golden.npz")


def test_quantize_matches_reference_vectors(g):
    q, sf = O.quantize_nvfp4(g["q_x"], g["q_gs"])
    assert np.array_equal(O.global_scale_for(g["q_x"]), g["q_gs"])
    assert np.array_equal(q.view(np.uint8), g["q_q"])
    assert np.array_equal(sf.view(np.uint8), g["q_sf"])
    assert np.array_equal(O.dequantize_nvfp4(q, sf, g["q_gs"]), g["q_back"])
    q2, sf2 = O.quantize_nvfp4(g["q_x"], g["q2_gs"])
    assert np.array_equal(q2.view(np.uint8), g["q2_q"])
    assert np.array_equal(sf2.view(np.uint8), g["q2_sf"])
    # the fixture really exercises the edge cases it claims to
    assert (g["q_sf"][0, 0, 0] == 0) and (g["q2_sf"].max() == 0x7E)  # zero block; clipped to 448


def test_gemm_reference_matches_reference_vectors(g):
    a_gs, b_gs = O.global_scale_for(g["g_a"]), O.global_scale_for(g["g_b"])
    a_q, a_sf = O.quantize_nvfp4(g["g_a"], a_gs)
    b_q, b_sf = O.quantize_nvfp4(g["g_b"], b_gs)
    out = O.masked_grouped_gemm_reference(a_q, a_sf, a_gs, b_q, b_sf, b_gs, g["g_alpha"],
                                          g["g_masked_m"])
    got, want = np.asarray(out, np.float32), g["g_out"]
    assert np.all(got[1, 5:] == 0) and np.all(want[1, 5:] == 0)
    # fp32 summation order differs between einsum and matmul: allow one bf16 ulp
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6)) <= 2.0 ** -7
    assert np.mean(got == want) > 0.95
    # and the float64 oracle agrees with the fp32 reference to bf16 accuracy
    f64 = O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, g["g_alpha"] / (a_gs * b_gs), g["g_masked_m"])
    ok, worst = O.tolerance_ok(want, f64)
    assert ok, worst


def test_silu_mul_and_moe_match_reference_vectors(g):
    assert np.array_equal(O.silu_mul(g["s_in"].astype(ml_dtypes.bfloat16)), g["s_out"])
    w1_gs, w2_gs = O.global_scale_for(g["m_w1"]), O.global_scale_for(g["m_w2"])
    w1_q, w1_sf = O.quantize_nvfp4(g["m_w1"], w1_gs)
    w2_q, w2_sf = O.quantize_nvfp4(g["m_w2"], w2_gs)
    hidden = g["m_hidden"].astype(ml_dtypes.bfloat16)
    out = O.moe_reference(hidden, w1_q, w1_sf, w1_gs, g["m_w1_alpha"], w2_q, w2_sf, w2_gs,
                          g["m_w2_alpha"], g["m_masked_m"], O.global_scale_for(g["m_hidden"]),
                          g["m_a2_gs"])
    got, want = np.asarray(out, np.float32), g["m_out"]
    assert np.all(got[1, 3:] == 0)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() / scale < 1e-1            # test_kernels.py:96-102 bounds
    assert np.sqrt(np.mean((got - want) ** 2)) / scale < 1e-2
    assert np.mean(got == want) > 0.9


def test_scale_tiling_matches_reference_vectors(g):
    tiled = O.to_mma_scale_layout(g["t_in"])
    assert np.array_equal(tiled, g["t_out"])
    assert np.array_equal(O.from_mma_scale_layout(tiled, 200), g["t_back"])
    assert np.array_equal(g["t_back"], g["t_in"])


# --- the reference's own known-answer checks (test_nvfp4.py) ----------------------

def test_exact_values_survive():            # test_nvfp4.py:27-40
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.5, -3.0, -6.0], np.float32)
    x = np.tile(grid, (1, 4, 4))[:, :, :48]
    gs = np.array([448.0 * 6.0 / 6.0], np.float32)
    q, sf = O.quantize_nvfp4(x, gs)
    assert np.array_equal(O.dequantize_nvfp4(q, sf, gs), x)


def test_quantization_error_bounded():      # test_nvfp4.py:43-61
    x = np.random.default_rng([0, 0]).standard_normal((2, 128, 256)).astype(np.float32)
    gs = O.global_scale_for(x)
    q, sf = O.quantize_nvfp4(x, gs)
    back = O.dequantize_nvfp4(q, sf, gs)
    step = sf.astype(np.float32) / gs.reshape(2, 1, 1)
    assert np.max(np.abs(back - x) - np.repeat(step, 16, axis=-1)) <= 0


def test_scale_layout_roundtrip_and_indices():   # test_nvfp4.py:64-97
    rng = np.random.default_rng([1, 0])
    sf = rng.integers(0, 100, (256, 32)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    tiled = O.to_mma_scale_layout(sf)
    assert tiled.shape == (2, 8, 32, 16)
    assert np.array_equal(O.from_mma_scale_layout(tiled, 256).view(np.uint8), sf.view(np.uint8))
    mn, ks = 256, 16
    src = (np.arange(mn * ks, dtype=np.float32).reshape(mn, ks) % 240).astype(ml_dtypes.float8_e4m3fn)
    t = O.to_mma_scale_layout(src).astype(np.float32)
    s = src.astype(np.float32)
    for row in range(mn):
        for col in range(ks):
            tt, a, b = row // 128, (row % 128) // 32, row % 32
            c, d = col // 4, col % 4
            assert t[tt, c, b, 4 * a + d] == s[row, col]


def test_moe_reference_runs_and_masks():    # test_nvfp4.py:100-117
    l, m, k, n = 2, 128, 256, 128
    rng = np.random.default_rng([2, 0])
    hidden = rng.standard_normal((l, m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    w1 = (rng.standard_normal((l, 2 * n, k)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((l, k, n)) * 0.05).astype(np.float32)
    w1_gs, w2_gs = O.global_scale_for(w1), O.global_scale_for(w2)
    w1_q, w1_sf = O.quantize_nvfp4(w1, w1_gs)
    w2_q, w2_sf = O.quantize_nvfp4(w2, w2_gs)
    ones = np.ones((l,), np.float32)
    out = O.moe_reference(hidden, w1_q, w1_sf, w1_gs, ones, w2_q, w2_sf, w2_gs, ones,
                          np.array([m, m // 2], np.int32),
                          O.global_scale_for(hidden.astype(np.float32)),
                          np.full((l,), 8.0, np.float32))
    o = out.astype(np.float32)
    assert out.shape == (l, m, k) and np.all(np.isfinite(o)) and np.all(o[1, m // 2:] == 0)
    assert np.count_nonzero(o[0]) > o[0].size // 2


def test_exact_operands_are_exact_in_fp32():   # test_kernels.py:28-36,85-86
    rng = np.random.default_rng([0, 7])
    a_q, a_sf = O.exact_operands(rng, 2, 32, 128)
    b_q, b_sf = O.exact_operands(rng, 2, 48, 128)
    alpha = np.exp2(rng.integers(-1, 2, 2)).astype(np.float32)
    ones = np.ones(2, np.float32)
    mm = np.array([32, 13], np.int32)
    f32 = O.masked_grouped_gemm_reference(a_q, a_sf, ones, b_q, b_sf, ones, alpha, mm, np.float32)
    f64 = O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, alpha, mm)
    assert np.array_equal(f32.astype(np.float64), f64)


def test_pack_unpack_e2m1():
    q = np.array([[0.5, -6.0, 1.0, 0.0]], np.float32).astype(ml_dtypes.float4_e2m1fn)
    p = O.pack_e2m1(q)
    assert p.tolist() == [[0x1 | (0xF << 4), 0x2 | (0x0 << 4)]]
    assert np.array_equal(O.unpack_e2m1(p).view(np.uint8), q.view(np.uint8))


# --- the numerics gate restatement ------------------------------------------------

def _parse(v):
    return float(v) if isinstance(v, str) else v


def test_gate_formats_match_reference_vectors():
    gold = json.loads((GOLD / "gate_golden.json").read_text())
    x = np.array([_parse(v) for v in gold["x"]], np.float64)
    for fmt, want in gold["fmt"].items():
        r = gate.round_to_format(x, fmt)
        w = np.array([_parse(v) for v in want["round"]], np.float64)
        assert np.array_equal(r, w, equal_nan=True), fmt
        assert np.array_equal(gate.ulp(x[np.isfinite(x)], fmt), np.array(want["ulp"])), fmt
        assert gate.ordinal(r[np.isfinite(r)], fmt).tolist() == want["ordinal"], fmt


def test_gate_verdicts_match_reference_vectors():
    gold = json.loads((GOLD / "gate_golden.json").read_text())["gate"]
    rng = np.random.default_rng([0, 1])
    # replay make_golden.py's stream
    rng.standard_normal(40); rng.integers(-20, 20, 40)
    oracle = rng.standard_normal((64, 48)) * 8.0
    ref = gate.round_to_format(oracle, "bf16")
    cases = {
        "same": ref.copy(),
        "one_ulp_noise": gate.round_to_format(oracle * (1 + rng.choice([-1, 0, 1], oracle.shape) * 2.0 ** -8), "bf16"),
        "sloppy": gate.round_to_format(oracle * 1.05, "bf16"),
    }
    nan_case = ref.copy(); nan_case[3, 4] = np.nan
    cases["nan"] = nan_case
    seen = set()
    for name, cand in cases.items():
        rep = gate.compare_outputs(ref, cand, oracle, "bf16")
        want = gold["cases"][name]
        assert rep.passed == want["passed"], name
        assert rep.special_mismatch == want["special"] and rep.max_ulp_ref_vs_cand == want["max_ulp"]
        assert rep.bitwise_equal_fraction == pytest.approx(want["bitwise"])
        for got, w in zip(rep.rows, want["rows"]):
            assert got[0] == w[0] and got[4] == w[4]
            assert got[1] == pytest.approx(w[1]) and got[2] == pytest.approx(w[2])
        seen.add(rep.passed)
    assert seen == {True, False}


# --- the bf16 x int4 oracle against the reference's own dequant / reference ----------

def test_int4_oracle_matches_reference_vectors():
    """oracle/mixed_int4.py against outputs of the reference's
    ports/hopper_mixed_dtype_grouped_gemm/problems.py (dequant :75-81, reference :84-87) run on
    int4-valued weights (tests/golden/make_golden.py): the dequantised weights bit for bit, the
    product within fp16 output rounding of the reference's fp32 accumulation."""
    import ml_dtypes

    from oracle import mixed_int4 as X4

    gold = np.load(GOLD / "int4_golden.npz")
    for i in range(int(gold["cases"])):
        A, Bq, scale = gold[f"c{i}_A"], gold[f"c{i}_Bq"], gold[f"c{i}_scale"]
        c, alpha = int(gold[f"c{i}_c"]), float(gold[f"c{i}_alpha"])
        assert Bq.min() == -8 and Bq.max() == 7
        w = X4.dequant(Bq, scale.astype(ml_dtypes.bfloat16), c)
        assert np.array_equal(np.asarray(w, np.float32), gold[f"c{i}_dequant"]), i
        # pack / unpack round trip of the byte layout the library consumes
        packed = X4.pack_int4(Bq)
        lo, hi = (packed & 0xF).astype(np.int8), (packed >> 4).astype(np.int8)
        back = np.stack([lo, hi], axis=-1).reshape(Bq.shape)
        assert np.array_equal(np.where(back >= 8, back - 16, back), Bq)
        m = A.shape[0]
        ref64 = X4.ragged_gemm_f64(A.astype(ml_dtypes.bfloat16), w[None], [0], [m], [alpha])
        want = gold[f"c{i}_reference"].astype(np.float64)          # fp16(alpha * fp32 accumulation)
        assert np.count_nonzero(want) > want.size // 2
        err = np.abs(ref64 - want)
        assert np.all(err <= 2.0 ** -10 * np.abs(ref64) + 1e-3 * np.sqrt(np.mean(ref64 ** 2)))
        if i == 0:      # small integers and quarter scales: every product is exact, so are the sums
            assert np.array_equal(ref64, want)
