"""Generate the golden fixtures in this directory from the reference's own code.

Run once where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

Two sources are executed, neither is copied:

* `src/mosaicist/verify` (pure numpy) is imported as is; its `round_to_format`, `ulp`,
  `ordinal` and `compare_outputs` are run on seeded inputs -> gate_golden.json.
* `experiments/flashinfer-megamoe-sm100a/nvfp4.py` is "plain JAX" and JAX cannot be
  installed here, so the module is executed on top of a stand-in `jax` whose
  `jax.numpy` is numpy plus the ml_dtypes narrow floats (the same casts JAX uses) ->
  nvfp4_golden.npz.  The stand-in only forwards names, with one exception: `jax.nn.sigmoid`
  is written out here as 1 / (1 + exp(-x)) in float32, so the silu_mul vectors rest on this
  file's statement of the sigmoid, not on JAX's; every other arithmetic statement that runs
  is the reference's.

* `ports/hopper_mixed_dtype_grouped_gemm/problems.py` (plain torch, runs on the CPU) is
  imported as is; its `dequant` and `reference` are run on groups whose quantised weights are
  int4 values held in int8, with bf16 group scales -> int4_golden.npz.  This pins
  oracle/mixed_int4.py, which the reference itself never exercised with int4.

The fixtures are small (a few KB) and are what tests/test_oracle_golden.py pins the
oracle against.
"""

from __future__ import annotations

import json
import pathlib
import sys
import types

import ml_dtypes
import numpy as np

HERE = pathlib.Path(__file__).resolve().parent


def _install_numpy_jax():
    jnp = types.ModuleType("jax.numpy")
    for name in ("max", "abs", "where", "clip", "einsum", "arange", "split", "pad", "array",
                 "float32", "int32", "full", "ones", "exp2", "tile"):
        setattr(jnp, name, getattr(np, name))
    jnp.float4_e2m1fn = ml_dtypes.float4_e2m1fn
    jnp.float8_e4m3fn = ml_dtypes.float8_e4m3fn
    jnp.bfloat16 = ml_dtypes.bfloat16
    nn = types.ModuleType("jax.nn")
    nn.sigmoid = lambda x: (np.float32(1.0) / (np.float32(1.0) + np.exp(-x))).astype(np.float32)
    jax = types.ModuleType("jax")
    jax.numpy, jax.nn, jax.Array = jnp, nn, np.ndarray
    sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.nn": nn})


def nvfp4_golden(ref_root: pathlib.Path) -> dict:
    _install_numpy_jax()
    sys.path.insert(0, str(ref_root / "experiments" / "flashinfer-megamoe-sm100a"))
    import nvfp4 as R  # the reference module, executed unmodified

    out = {}
    rng = np.random.default_rng([0, 0])
    # quantize: plain, with a zero block, with values that clip, with a tiny block
    x = rng.standard_normal((2, 8, 64)).astype(np.float32)
    x[0, 0, :16] = 0.0
    x[0, 1, 16:32] *= 1e-6
    x[1, 2, 5] = 40.0
    gs = R.global_scale_for(x)
    q, sf = R.quantize_nvfp4(x, gs)
    out.update(q_x=x, q_gs=gs, q_q=q.view(np.uint8), q_sf=sf.view(np.uint8),
               q_back=R.dequantize_nvfp4(q, sf, gs))
    # a fixed global scale that forces the e4m3 clip and sub-normal scales
    gs2 = np.array([4096.0, 0.01], np.float32)
    q2, sf2 = R.quantize_nvfp4(x, gs2)
    out.update(q2_gs=gs2, q2_q=q2.view(np.uint8), q2_sf=sf2.view(np.uint8))

    # grouped GEMM reference with masking and alpha
    l, m, n, k = 2, 16, 24, 64
    a = rng.standard_normal((l, m, k)).astype(np.float32)
    b = (rng.standard_normal((l, n, k)) * 0.05).astype(np.float32)
    a_gs, b_gs = R.global_scale_for(a), R.global_scale_for(b)
    a_q, a_sf = R.quantize_nvfp4(a, a_gs)
    b_q, b_sf = R.quantize_nvfp4(b, b_gs)
    alpha = np.array([0.75, 1.5], np.float32)
    masked_m = np.array([16, 5], np.int32)
    g = R.masked_grouped_gemm_reference(a_q, a_sf, a_gs, b_q, b_sf, b_gs, alpha, masked_m)
    out.update(g_a=a, g_b=b, g_alpha=alpha, g_masked_m=masked_m,
               g_out=np.asarray(g, np.float32))

    # silu_mul and the full MoE reference
    gu = rng.standard_normal((2, 4, 32)).astype(np.float32).astype(ml_dtypes.bfloat16)
    out.update(s_in=np.asarray(gu, np.float32), s_out=R.silu_mul(gu))
    l, m, k, n = 2, 8, 64, 32
    hidden = rng.standard_normal((l, m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    w1 = (rng.standard_normal((l, 2 * n, k)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((l, k, n)) * 0.05).astype(np.float32)
    w1_gs, w2_gs = R.global_scale_for(w1), R.global_scale_for(w2)
    w1_q, w1_sf = R.quantize_nvfp4(w1, w1_gs)
    w2_q, w2_sf = R.quantize_nvfp4(w2, w2_gs)
    w1_alpha = np.array([0.5, 1.25], np.float32)
    w2_alpha = np.array([1.5, 0.75], np.float32)
    mm = np.array([8, 3], np.int32)
    in_gs = R.global_scale_for(np.asarray(hidden, np.float32))
    a2_gs = np.array([8.0, 8.0], np.float32)
    moe = R.moe_reference(hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha,
                          mm, in_gs, a2_gs)
    out.update(m_hidden=np.asarray(hidden, np.float32), m_w1=w1, m_w2=w2,
               m_w1_alpha=w1_alpha, m_w2_alpha=w2_alpha, m_masked_m=mm, m_a2_gs=a2_gs,
               m_out=np.asarray(moe, np.float32))

    # scale tiling
    sfm = (np.arange(200 * 8) % 240).astype(np.uint8).reshape(200, 8)
    tiled = R.to_mma_scale_layout(sfm)
    out.update(t_in=sfm, t_out=np.asarray(tiled), t_back=np.asarray(R.from_mma_scale_layout(tiled, 200)))
    return out


def gate_golden(ref_root: pathlib.Path) -> dict:
    sys.path.insert(0, str(ref_root / "src"))
    from mosaicist.verify import formats as F
    from mosaicist.verify import numerics as N

    rng = np.random.default_rng([0, 1])
    x = np.concatenate([rng.standard_normal(40) * np.exp2(rng.integers(-20, 20, 40)),
                        [0.0, -0.0, 1e-40, 3e38, 70000.0, 500.0, np.inf, -np.inf, np.nan]])
    out = {"x": [float(v) if np.isfinite(v) else repr(float(v)) for v in x], "fmt": {}}
    for fmt in ("f32", "f16", "bf16", "e4m3", "e5m2"):
        r = F.round_to_format(x, fmt)
        finite = np.isfinite(r)
        out["fmt"][fmt] = {
            "round": [float(v) if np.isfinite(v) else repr(float(v)) for v in r],
            "ulp": [float(v) for v in F.ulp(x[np.isfinite(x)], fmt)],
            "ordinal": [int(v) for v in F.ordinal(r[finite], fmt)],
        }
    # gate verdicts on seeded cases: a faithful candidate, a sloppy one, a NaN mismatch
    oracle = rng.standard_normal((64, 48)) * 8.0
    ref = F.round_to_format(oracle, "bf16")
    cases = {
        "same": ref.copy(),
        "one_ulp_noise": F.round_to_format(oracle * (1 + rng.choice([-1, 0, 1], oracle.shape) * 2.0 ** -8), "bf16"),
        "sloppy": F.round_to_format(oracle * 1.05, "bf16"),
    }
    nan_case = ref.copy()
    nan_case[3, 4] = np.nan
    cases["nan"] = nan_case
    out["gate"] = {"seed": [0, 1], "cases": {}}
    for name, cand in cases.items():
        rep = N.compare_outputs(ref, cand, oracle, "bf16")
        out["gate"]["cases"][name] = {
            "passed": bool(rep.passed),
            "rows": [[r.q, r.ref_err, r.cand_err, r.bound, bool(r.ok)] for r in rep.quantiles],
            "bitwise": rep.bitwise_equal_fraction,
            "max_ulp": rep.max_ulp_ref_vs_cand,
            "special": rep.special_mismatch,
        }
    return out


def int4_golden(ref_root: pathlib.Path) -> dict:
    """dequant() and reference() of the reference's mixed-dtype port on int4-valued weights."""
    import torch

    sys.path.insert(0, str(ref_root / "ports" / "hopper_mixed_dtype_grouped_gemm"))
    import problems as P   # the reference module, executed unmodified

    g = torch.Generator(device="cpu").manual_seed(7)
    out = {}
    # (m, n, k, scale group): small-integer activations as the reference's own generator draws
    # them, then N(0,1) activations and |N(0, 0.02)| scales as the benchmark configuration has them
    cases = [(24, 16, 256, 128, "ints"), (40, 32, 384, 128, "normal"), (8, 16, 128, 64, "normal")]
    for i, (m, n, k, c, kind) in enumerate(cases):
        if kind == "ints":
            A = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16)
            scale = (torch.randint(1, 5, (n, k // c), generator=g).to(torch.float32) / 4).to(torch.bfloat16)
        else:
            A = torch.randn((m, k), generator=g).to(torch.bfloat16)
            scale = (torch.randn((n, k // c), generator=g) * 0.02).abs().to(torch.bfloat16)
        Bq = torch.randint(-8, 8, (n, k), generator=g).to(torch.int8)
        alpha = [1.0, 0.5, 2.0][i]
        gp = P.Group(m, n, k, alpha, 0.0, A, Bq, scale, torch.zeros((m, n), dtype=torch.float16),
                     torch.empty((m, n), dtype=torch.float16))
        out.update({f"c{i}_A": A.float().numpy(), f"c{i}_Bq": Bq.numpy(), f"c{i}_scale": scale.float().numpy(),
                    f"c{i}_c": np.int32(c), f"c{i}_alpha": np.float32(alpha),
                    f"c{i}_dequant": P.dequant(gp).float().numpy(),
                    f"c{i}_reference": P.reference(gp).float().numpy()})
    out["cases"] = np.int32(len(cases))
    return out


def main():
    import os

    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MOSAICIST_REFERENCE")
    if not where:
        raise SystemExit("usage: make_golden.py /path/to/reference  (or set MOSAICIST_REFERENCE)")
    ref_root = pathlib.Path(where)
    np.savez_compressed(HERE / "nvfp4_golden.npz", **nvfp4_golden(ref_root))
    (HERE / "gate_golden.json").write_text(json.dumps(gate_golden(ref_root), indent=1))
    np.savez_compressed(HERE / "int4_golden.npz", **int4_golden(ref_root))
    print("wrote", HERE / "nvfp4_golden.npz", HERE / "gate_golden.json", HERE / "int4_golden.npz")


if __name__ == "__main__":
    main()
