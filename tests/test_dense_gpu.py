"""Dense fp16 / bf16 GEMM against the float64 oracle (a.double() @ b.double(), the
reference's oracle for its dense problem, experiments/hopper_gemm/ref_cutedsl.py:70).
Exact on small-integer operands; for N(0,1)/sqrt(k) operands the bound is one output ulp plus
a floor: |err| <= 2^-10 |ref| + 1e-3 rms(ref) for fp16 (2^-7 for bf16), and the quantile gate
with cuBLAS as the reference arm."""

import numpy as np
import pytest
import torch

from oracle import gate

pytestmark = pytest.mark.gpu


def _tol(got, ref, rel):
    err = np.abs(got - ref)
    bound = rel * np.abs(ref) + 1e-3 * np.sqrt(np.mean(ref ** 2))
    assert np.all(err <= bound), float((err / bound).max())


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 256, 512), (512, 768, 1024), (384, 520, 200),
                                   (100, 72, 40), (1024, 1024, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_exact_integers(m, n, k, dtype):
    from mosaicist_b200 import _lib, ops

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    hi = 4 if dtype == torch.float16 else 2          # bf16 holds integers exactly only up to 256
    a = torch.randint(1 - hi, hi, (m, k), device="cuda", generator=g).to(dtype)
    b = torch.randint(1 - hi, hi, (k, n), device="cuda", generator=g).to(dtype)
    if k > 512:                          # keep every partial sum exactly representable in the output
        a = a * (torch.rand((m, k), device="cuda", generator=g) < 0.05).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    ops.gemm_f16(a, b, out=out)
    assert _lib.status_word() == 0
    ref = a.double().cpu().numpy() @ b.double().cpu().numpy()
    assert np.abs(ref).max() <= (2048 if dtype == torch.float16 else 256)
    assert np.count_nonzero(ref) > ref.size // 2
    assert np.array_equal(out.double().cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k,max_ctas", [(256, 1024, 64, 2), (512, 1024, 512, 4), (384, 520, 200, 2),
                                            (768, 1600, 1024, 6), (100, 1000, 40, 2), (512, 2048, 4096, 8)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_wide_tiles_exact_and_equal_to_narrow(m, n, k, max_ctas, dtype):
    """The 256 x 512 tile form (two MMAs per K step sharing the A stage), reached here by
    shrinking the grid until every CTA pair has at least two wide tiles: exact on integer
    operands, and bit-identical to the 256 x 256 form (a negative max_ctas forces that one)."""
    from mosaicist_b200 import _lib, ops

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    hi = 4 if dtype == torch.float16 else 2
    a = torch.randint(1 - hi, hi, (m, k), device="cuda", generator=g).to(dtype)
    b = torch.randint(1 - hi, hi, (k, n), device="cuda", generator=g).to(dtype)
    if k > 512:
        a = a * (torch.rand((m, k), device="cuda", generator=g) < 0.05).to(dtype)
    assert ((m + 255) // 256) * ((n + 511) // 512) >= max_ctas      # the launcher picks the wide form
    wide = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    narrow = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    ops.gemm_f16(a, b, out=wide, max_ctas=max_ctas)
    ops.gemm_f16(a, b, out=narrow, max_ctas=-max_ctas)
    assert _lib.status_word() == 0
    ref = a.double().cpu().numpy() @ b.double().cpu().numpy()
    assert np.count_nonzero(ref) > ref.size // 2
    assert np.array_equal(wide.double().cpu().numpy(), ref)
    assert torch.equal(wide, narrow)
    # random operands: the two forms accumulate in the same order, so they agree bit for bit
    a = (torch.randn((m, k), device="cuda", generator=g) / k ** 0.5).to(dtype)
    b = (torch.randn((k, n), device="cuda", generator=g) / k ** 0.5).to(dtype)
    assert torch.equal(ops.gemm_f16(a, b, max_ctas=max_ctas), ops.gemm_f16(a, b, max_ctas=-max_ctas))
    assert _lib.status_word() == 0


@pytest.mark.parametrize("dtype,rel", [(torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -7)])
def test_dense_random_and_column_shards(dtype, rel):
    from mosaicist_b200 import _lib, ops

    m, n, k = 512, 1024, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    a = (torch.randn((m, k), device="cuda", generator=g) / k ** 0.5).to(dtype)
    b = (torch.randn((k, n), device="cuda", generator=g) / k ** 0.5).to(dtype)
    out = ops.gemm_f16(a, b)
    ref = a.double().cpu().numpy() @ b.double().cpu().numpy()
    got = out.double().cpu().numpy()
    _tol(got, ref, rel)
    # the gate's reference arm is a kernel of the same class on the same inputs (cuBLAS through
    # torch.matmul), as the reference uses it: candidate and reference kernel against the oracle
    lib_out = torch.matmul(a, b).double().cpu().numpy()
    rep = gate.compare_outputs(lib_out, got, ref, "f16" if dtype == torch.float16 else "bf16")
    assert rep.passed, rep.failures
    # N-sharded form: two column shards written into one output, no collective
    out2 = torch.empty_like(out)
    for cols in (slice(0, 512), slice(512, 1024)):
        ops.gemm_f16(a, b[:, cols], out=out2[:, cols])
    assert _lib.status_word() == 0
    assert torch.equal(out, out2)
