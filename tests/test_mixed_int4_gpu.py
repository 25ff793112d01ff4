"""bf16 x int4 grouped GEMM against the oracle.  Small-integer inputs with power-of-two-ish
scales make everything exact (the reference's own pattern, problems.py:54-60, check_matrix.py);
random inputs are held to |err| <= 2^-7 |ref| + 1e-3 rms(ref) and the quantile gate with a
cuBLAS bf16 GEMM on the same operands as the reference arm."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import gate, mixed_int4 as X, nvfp4 as O

pytestmark = pytest.mark.gpu


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _bf16_t(a):
    return T(np.asarray(a, np.float32)).to(torch.bfloat16)


def _layout(rows_list):
    offs, tot = [], 0
    for r in rows_list:
        offs.append(tot)
        tot += (r + 127) // 128 * 128
    return offs, max(tot, 128)


def test_int4_dequant_bit_exact():
    from mosaicist_b200 import ops

    l, n, k, gsz = 2, 64, 512, 128
    rng = np.random.default_rng(0)
    q = rng.integers(-8, 8, (l, n, k)).astype(np.int8)
    sc = np.abs(rng.standard_normal((l, n, k // gsz)) * 0.02).astype(np.float32).astype(ml_dtypes.bfloat16)
    got = ops.dequant_int4(T(X.pack_int4(q)), _bf16_t(sc), gsz).float().cpu().numpy()
    want = X.dequant(q, sc, gsz).astype(np.float32)
    assert np.array_equal(got, want) and np.count_nonzero(want) > want.size // 2
    assert (q == -8).any() and (q == 7).any()


@pytest.mark.parametrize("rows_list,n,k", [([128], 256, 128), ([64, 512, 0, 300, 17], 256, 1024),
                                           ([250, 1000, 16], 512, 384),       # check_matrix.py ragged M
                                           # around the 256- and 512-row edges of the tall tiles
                                           ([256, 257, 511, 512, 513, 1025, 769], 256, 256)])
@pytest.mark.parametrize("fused", [True, False], ids=["fused", "two_launches"])
def test_mixed_int4_exact(rows_list, n, k, fused):
    from mosaicist_b200 import _lib, ops

    gsz = 128
    l = len(rows_list)
    offs, tot = _layout(rows_list)
    rng = np.random.default_rng([l, n, k])
    a = rng.integers(-2, 3, (tot, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    q = rng.integers(-2, 3, (l, n, k)).astype(np.int8)
    sc = (rng.integers(1, 5, (l, n, k // gsz)).astype(np.float32) / 4).astype(ml_dtypes.bfloat16)   # problems.py:58
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    out = torch.full((tot, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.mixed_grouped_gemm_int4(_bf16_t(a), T(X.pack_int4(q)), _bf16_t(sc), T(np.array(offs, np.int32)),
                                T(np.array(rows_list, np.int32)), T(alpha), gsz, out=out, fused=fused)
    assert _lib.status_word() == 0
    want = X.ragged_gemm_f64(a, X.dequant(q, sc, gsz), offs, rows_list, alpha)
    # every partial sum is a multiple of 1/8 below 2^20: exact in fp32, so the only rounding
    # is the final one to bf16
    assert np.abs(want).max() < 2 ** 20 and np.array_equal(want * 8, np.round(want * 8))
    want = O.bf16_round(want)
    got = out.float().cpu().numpy()
    mask = np.zeros((tot, 1), bool)
    for o, r in zip(offs, rows_list):
        mask[o:o + r] = True
    assert np.array_equal(np.where(mask, got, 0), want)
    assert np.isnan(got[~mask[:, 0]]).all() and np.count_nonzero(want) > mask.sum() * n // 2


def test_mixed_int4_random_within_tolerance():
    from mosaicist_b200 import _lib, ops

    rows_list, n, k, gsz = [300, 90, 512], 512, 1024, 128
    l = len(rows_list)
    offs, tot = _layout(rows_list)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((tot, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    q = rng.integers(-8, 8, (l, n, k)).astype(np.int8)
    sc = np.abs(rng.standard_normal((l, n, k // gsz)) * 0.02).astype(np.float32).astype(ml_dtypes.bfloat16)
    out = ops.mixed_grouped_gemm_int4(_bf16_t(a), T(X.pack_int4(q)), _bf16_t(sc), T(np.array(offs, np.int32)),
                                      T(np.array(rows_list, np.int32)))
    assert _lib.status_word() == 0
    ref = X.ragged_gemm_f64(a, X.dequant(q, sc, gsz), offs, rows_list)
    got = out.float().cpu().numpy()
    bd = _bf16_t(X.dequant(q, sc, gsz).astype(np.float32))
    at = _bf16_t(a)
    for g_, (o, r) in enumerate(zip(offs, rows_list)):
        ok, worst = O.tolerance_ok(got[o:o + r], ref[o:o + r])
        assert ok, worst
        # gate with a library bf16 GEMM (cuBLAS via torch) on the same operands as reference arm
        lib_out = torch.matmul(at[o:o + r], bd[g_].T).float().cpu().numpy()
        rep = gate.compare_outputs(lib_out, got[o:o + r], ref[o:o + r], "bf16")
        assert rep.passed, rep.failures


@pytest.mark.parametrize("gsz,k", [(128, 1024), (64, 448), (256, 1536)])
def test_fused_int4_kernel_equals_the_two_launch_path(gsz, k):
    """Random activations, the full int4 range and arbitrary scales: the in-kernel expansion
    (converter warps writing the swizzled bf16 tile) must give the bits of the separate
    expansion kernel followed by the bf16 grouped GEMM."""
    from mosaicist_b200 import _lib, ops

    rows_list, n = [300, 0, 129, 512, 7], 512
    l = len(rows_list)
    offs, tot = _layout(rows_list)
    g = torch.Generator(device="cuda").manual_seed(k)
    a = torch.randn((tot, k), device="cuda", generator=g).bfloat16()
    bq = torch.randint(0, 256, (l, n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sc = (torch.randn((l, n, k // gsz), device="cuda", generator=g) * 0.05).bfloat16()
    alpha = torch.rand((l,), device="cuda", generator=g) + 0.5
    o_t, r_t = T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32))
    one = torch.full((tot, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    two = torch.full((tot, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.mixed_grouped_gemm_int4(a, bq, sc, o_t, r_t, alpha, gsz, out=one, fused=True)
    ops.mixed_grouped_gemm_int4(a, bq, sc, o_t, r_t, alpha, gsz, out=two, fused=False)
    assert _lib.status_word() == 0
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))       # NaN rows compare as bits
    assert int(torch.isnan(one).sum()) == (tot - sum(rows_list)) * n
