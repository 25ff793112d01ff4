"""Parity of the CUDA quantisation / scale re-tiling kernels with the CPU oracle (bit-exact:
these are byte-producing kernels)."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import nvfp4 as O

pytestmark = pytest.mark.gpu


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _data(l, m, k, seed, inf=False):
    x = np.random.default_rng([seed, 0]).standard_normal((l, m, k)).astype(np.float32)
    x[0, 0, :16] = 0.0              # an all-zero block: scale 0, values 0
    x[0, 1, 16:32] *= 1e-6          # a block whose scale underflows e4m3
    x[-1, 2, 5] = 40.0              # an outlier that dominates its block
    if inf:                         # infinite values saturate to +-6, their block's scale to 448
        x[0, 3, 40], x[0, 3, 41] = np.inf, -np.inf
    return x


@pytest.mark.parametrize("l,m,k", [(2, 128, 256), (3, 256, 64), (1, 384, 2048)])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_quantize_bit_exact(l, m, k, tiled, dtype):
    from mosaicist_b200 import ops

    x = _data(l, m, k, 11, inf=True)    # group 0 gets a fixed global scale below
    if dtype == "bf16":
        x = x.astype(ml_dtypes.bfloat16).astype(np.float32)
    gs = O.global_scale_for(x)
    gs[0] = 4096.0                  # forces the clip of the block scale at 448
    want_q, want_sf = O.quantize_nvfp4(x, gs)
    xt = T(x).to(torch.bfloat16) if dtype == "bf16" else T(x)
    q, sf = ops.quantize_nvfp4(xt, T(gs), None, tiled_scales=tiled)
    assert np.array_equal(q.cpu().numpy(), O.pack_e2m1(want_q))
    want_sf_b = O.e4m3_bytes(O.retile(want_sf)) if tiled else O.e4m3_bytes(want_sf)
    assert np.array_equal(sf.cpu().numpy(), want_sf_b)
    assert want_sf_b.max() == 0x7E and (want_sf_b == 0).any()      # the edge cases are really there


def test_quantize_skips_masked_rows():
    from mosaicist_b200 import ops

    l, m, k = 2, 128, 128
    x = _data(l, m, k, 5)
    gs = O.global_scale_for(x)
    masked = np.array([128, 7], np.int32)
    q, sf = ops.quantize_nvfp4(T(x), T(gs), T(masked), tiled_scales=False)
    want_q, want_sf = O.quantize_nvfp4(x, gs)
    qh, sfh = q.cpu().numpy(), sf.cpu().numpy()
    assert np.array_equal(qh[0], O.pack_e2m1(want_q)[0])
    assert (qh[0, 1, 8:16] & 0x88).any()          # negative zeros of the dead block survive
    assert np.array_equal(qh[1, :7], O.pack_e2m1(want_q)[1, :7])
    assert np.array_equal(sfh[1, :7], O.e4m3_bytes(want_sf)[1, :7]) and not sfh[1, 7:].any()


def test_silu_mul_quantize_matches_oracle():
    """The activation goes through expf on the device and np.exp on the host, so allow the
    rare block whose rounding flips; at least 99.9 % of bytes must be identical and every
    dequantised value within one e2m1 step."""
    from mosaicist_b200 import ops

    l, m, n = 2, 128, 256
    gu = np.random.default_rng([9, 0]).standard_normal((l, m, 2 * n)).astype(np.float32)
    gu = gu.astype(ml_dtypes.bfloat16)
    act = O.silu_mul(gu)
    gs = O.global_scale_for(act)
    want_q, want_sf = O.quantize_nvfp4(act, gs)
    q, sf = ops.silu_mul_quantize_nvfp4(T(np.asarray(gu, np.float32)).to(torch.bfloat16), T(gs), None,
                                        tiled_scales=False)
    qh, sfh = q.cpu().numpy(), sf.cpu().numpy()
    assert np.mean(qh == O.pack_e2m1(want_q)) > 0.999
    assert np.mean(sfh == O.e4m3_bytes(want_sf)) > 0.999
    back = O.dequantize_nvfp4(O.unpack_e2m1(qh), sfh.view(ml_dtypes.float8_e4m3fn), gs)
    step = want_sf.astype(np.float32) / gs.reshape(l, 1, 1)
    assert np.all(np.abs(back - act) <= np.repeat(step, 16, axis=-1) * 1.0001 + 1e-12)


@pytest.mark.parametrize("g,mn,ks", [(1, 256, 32), (3, 200, 8), (2, 128, 128), (1, 1, 4)])
def test_sf_swizzle_bit_exact(g, mn, ks):
    from mosaicist_b200 import ops

    sf = np.random.default_rng([g, mn, ks]).integers(0, 256, (g, mn, ks)).astype(np.uint8)
    got = ops.to_mma_scale_layout(T(sf)).cpu().numpy()
    want = np.stack([O.to_mma_scale_layout(s) for s in sf])
    assert got.shape == want.shape and np.array_equal(got, want)
    # the independent index formula of the reference's test (test_nvfp4.py:75-97)
    t, a, b, c, d = 0, min(3, (mn - 1) // 32), (mn - 1) % 32, ks // 4 - 1, 3
    row = 128 * t + 32 * a + b
    if row < mn:
        assert got[0, t, c, b, 4 * a + d] == sf[0, row, 4 * c + d]


def test_ragged_quantize_feeds_the_gemm():
    """quantize (ragged, tiled scales) -> ragged GEMM equals the oracle's quantize -> GEMM."""
    from mosaicist_b200 import _lib, ops

    rows_list, n, k = [130, 0, 64], 128, 256
    l = len(rows_list)
    offs = [0, 256, 256]
    tot = 384
    x = np.random.default_rng([12, 0]).standard_normal((tot, k)).astype(np.float32)
    gs = np.array([300.0, 1.0, 500.0], np.float32)
    q, sf = ops.quantize_nvfp4_ragged(T(x), T(gs), T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32)))
    rng = np.random.default_rng(13)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    out = ops.ragged_grouped_gemm_nvfp4(q, sf, T(O.pack_e2m1(b_q)), T(O.e4m3_bytes(O.retile(b_sf))),
                                        T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32)))
    assert _lib.status_word() == 0
    got = out.float().cpu().numpy()
    for g_, (o, r) in enumerate(zip(offs, rows_list)):
        if not r:
            continue
        a_q, a_sf = O.quantize_nvfp4(x[None, o:o + r], gs[g_:g_ + 1])
        assert np.array_equal(q.cpu().numpy()[o:o + r], O.pack_e2m1(a_q)[0])
        ref = O.grouped_gemm_f64(a_q, a_sf, b_q[g_:g_ + 1], b_sf[g_:g_ + 1])[0]
        assert np.array_equal(got[o:o + r], O.bf16_round(ref))


# --- MXFP8 quantiser and the global-scale reduction -----------------------------------------

def _mx_data(rows, k, seed):
    x = np.random.default_rng([seed, 1]).standard_normal((rows, k)).astype(np.float32)
    x[0, :32] = 0.0                                           # an all-zero block: scale byte 0
    x[1, 32:64] = 0.0
    x[1, 40] = 448.0 * 2.0 ** -3                              # blockmax = 448 * 2^e exactly: scale 2^e, q = 448
    x[2, 64:96] *= 0.0
    x[2, 70] = np.nextafter(np.float32(448.0 * 2.0 ** 5), np.float32(np.inf))   # one ulp above: scale 2^(e+1)
    x[3, 96:128] = 0.0
    x[3, 97], x[3, 98] = 1e-40, -3e-41                        # a sub-normal block: smallest scale, values survive
    x[4, 5] = -3.0e38                                         # the largest exponents
    x[5, :32] *= 1e-30
    return x


@pytest.mark.parametrize("rows,k", [(128, 128), (200, 384), (512, 7168)])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mxfp8_quantize_bit_exact(rows, k, tiled, dtype):
    from mosaicist_b200 import ops
    from oracle import mxfp8 as X

    x = _mx_data(rows, k, 3)
    if dtype == "bf16":
        x = x.astype(ml_dtypes.bfloat16).astype(np.float32)
    want_q, want_sf = X.quantize_mxfp8(x)
    xt = T(x).to(torch.bfloat16) if dtype == "bf16" else T(x)
    q, sf = ops.quantize_mxfp8(xt, tiled_scales=tiled)
    assert np.array_equal(q.cpu().numpy(), want_q.view(np.uint8))
    want_sf_b = O.to_mma_scale_layout(want_sf) if tiled else want_sf
    assert np.array_equal(sf.cpu().numpy(), want_sf_b)
    # the edge cases are really there
    assert want_sf[0, 0] == 0 and want_sf[1, 1] == 124 and want_q.view(np.uint8)[1, 40] == 0x7E
    if dtype == "f32":
        assert want_sf[2, 2] == 133 and want_sf[3, 3] == 0 and want_q.view(np.uint8)[3, 97] != 0
    # every dequantised value is within half a step of its block's grid
    back = X.dequantize_mxfp8(want_q, want_sf)
    step = np.repeat(np.ldexp(1.0, want_sf.astype(np.int32) - 127), 32, axis=-1) * 32.0   # widest e4m3 spacing: 2^5
    assert np.all(np.abs(back - x) <= 0.5 * step + 1e-45)


def test_mxfp8_quantize_ragged_skips_rows_outside_groups():
    from mosaicist_b200 import ops
    from oracle import mxfp8 as X

    rows_list, k = [100, 0, 130, 1], 256
    offs, tot = [0, 128, 128, 384], 512
    x = _mx_data(tot, k, 4)
    want_q, want_sf = X.quantize_mxfp8(x)
    q = torch.full((tot, k), 0xEE, dtype=torch.uint8, device="cuda")
    sf = torch.full((tot // 128, k // 128, 32, 16), 0xEE, dtype=torch.uint8, device="cuda")
    ops.quantize_mxfp8(T(x), True, T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32)), out=(q, sf))
    live = np.zeros(tot, bool)
    for o, r in zip(offs, rows_list):
        live[o:o + r] = True
    qh = q.cpu().numpy()
    assert np.array_equal(qh[live], want_q.view(np.uint8)[live]) and (qh[~live] == 0xEE).all()
    sf_rows = O.from_mma_scale_layout(sf.cpu().numpy(), tot)
    assert np.array_equal(sf_rows[live], want_sf[live]) and (sf_rows[~live] == 0xEE).all()


@pytest.mark.parametrize("shape", [(3, 128, 256), (8, 512, 2048), (1, 8, 8)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_global_scale_matches_oracle(shape, dtype):
    from mosaicist_b200 import ops

    x = np.random.default_rng([9, shape[1]]).standard_normal(shape).astype(np.float32)
    if shape[0] > 1:
        x[1] = 0.0                                            # amax == 0 counts as 1
    x[0, 0, 3] = -77.25
    if dtype == "bf16":
        x = x.astype(ml_dtypes.bfloat16).astype(np.float32)
    xt = T(x).to(torch.bfloat16) if dtype == "bf16" else T(x)
    got = ops.global_scale_for(xt).cpu().numpy()
    want = O.global_scale_for(x)
    assert np.array_equal(got, want) and got[0] == np.float32(2688.0) / np.abs(x[0]).max()
    if shape[0] > 1:
        assert got[1] == np.float32(2688.0)


def test_mxfp8_quantiser_feeds_the_gemm():
    """Quantiser kernel -> grouped MXFP8 GEMM == the oracle's quantiser -> float64 product."""
    from mosaicist_b200 import _lib, ops
    from oracle import mxfp8 as X

    rows_list, n, k = [300, 128, 77], 256, 896
    offs, tot = [0, 384, 512], 640
    a = np.random.default_rng([4, 0]).standard_normal((tot, k)).astype(np.float32)
    b = np.random.default_rng([4, 1]).standard_normal((3 * n, k)).astype(np.float32)
    o_t, r_t = T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32))
    a_q, a_sf = ops.quantize_mxfp8(T(a), True, o_t, r_t)
    b_q, b_sf = ops.quantize_mxfp8(T(b))
    out = ops.ragged_grouped_gemm_mxfp8(a_q, a_sf, b_q.view(3, n, k), b_sf.view(3, n // 128, k // 128, 32, 16), o_t, r_t)
    assert _lib.status_word() == 0
    want_aq, want_asf = X.quantize_mxfp8(a)
    want_bq, want_bsf = X.quantize_mxfp8(b)
    ref = X.ragged_grouped_gemm_f64(want_aq, want_asf, want_bq.reshape(3, n, k), want_bsf.reshape(3, n, -1), offs, rows_list)
    got = out.float().cpu().numpy()
    for o, r in zip(offs, rows_list):
        ok, worst = O.tolerance_ok(got[o:o + r], ref[o:o + r])
        assert ok, worst
