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


def _data(l, m, k, seed):
    x = np.random.default_rng([seed, 0]).standard_normal((l, m, k)).astype(np.float32)
    x[0, 0, :16] = 0.0              # an all-zero block: scale 0, values 0
    x[0, 1, 16:32] *= 1e-6          # a block whose scale underflows e4m3
    x[-1, 2, 5] = 40.0              # an outlier that dominates its block
    return x


@pytest.mark.parametrize("l,m,k", [(2, 128, 256), (3, 256, 64), (1, 384, 2048)])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_quantize_bit_exact(l, m, k, tiled, dtype):
    from mosaicist_b200 import ops

    x = _data(l, m, k, 11)
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
