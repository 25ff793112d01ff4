"""Parity of the CUDA block-scaled grouped GEMM with the CPU oracle, through the C ABI.

Mirrors the reference's kernel tests (experiments/flashinfer-megamoe-sm100a/
test_kernels.py:28-92, verify_b200.py:53-87): exact operands must agree bit for bit,
random operands within tolerance, masked rows are compared only below masked_m, and every
comparison proves it is non-trivial.  Tolerance for bf16 outputs against the float64
oracle: |err| <= 2^-7 |ref| + 1e-3 rms(ref); the reference's own quantile gate must pass
too."""

import numpy as np
import pytest
import torch

from oracle import gate, mxfp8 as X, nvfp4 as O

pytestmark = pytest.mark.gpu


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _nontrivial(want):
    w = np.asarray(want, np.float64)
    assert np.count_nonzero(w) >= 0.5 * w.size and (w.max() - w.min()) >= 1e-3   # verify_b200.py:55-61


def run_masked(a_q, a_sf, b_q, b_sf, alpha, masked_m, cfg):
    from mosaicist_b200 import _lib, ops

    l, m, _ = a_q.shape
    n = b_q.shape[1]
    out = torch.full((l, m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.masked_grouped_gemm(T(O.pack_e2m1(a_q)), T(O.e4m3_bytes(O.retile(a_sf))),
                            T(O.pack_e2m1(b_q)), T(O.e4m3_bytes(O.retile(b_sf))),
                            None if alpha is None else T(alpha),
                            None if masked_m is None else T(masked_m), cfg, out=out)
    assert _lib.status_word() == 0
    return out.float().cpu().numpy()


def _cfg(**kw):
    from mosaicist_b200 import ops

    return ops.GemmConfig(**kw)


EXACT_CASES = [
    # l, m, n, k, config                       (first two: test_kernels.py:78-83)
    (2, 256, 256, 512, {}),
    (3, 128, 256, 1024, {}),
    (1, 128, 128, 64, {}),                     # a single MMA
    (2, 256, 512, 576, {"stages": 2}),         # partial last K stage, shallow ring
    (2, 256, 256, 512, {"tile_n": 256}),
    (2, 256, 512, 4096, {"tile_n": 256, "stages": 3, "raster": 1}),   # verify_b200.py k=4096
    (5, 384, 384, 320, {"max_ctas": 7}),       # more tiles than CTAs: persistent loop
    (2, 128, 256, 2048, {"stages": 6, "raster": 1}),
    # two CTAs per 256x256 tile (cta_group::2), incl. an odd number of m-tiles per group
    (1, 256, 256, 64, {"cta_pair": 1}),
    (2, 512, 512, 576, {"cta_pair": 1}),
    (3, 384, 256, 1024, {"cta_pair": 1, "stages": 2}),
    (5, 512, 768, 1280, {"cta_pair": 1, "max_ctas": 6}),
    # scale factors written into TMEM by dedicated warps (tcgen05.st) instead of tcgen05.cp
    (2, 512, 512, 576, {"cta_pair": 1, "sf_warps": 1}),
]


@pytest.mark.parametrize("l,m,n,k,cfg", EXACT_CASES)
@pytest.mark.parametrize("seed", [0, 1])
def test_exact_operands_bit_exact(l, m, n, k, cfg, seed):
    rng = np.random.default_rng([seed, l, m, n, k])
    a_q, a_sf = O.exact_operands(rng, l, m, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    masked_m = np.array(([m, max(1, m // 2 - 3)] + [m] * l)[:l], np.int32)   # test_kernels.py:50
    got = run_masked(a_q, a_sf, b_q, b_sf, alpha, masked_m, _cfg(**cfg))
    want = O.bf16_round(O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, alpha, masked_m))
    rows = np.arange(m)[None, :, None] < masked_m[:, None, None]
    _nontrivial(want[0])
    assert np.array_equal(np.where(rows, got, 0), want)
    # rows at or beyond masked_m are never written
    assert np.isnan(got[~np.broadcast_to(rows, got.shape)]).all()


@pytest.mark.parametrize("cfg", [{}, {"cta_pair": 2}])
def test_headline_shape_ragged_rows_bit_exact(cfg):
    """The headline shape (l=8, m=512, n=2048, k=2048) with ragged row counts - a full group, an
    odd count, a single row, an empty group, one and three whole 128-row blocks, one row short of
    full - on exact operands: bit-exact below masked_m, nothing written at or beyond it."""
    l, m, n, k = 8, 512, 2048, 2048
    rng = np.random.default_rng([3, l, m, n, k])
    a_q, a_sf = O.exact_operands(rng, l, m, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    masked_m = np.array([512, 253, 1, 0, 128, 384, 511, 512], np.int32)
    got = run_masked(a_q, a_sf, b_q, b_sf, alpha, masked_m, _cfg(**cfg))
    want = O.bf16_round(O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, alpha, masked_m))
    rows = np.arange(m)[None, :, None] < masked_m[:, None, None]
    _nontrivial(want[0])
    assert np.array_equal(np.where(rows, got, 0), want)
    assert np.isnan(got[~np.broadcast_to(rows, got.shape)]).all()


def test_edge_groups_empty_and_single_row():
    l, m, n, k = 4, 256, 128, 256
    rng = np.random.default_rng(7)
    a_q, a_sf = O.exact_operands(rng, l, m, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    masked_m = np.array([0, 1, 256, 129], np.int32)
    got = run_masked(a_q, a_sf, b_q, b_sf, None, masked_m, _cfg())
    want = O.bf16_round(O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, None, masked_m))
    rows = np.arange(m)[None, :, None] < masked_m[:, None, None]
    assert np.array_equal(np.where(rows, got, 0), want)
    assert np.isnan(got[0]).all()


@pytest.mark.parametrize("cfg", [{}, {"tile_n": 256}, {"cta_pair": 1}])
def test_random_operands_within_tolerance_and_gate(cfg):
    """Seeded N(0,1) operands quantised by the oracle with gs = 64 (test_kernels.py:43-48)."""
    l, m, n, k = 2, 256, 256, 512
    a = np.random.default_rng([0, 0]).standard_normal((l, m, k)).astype(np.float32)
    b = np.random.default_rng([0, 1]).standard_normal((l, n, k)).astype(np.float32)
    gs = np.full((l,), 64.0, np.float32)
    a_q, a_sf = O.quantize_nvfp4(a, gs)
    b_q, b_sf = O.quantize_nvfp4(b, gs)
    alpha = np.random.default_rng([0, 2]).uniform(0.5, 2.0, l).astype(np.float32)
    got = run_masked(a_q, a_sf, b_q, b_sf, alpha, None, _cfg(**cfg))
    ref64 = O.grouped_gemm_f64(a_q, a_sf, b_q, b_sf, alpha)
    _nontrivial(ref64)
    ok, worst = O.tolerance_ok(got, ref64)
    assert ok, f"worst error / bound = {worst}"
    assert np.abs(got - ref64).max() / np.abs(ref64).max() < 5e-3          # test_kernels.py:87-89
    rep = gate.gate_bf16(got, ref64)
    assert rep.passed, rep.failures


def test_headline_shape_properties():
    """l=8, m=512, n=2048, k=2048 on device-quantised N(0,1) data: size-independent checks
    (linearity in alpha, agreement of the two tile shapes, a sampled float64 check)."""
    from mosaicist_b200 import _lib, ops
    from mosaicist_b200.formats import dequant_nvfp4

    l, m, n, k = 8, 512, 2048, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((l, m, k), device="cuda", generator=g)
    b = torch.randn((l, n, k), device="cuda", generator=g)
    gs = torch.full((l,), 64.0, device="cuda")
    a_q, a_sf = ops.quantize_nvfp4(a, gs)
    b_q, b_sf = ops.quantize_nvfp4(b, gs)
    one = torch.ones((l,), device="cuda")
    o1 = ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, one, None, ops.GemmConfig())
    o2 = ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, 2 * one, None, ops.GemmConfig(tile_n=256))
    o3 = ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, one, None, ops.GemmConfig(cta_pair=1))
    assert _lib.status_word() == 0
    assert torch.equal(o1.float() * 2, o2.float())        # power-of-two alpha is exact in bf16
    assert torch.equal(o1, o3)                            # every kernel variant, same bits
    gi = 5
    rows = slice(128, 160)
    ref = dequant_nvfp4(a_q[gi].cpu().numpy(), a_sf[gi].cpu().numpy())[rows] @ \
        dequant_nvfp4(b_q[gi].cpu().numpy(), b_sf[gi].cpu().numpy()).T
    ok, worst = O.tolerance_ok(o1[gi, rows].float().cpu().numpy(), ref)
    assert ok, worst
    assert np.array_equal(o1[gi, rows].float().cpu().numpy(), O.bf16_round(ref))


RAGGED = [
    ([128], 128, 128, {}),
    ([200, 0, 50, 384], 256, 1024, {}),
    ([200, 0, 50, 384], 256, 1024, {"tile_n": 256}),
    ([1, 127, 129, 300, 5], 384, 640, {"max_ctas": 3}),
    ([200, 0, 50, 384, 257], 256, 1024, {"cta_pair": 1}),
    ([1, 127, 129, 300, 5], 512, 640, {"cta_pair": 1, "max_ctas": 4}),
    # short tiles of the pair kernel: every count of 32-row A boxes in either CTA, next to full tiles
    ([32, 33, 64, 96, 97, 128, 160, 161, 224, 255, 256, 288, 289, 400, 512, 31], 256, 896, {"cta_pair": 1}),
    ([289, 161, 33, 544], 512, 384, {"cta_pair": 1, "max_ctas": 2, "stages": 3}),
    # tokens on the MMA's N side: one- and two-MMA tiles, several token tiles, tiny groups
    ([272, 1, 16, 17, 320, 321, 576, 640, 129, 255, 256, 0, 82], 512, 640, {"cta_pair": 3}),
    ([305, 240, 1000], 256, 896, {"cta_pair": 3, "max_ctas": 4}),
]


def _ragged_layout(rows_list):
    offs, tot = [], 0
    for r in rows_list:
        offs.append(tot)
        tot += (r + 127) // 128 * 128
    return offs, max(tot, 128)


@pytest.mark.parametrize("rows_list,n,k,cfg", RAGGED)
def test_mxfp8_ragged_bit_exact(rows_list, n, k, cfg):
    from mosaicist_b200 import _lib, ops

    rng = np.random.default_rng([2, n, k, len(rows_list)])
    l = len(rows_list)
    offs, tot = _ragged_layout(rows_list)
    a_q, a_sf = X.exact_operands(rng, tot, k)
    b = [X.exact_operands(rng, n, k) for _ in range(l)]
    b_q, b_sf = np.stack([x[0] for x in b]), np.stack([x[1] for x in b])
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    rs = np.exp2(rng.integers(-1, 2, tot)).astype(np.float32)
    out = torch.full((tot, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.ragged_grouped_gemm_mxfp8(
        T(a_q.view(np.uint8)), T(O.to_mma_scale_layout(a_sf)), T(b_q.view(np.uint8)),
        T(np.stack([O.to_mma_scale_layout(s) for s in b_sf])), T(np.array(offs, np.int32)),
        T(np.array(rows_list, np.int32)), T(alpha), T(rs), _cfg(**cfg), out=out)
    assert _lib.status_word() == 0
    got = out.float().cpu().numpy()
    want = O.bf16_round(X.ragged_grouped_gemm_f64(a_q, a_sf, b_q, b_sf, offs, rows_list, alpha, rs))
    mask = np.zeros((tot, 1), bool)
    for o, r in zip(offs, rows_list):
        mask[o:o + r] = True
    _nontrivial(want[mask[:, 0]])
    assert np.array_equal(np.where(mask, got, 0), want)
    assert np.isnan(got[~mask[:, 0]]).all()


RAGGED_NVFP4 = RAGGED[1:-2] + [
    # tokens on the MMA's N side (cta_pair=3): tiles of one MMA (<= 256 rows), of two (257 - 320), several
    # token tiles per group (the last one taking a remainder of up to 64), empty and one-row groups
    ([200, 0, 50, 384, 257], 256, 1024, {"cta_pair": 3}),
    ([272, 1, 16, 17, 320, 321, 576, 640, 129, 255, 256], 512, 640, {"cta_pair": 3}),
    ([305, 240, 1000], 256, 896, {"cta_pair": 3, "max_ctas": 4}),
]


@pytest.mark.parametrize("rows_list,n,k,cfg", RAGGED_NVFP4)
def test_nvfp4_ragged_row_scale_bit_exact(rows_list, n, k, cfg):
    from mosaicist_b200 import _lib, ops

    rng = np.random.default_rng([3, n, k])
    l = len(rows_list)
    offs, tot = _ragged_layout(rows_list)
    a_q, a_sf = O.exact_operands(rng, 1, tot, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    rs = np.exp2(rng.integers(-1, 2, tot)).astype(np.float32)
    out = torch.full((tot, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.ragged_grouped_gemm_nvfp4(
        T(O.pack_e2m1(a_q[0])), T(O.e4m3_bytes(O.to_mma_scale_layout(a_sf[0]))),
        T(O.pack_e2m1(b_q)), T(O.e4m3_bytes(O.retile(b_sf))), T(np.array(offs, np.int32)),
        T(np.array(rows_list, np.int32)), T(alpha), T(rs), _cfg(**cfg), out=out)
    assert _lib.status_word() == 0
    got = out.float().cpu().numpy()
    want = np.zeros((tot, n))
    for g_, (o, r) in enumerate(zip(offs, rows_list)):
        if r:
            y = O.grouped_gemm_f64(a_q[:, o:o + r], a_sf[:, o:o + r], b_q[g_:g_ + 1], b_sf[g_:g_ + 1])[0]
            want[o:o + r] = y * alpha[g_] * rs[o:o + r, None]
    mask = np.zeros((tot, 1), bool)
    for o, r in zip(offs, rows_list):
        mask[o:o + r] = True
    assert np.array_equal(np.where(mask, got, 0), O.bf16_round(want))


def test_random_mxfp8_within_tolerance():
    from mosaicist_b200 import _lib, ops

    rows_list, n, k = [300, 128, 77], 256, 896
    l = len(rows_list)
    offs, tot = _ragged_layout(rows_list)
    a = np.random.default_rng([4, 0]).standard_normal((tot, k)).astype(np.float32)
    b = np.random.default_rng([4, 1]).standard_normal((l, n, k)).astype(np.float32)
    a_q, a_sf = X.quantize_mxfp8(a)
    b_q, b_sf = X.quantize_mxfp8(b)
    out = ops.ragged_grouped_gemm_mxfp8(
        T(a_q.view(np.uint8)), T(O.to_mma_scale_layout(a_sf)), T(b_q.view(np.uint8)),
        T(np.stack([O.to_mma_scale_layout(s) for s in b_sf])), T(np.array(offs, np.int32)),
        T(np.array(rows_list, np.int32)))
    assert _lib.status_word() == 0
    ref = X.ragged_grouped_gemm_f64(a_q, a_sf, b_q, b_sf, offs, rows_list)
    got = out.float().cpu().numpy()
    for o, r in zip(offs, rows_list):
        ok, worst = O.tolerance_ok(got[o:o + r], ref[o:o + r])
        assert ok, worst
        assert gate.gate_bf16(got[o:o + r], ref[o:o + r]).passed


def test_torch_custom_op_matches_direct_call():
    import mosaicist_b200.torch_ops  # noqa: F401
    from mosaicist_b200 import ops

    l, m, n, k = 2, 256, 256, 512
    g = torch.Generator(device="cuda").manual_seed(1)
    u8 = lambda *s, lo=0, hi=256: torch.randint(lo, hi, s, dtype=torch.uint8, device="cuda", generator=g)
    a_q, b_q = u8(l, m, k // 2), u8(l, n, k // 2)
    a_sf, b_sf = u8(l, m // 128, k // 64, 32, 16, lo=0x30, hi=0x40), u8(l, n // 128, k // 64, 32, 16, lo=0x30, hi=0x40)
    masked = torch.tensor([m, 77], dtype=torch.int32, device="cuda")
    got = torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4(a_q, a_sf, b_q, b_sf, None, masked)
    want = ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, None, masked,
                                   out=torch.zeros((l, m, n), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(got, want) and int((got[1, 77:] != 0).sum()) == 0 and int((got[1, :77] != 0).sum()) > 0
    # the quantisers and the ragged GEMM as operators
    x = torch.randn((l, m, k), device="cuda", generator=g).bfloat16()
    gs = torch.full((l,), 448.0, device="cuda")
    q_op, sf_op = torch.ops.mosaicist_sm100a.quantize_nvfp4(x, gs, None)
    q_d, sf_d = ops.quantize_nvfp4(x, gs)
    assert torch.equal(q_op, q_d) and torch.equal(sf_op, sf_d)
    q_op, sf_op = torch.ops.mosaicist_sm100a.silu_mul_quantize_nvfp4(x, gs, None)
    q_d, sf_d = ops.silu_mul_quantize_nvfp4(x, gs)
    assert torch.equal(q_op, q_d) and torch.equal(sf_op, sf_d)
    offs = torch.tensor([0, 256], dtype=torch.int32, device="cuda")
    rows = torch.tensor([200, 256], dtype=torch.int32, device="cuda")
    y_op = torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4_ragged(a_q.view(l * m, -1), a_sf.view(l * m // 128, k // 64, 32, 16),
                                                                 b_q, b_sf, offs, rows, None, None)
    y_d = ops.ragged_grouped_gemm_nvfp4(a_q.view(l * m, -1), a_sf.view(l * m // 128, k // 64, 32, 16), b_q, b_sf, offs,
                                        rows, out=torch.zeros((l * m, n), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(y_op, y_d) and int((y_op[200:256] != 0).sum()) == 0
    # the MXFP8 chain, the dense GEMM and the bf16 x int4 grouped GEMM as operators
    P = torch.ops.mosaicist_sm100a
    assert torch.equal(P.global_scale_for(x), ops.global_scale_for(x))
    xa = torch.randn((l * m, k), device="cuda", generator=g).bfloat16()
    xb = torch.randn((l * n, k), device="cuda", generator=g).bfloat16()
    (qa, sa), (qb, sb) = P.quantize_mxfp8(xa), P.quantize_mxfp8(xb)
    qa_d, sa_d = ops.quantize_mxfp8(xa)
    assert torch.equal(qa, qa_d) and torch.equal(sa, sa_d)
    y_op = P.grouped_gemm_mxfp8_ragged(qa, sa, qb.view(l, n, k), sb.view(l, n // 128, k // 128, 32, 16), offs, rows, None, None)
    y_d = ops.ragged_grouped_gemm_mxfp8(qa, sa, qb.view(l, n, k), sb.view(l, n // 128, k // 128, 32, 16), offs, rows,
                                        out=torch.zeros((l * m, n), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(y_op, y_d) and int((y_op[200:256] != 0).sum()) == 0 and int((y_op[:200] != 0).sum()) > 0
    bt = xb[:n].t().contiguous()                                   # (k, n)
    assert torch.equal(P.gemm_f16(xa, bt), ops.gemm_f16(xa, bt))
    w_q = u8(l, n, k // 2)
    w_s = (torch.rand((l, n, k // 128), device="cuda", generator=g) * 0.02 + 0.01).bfloat16()
    y_op = P.grouped_gemm_bf16_int4_ragged(xa, w_q, w_s, offs, rows, None, 128)
    y_d = ops.mixed_grouped_gemm_int4(xa, w_q, w_s, offs, rows, None, 128,
                                      out=torch.zeros((l * m, n), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(y_op, y_d) and int((y_op[200:256] != 0).sum()) == 0 and int((y_op[:200] != 0).sum()) > 0


@pytest.mark.parametrize("rows_list,n,k", [([256], 256, 256), ([300, 0, 77, 512, 129], 512, 640),
                                           ([1, 320, 257, 0, 33], 256, 2048)])
def test_scatter_epilogue_equals_store_then_permute(rows_list, n, k):
    """msc_grouped_gemm_nvfp4_scatter_ragged: every valid row lands, bit for bit, where its code
    says - across two destination buffers, in a random order - rows coded negative are dropped,
    and nothing else is written."""
    import ctypes

    from mosaicist_b200 import _lib, ops

    rng = np.random.default_rng([9, n, k])
    l = len(rows_list)
    offs, tot = _ragged_layout(rows_list)
    a_q, a_sf = O.exact_operands(rng, 1, tot, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    alpha = np.exp2(rng.integers(-1, 2, l)).astype(np.float32)
    rs = np.exp2(rng.integers(-1, 2, tot)).astype(np.float32)
    args = (T(O.pack_e2m1(a_q[0])), T(O.e4m3_bytes(O.to_mma_scale_layout(a_sf[0]))), T(O.pack_e2m1(b_q)),
            T(O.e4m3_bytes(O.retile(b_sf))), T(np.array(offs, np.int32)), T(np.array(rows_list, np.int32)),
            T(alpha), T(rs))
    stored = torch.zeros((tot, n), dtype=torch.bfloat16, device="cuda")
    ops.ragged_grouped_gemm_nvfp4(*args, ops.GemmConfig(cta_pair=1), out=stored)

    valid = np.concatenate([np.arange(o, o + r) for o, r in zip(offs, rows_list)]).astype(np.int64)
    slots = rng.permutation(len(valid))                      # destination slot of every valid row
    which = rng.integers(0, 2, len(valid))                   # destination buffer of every valid row
    dropped = rng.random(len(valid)) < 0.1
    code = np.full(tot, -1, np.int32)
    code[valid] = np.where(dropped, -1, (which << 26) | slots).astype(np.int32)
    dest = [torch.full((len(valid), n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    bases = (ctypes.c_void_p * 2)(dest[0].data_ptr(), dest[1].data_ptr())
    a_qt, a_sft, b_qt, b_sft, o_t, r_t, al_t, rs_t = args
    _lib.check(_lib.load().msc_grouped_gemm_nvfp4_scatter_ragged(
        a_qt.data_ptr(), a_sft.data_ptr(), b_qt.data_ptr(), b_sft.data_ptr(), al_t.data_ptr(), o_t.data_ptr(),
        r_t.data_ptr(), rs_t.data_ptr(), T(code).data_ptr(), bases, 2, len(valid), l, tot, n, k,
        ops.GemmConfig().c(), torch.cuda.current_stream().cuda_stream))
    assert _lib.status_word() == 0
    want = [torch.full_like(d, float("nan")) for d in dest]
    for row, slot, w, drop in zip(valid, slots, which, dropped):
        if not drop:
            want[w][slot] = stored[row]
    for d, w in zip(dest, want):
        assert torch.equal(d.view(torch.int16), w.view(torch.int16))
    assert int((~torch.isnan(dest[0])).sum() + (~torch.isnan(dest[1])).sum()) == int((~dropped).sum()) * n

    # codes that name a destination or a row the call was not given are refused and reported:
    # only one destination and half of its rows are declared, everything else must stay NaN
    for d in dest:
        d.fill_(float("nan"))
    half = len(valid) // 2
    _lib.check(_lib.load().msc_grouped_gemm_nvfp4_scatter_ragged(
        a_qt.data_ptr(), a_sft.data_ptr(), b_qt.data_ptr(), b_sft.data_ptr(), al_t.data_ptr(), o_t.data_ptr(),
        r_t.data_ptr(), rs_t.data_ptr(), T(code).data_ptr(), bases, 1, max(half, 1), l, tot, n, k,
        ops.GemmConfig().c(), torch.cuda.current_stream().cuda_stream))
    refused = (~dropped) & ((which != 0) | (slots >= max(half, 1)))
    assert (_lib.status_word() == 0x00C00000) == bool(refused.any())
    assert bool(torch.isnan(dest[1]).all())
    want0 = torch.full_like(dest[0], float("nan"))
    for row, slot, w, drop in zip(valid, slots, which, dropped):
        if not drop and w == 0 and slot < max(half, 1):
            want0[slot] = stored[row]
    assert torch.equal(dest[0].view(torch.int16), want0.view(torch.int16))


@pytest.mark.parametrize("cta_pair", [1, 2, 3])
def test_group_table_beyond_the_buffers_is_cut_not_followed(cta_pair):
    """A group table that reaches past rows_total (what an overflowing expert-parallel step or a
    stale table hands the GEMM): the kernels are told rows_total = 384 while every buffer really
    holds 1024 rows, so the rows past 384 are a guard band inside the allocation.  The band must
    stay untouched, rows below 384 must equal the honest call, for the plain store and the fused
    SwiGLU epilogue alike."""
    from mosaicist_b200 import _lib, ops

    n, k, told, real = 256, 256, 384, 1024
    rng = np.random.default_rng([21, cta_pair])
    a_q, a_sf = O.exact_operands(rng, 1, real, k)
    b_q, b_sf = O.exact_operands(rng, 3, n, k)
    a_qt, a_sft = T(O.pack_e2m1(a_q[0])), T(O.e4m3_bytes(O.to_mma_scale_layout(a_sf[0])))
    b_qt, b_sft = T(O.pack_e2m1(b_q)), T(O.e4m3_bytes(O.retile(b_sf)))
    lib, st = _lib.load(), torch.cuda.current_stream().cuda_stream
    # group 0 fits, group 1 straddles the end, group 2 starts beyond it (and one negative offset)
    bad_off, bad_rows = T(np.array([0, 256, 640], np.int32)), T(np.array([200, 700, 300], np.int32))
    ok_off, ok_rows = T(np.array([0, 256, 0], np.int32)), T(np.array([200, 128, 0], np.int32))
    cfg = ops.GemmConfig(cta_pair=cta_pair).c()
    outs = []
    for off, rows in ((bad_off, bad_rows), (ok_off, ok_rows)):
        out = torch.full((real, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        _lib.check(lib.msc_grouped_gemm_nvfp4_ragged(a_qt.data_ptr(), a_sft.data_ptr(), b_qt.data_ptr(),
                                                     b_sft.data_ptr(), None, off.data_ptr(), rows.data_ptr(),
                                                     None, out.data_ptr(), 3, told, n, k, cfg, st))
        outs.append(out)
    assert _lib.status_word() == 0
    assert bool(torch.isnan(outs[0][told:]).all()), "rows past rows_total were written"
    assert torch.equal(outs[0][:told].view(torch.int16), outs[1][:told].view(torch.int16))
    assert int((~torch.isnan(outs[0][:told])).sum()) == (200 + 128) * n
    if cta_pair in (1, 3):
        if cta_pair == 3:      # the tokens-on-N form reads the interleaved copy of the weights
            b_qt, b_sft = ops.swiglu_interleave_w1(b_qt, b_sft)
        gs = T(np.full(3, 8.0, np.float32))
        al = T(np.ones(3, np.float32))
        res = []
        for off, rows in ((bad_off, bad_rows), (ok_off, ok_rows)):
            d_q = torch.full((real, n // 4), 0xEE, dtype=torch.uint8, device="cuda")
            d_sf = torch.full((real // 128, n // 128, 32, 16), 0xEE, dtype=torch.uint8, device="cuda")
            _lib.check(lib.msc_grouped_gemm_nvfp4_swiglu_ragged(
                a_qt.data_ptr(), a_sft.data_ptr(), b_qt.data_ptr(), b_sft.data_ptr(), al.data_ptr(), off.data_ptr(),
                rows.data_ptr(), gs.data_ptr(), d_q.data_ptr(), d_sf.data_ptr(), 3, told, n, k, cfg, st))
            res.append((d_q, d_sf))
        assert _lib.status_word() == 0
        assert bool((res[0][0][told:] == 0xEE).all()) and bool((res[0][1][told // 128:] == 0xEE).all())
        assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])


def test_shutdown_drops_cached_tensor_maps_and_the_next_call_rebuilds_them():
    from mosaicist_b200 import _lib, ops

    l, m, n, k = 1, 256, 256, 256
    rng = np.random.default_rng(12)
    a_q, a_sf = O.exact_operands(rng, l, m, k)
    b_q, b_sf = O.exact_operands(rng, l, n, k)
    args = (T(O.pack_e2m1(a_q)), T(O.e4m3_bytes(O.retile(a_sf))), T(O.pack_e2m1(b_q)), T(O.e4m3_bytes(O.retile(b_sf))))
    first = ops.masked_grouped_gemm(*args).clone()
    assert _lib.load().msc_shutdown() == 0
    again = ops.masked_grouped_gemm(*args)
    assert torch.equal(first, again) and _lib.status_word() == 0
