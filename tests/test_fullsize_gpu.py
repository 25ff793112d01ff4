"""The benchmark configurations at their OWN sizes against the float64 CPU oracle, on a sample.

A full float64 product of these problems is out of reach of the host (1.1 PFLOP for the dense
one), a sample is not: a few hundred output rows, all columns, chosen with a seeded generator
and always including the last rows of ragged groups, cost seconds.  Every case runs the same
operator call the benchmark times, at the size the benchmark times it, and proves it is
non-trivial (experiments/flashinfer-megamoe-sm100a/verify_b200.py:55-61).

Tolerances: bf16 outputs |err| <= 2^-7 |ref| + 1e-3 rms(ref); fp16 outputs 2^-10 in place of
2^-7; the routed layer within the reference's MoE bounds (test_kernels.py:94-102)."""

import importlib

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import mixed_int4 as X4, moe as M, mxfp8 as X8, nvfp4 as O

pytestmark = pytest.mark.gpu


def _nontrivial(ref):
    ref = np.asarray(ref, np.float64)
    assert np.count_nonzero(ref) >= 0.5 * ref.size and ref.max() - ref.min() >= 1e-3


def _within(got, ref, rel):
    ref = np.asarray(ref, np.float64)
    err = np.abs(np.asarray(got, np.float64) - ref)
    bound = rel * np.abs(ref) + 1e-3 * np.sqrt(np.mean(ref ** 2))
    assert np.all(err <= bound), float((err / bound).max())


def _full_size(name, monkeypatch):
    for var in ("MOSAICIST_SHRINK", "MOSAICIST_DENSE_DIM", "MOSAICIST_KNOBS", "MOSAIC_GPU_DUMP_TO"):
        monkeypatch.delenv(var, raising=False)
    return importlib.reload(importlib.import_module(f"mosaicist_b200.candidates.{name}"))


def test_dense_fp16_8192_cubed_sampled_rows(monkeypatch):
    """C = A B at 8192^3 (experiments/hopper_gemm/ref_cutedsl.py:70: the oracle is
    a.double() @ b.double()): 256 random rows, every column."""
    from mosaicist_b200 import _lib

    m = _full_size("cand_cuda_dense", monkeypatch)
    assert m.DIM == 8192
    fn, args = m.build()
    out = fn(*args)
    torch.cuda.synchronize()
    assert _lib.status_word() == 0
    a, b = m._inputs()
    rows = np.sort(np.random.default_rng(2).choice(8192, 256, replace=False))
    rows[0], rows[-1] = 0, 8191
    ref = a[torch.from_numpy(rows).cuda()].cpu().numpy().astype(np.float64) @ b.cpu().numpy().astype(np.float64)
    got = out[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    _nontrivial(ref)
    _within(got, ref, 2.0 ** -10)


def test_mxfp8_zipf_groups_sampled_rows(monkeypatch):
    """32 groups, Zipf(1.2) row counts summing to 16384, n = 4096, k = 7168: rows of the largest
    group, of the smallest one and of groups whose row count straddles a 128-row tile."""
    from mosaicist_b200 import _lib

    m = _full_size("cand_cuda_mxfp8", monkeypatch)
    assert (m.TOTAL, m.N, m.K) == (16384, 4096, 7168)
    fn, args = m.build()
    out = fn(*args)
    torch.cuda.synchronize()
    assert _lib.status_word() == 0
    a_q, _, b_q, _, offs, rows, a_s, b_s = m._inputs()
    offs, rows = offs.tolist(), rows.tolist()
    assert sum(rows) == 16384 and min(rows) >= 1
    straddlers = [g for g, r in enumerate(rows) if r > 128 and r % 128]
    picked = {0, len(rows) - 1, straddlers[0], straddlers[-1]}
    rng = np.random.default_rng(3)
    for g in sorted(picked):
        r = rows[g]
        sel = np.unique(np.concatenate([rng.choice(r, min(r, 40), replace=False), [0, r - 1]]))
        idx = torch.from_numpy(offs[g] + sel).cuda()
        a = X8.dequantize_mxfp8(a_q[idx].cpu().numpy().view(ml_dtypes.float8_e4m3fn), a_s[idx].cpu().numpy())
        b = X8.dequantize_mxfp8(b_q[g].cpu().numpy().view(ml_dtypes.float8_e4m3fn), b_s[g].cpu().numpy())
        ref = a @ b.T
        _nontrivial(ref)
        _within(out[idx].float().cpu().numpy(), ref, 2.0 ** -7)
    # rows between the groups were never written (the output started as zeros)
    gap = [o + r for o, r in zip(offs, rows) if r % 128]
    assert all(int((out[g_] != 0).sum()) == 0 for g_ in gap[:4])


def test_bf16_int4_64_groups_sampled_rows(monkeypatch):
    """64 groups with m ~ U{64..512}, n = 2048, k = 7168, group size 128: rows of four groups
    against dequant + float64 product (ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-87)."""
    from mosaicist_b200 import _lib

    m = _full_size("cand_cuda_int4", monkeypatch)
    assert (m.GROUPS, m.N, m.K) == (64, 2048, 7168)
    fn, args = m.build()
    out = fn(*args)
    torch.cuda.synchronize()
    assert _lib.status_word() == 0
    a, b_q, scales, offs, rows = m._inputs()
    offs, rows = offs.tolist(), rows.tolist()
    rng = np.random.default_rng(4)
    for g in (0, int(np.argmin(rows)), int(np.argmax(rows)), 63):
        r = rows[g]
        sel = np.unique(np.concatenate([rng.choice(r, 30, replace=False), [0, r - 1]]))
        idx = torch.from_numpy(offs[g] + sel).cuda()
        packed = b_q[g].cpu().numpy()
        q = np.stack([packed & 0xF, packed >> 4], axis=-1).reshape(m.N, m.K).astype(np.int8)
        q = np.where(q >= 8, q - 16, q)
        w = X4.dequant(q, scales[g].float().cpu().numpy().astype(ml_dtypes.bfloat16), m.GROUP_SIZE)
        ref = a[idx].float().cpu().numpy().astype(np.float64) @ np.asarray(w, np.float64).T
        _nontrivial(ref)
        _within(out[idx].float().cpu().numpy(), ref, 2.0 ** -7)


def test_megamoe_deepseek_shape_sampled_tokens():
    """8192 tokens, hidden 7168, 256 experts, top-8, intermediate 2048 on one GPU; six tokens
    go through the oracle's routed layer with the weights of the experts they were routed to."""
    from mosaicist_b200 import _lib
    from mosaicist_b200.bench_moe import rand_weights
    from mosaicist_b200.moe import MegaMoE

    T_, h, E, k, n = 8192, 7168, 256, 8, 2048
    dev = torch.device("cuda", 0)
    w = rand_weights(E, n, h, dev, 17)
    w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha = w
    gs_in = torch.full((E,), 2688.0 / 5.0, dtype=torch.float32, device=dev)
    gs_a2 = torch.full((E,), 2688.0 / 8.0, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(99)
    tokens = torch.randn((T_, h), device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn((T_, E), device=dev, generator=g)
    layer = MegaMoE(*w, gs_in, gs_a2, topk=k, max_tokens=T_)
    out = layer.forward(tokens, logits)
    torch.cuda.synchronize()
    assert _lib.status_word() == 0

    sample = np.array([0, 1, 4095, 5000, 8190, 8191])
    lg = logits[torch.from_numpy(sample).cuda()].cpu().numpy()
    ids, wts = M.route_topk(lg, k)
    assert np.array_equal(ids, layer.ids[torch.from_numpy(sample).cuda()].cpu().numpy())
    used = np.unique(ids)
    local = np.searchsorted(used, ids).astype(np.int32)           # expert ids renumbered 0..len(used)-1
    sel = torch.from_numpy(used).cuda()

    def values(q, sf, rows):
        qv = O.unpack_e2m1(q[sel].cpu().numpy())
        sfv = np.stack([O.from_mma_scale_layout(s, rows) for s in sf[sel].cpu().numpy()]).view(ml_dtypes.float8_e4m3fn)
        return qv, sfv

    w1v, w1s = values(w1_q, w1_sf, 2 * n)
    w2v, w2s = values(w2_q, w2_sf, h)
    pick = lambda t: t[sel].cpu().numpy()
    tok = tokens[torch.from_numpy(sample).cuda()].float().cpu().numpy().astype(ml_dtypes.bfloat16)
    want = M.routed_moe(tok, local, wts, w1v, w1s, pick(w1_gs), pick(w1_alpha), w2v, w2s, pick(w2_gs),
                        pick(w2_alpha), pick(gs_in), pick(gs_a2), 0)
    got = out[torch.from_numpy(sample).cuda()].float().cpu().numpy()
    scale = max(np.abs(want).max(), 1e-6)
    rel = np.abs(got - want).max() / scale
    rms = np.sqrt(np.mean((got - want) ** 2)) / scale
    assert rel < 1e-1 and rms < 1e-2, (rel, rms)                  # test_kernels.py:94-102
    assert np.count_nonzero(want) > 0.9 * want.size
