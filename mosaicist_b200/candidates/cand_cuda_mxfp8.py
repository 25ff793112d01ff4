"""Capture module for the MXFP8 grouped GEMM (benchmark configuration 3): 32 groups whose row
counts follow Zipf(1.2) and sum to 16384, n = 4096, k = 7168; e4m3 values with one ue8m0 scale
per 32 K-elements, scale = 2^ceil(log2(blockmax / 448)), bf16 output.  The reference has no
MXFP8 code (its nearest relative is the fp8 block-scaled layer of
experiments/flashinfer-megamoe-sm90a/quant.py:47-75), so the definition is the benchmark's;
`reference()` is the float64 product of the dequantised operands, computed on the GPU.
$MOSAICIST_SHRINK divides the rows, n and k (a power of two up to 8) for quick captures.
"""

from __future__ import annotations

import os

from ._common import drop_artifacts, from_env

SHRINK = int(os.environ.get("MOSAICIST_SHRINK", "1"))
GROUPS, TOTAL, N, K = 32, 16384 // SHRINK, 4096 // SHRINK, 7168 // SHRINK
SEED = 0
KNOBS = {"stages": [0, 3, 4, 5], "cta_pair": [0, 1, 2], "tile_n": [0, 128, 256]}
STRUCTURAL = ("cta_pair", "tile_n")
DEFAULTS = {"stages": 0, "cta_pair": 0, "tile_n": 0}


def rows_per_group():
    w = [1.0 / r ** 1.2 for r in range(1, GROUPS + 1)]
    rows = [max(1, int(x / sum(w) * TOTAL)) for x in w]
    rows[0] += TOTAL - sum(rows)
    return rows


def _layout(rows):
    offs, at = [], 0
    for r in rows:
        offs.append(at)
        at += (r + 127) // 128 * 128
    return offs, at


def _quantize(x):
    """(rows, k) f32 -> e4m3 bytes (rows, k) and ue8m0 bytes (rows, k/32) row-major, by the
    library's MXFP8 quantiser."""
    from .. import ops

    return ops.quantize_mxfp8(x.contiguous(), tiled_scales=False)


def _inputs():
    """(a_q, a_sf tiled, b_q, b_sf tiled, group_offsets, group_rows, row-major scales)."""
    import torch

    from .. import ops

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(SEED)
    rows = rows_per_group()
    offs, tot = _layout(rows)
    a = torch.zeros((tot, K), device=dev)
    for o, r in zip(offs, rows):
        a[o:o + r] = torch.randn((r, K), device=dev, generator=g)
    a_q, a_s = _quantize(a)
    b_q, b_s = _quantize(torch.randn((GROUPS * N, K), device=dev, generator=g))
    a_sf = ops.to_mma_scale_layout(a_s.view(1, tot, K // 32))[0]
    b_sf = ops.to_mma_scale_layout(b_s.view(GROUPS, N, K // 32))
    return (a_q, a_sf, b_q.view(GROUPS, N, K), b_sf, torch.tensor(offs, dtype=torch.int32, device=dev),
            torch.tensor(rows, dtype=torch.int32, device=dev), a_s, b_s.view(GROUPS, N, K // 32))


def _dequant(q, s):
    import torch

    rows, k = q.shape
    val = q.view(torch.float8_e4m3fn).double().view(rows, k // 32, 32)
    return (val * torch.exp2(s.double() - 127.0)[:, :, None]).view(rows, k)


def reference():
    """(padded rows, n) float64; rows outside every group are zero."""
    import torch

    a_q, _, b_q, _, offs, rows, a_s, b_s = _inputs()
    out = torch.zeros((a_q.shape[0], N), dtype=torch.float64, device=a_q.device)
    for g, (o, r) in enumerate(zip(offs.tolist(), rows.tolist())):
        out[o:o + r] = _dequant(a_q[o:o + r], a_s[o:o + r]) @ _dequant(b_q[g], b_s[g]).T
    return out.cpu().numpy()


def build():
    import torch

    from .. import ops

    k = from_env(DEFAULTS)
    cfg = ops.GemmConfig(tile_n=int(k["tile_n"]), stages=int(k["stages"]), cta_pair=int(k["cta_pair"]))
    a_q, a_sf, b_q, b_sf, offs, rows, _, _ = _inputs()
    out = torch.zeros((a_q.shape[0], N), dtype=torch.bfloat16, device=a_q.device)
    single = int(k["cta_pair"]) == 2 or int(k["tile_n"]) != 0
    # mangled template arguments: <kind, stages, ...> of the pair kernel, <kind, tile_n, stages> of the other
    pair_stages = min(max(int(k["stages"]) or 5, 2), 5)
    tile = int(k["tile_n"]) or 128
    single_stages = min(int(k["stages"]) or 9, 5 if tile == 128 else 3)
    drop_artifacts("single" if single else "pair",
                   f"gemm_blockscaled_kernelILi1ELi{tile}ELi{single_stages}E" if single
                   else f"gemm_pair_kernelILi1ELi{pair_stages}ELb0ELb0ELb0E")

    def fn():
        return ops.ragged_grouped_gemm_mxfp8(a_q, a_sf, b_q, b_sf, offs, rows, None, None, cfg, out=out)

    return fn, ()
