"""Capture module for the CUDA NVFP4 masked grouped GEMM (drop-in for the reference's
experiments/loop/cand_pallas_gemm.py: same problem, same interface, same oracle formula).

Problem: l=8 groups, m=512, n=2048, k=2048; A ~ N(0,1), B ~ 0.05 N(0,1), both quantised
with a fixed global scale of 64 (cand_pallas_gemm.py:41-51); alpha = 1, every row valid.
Inputs come from numpy's `default_rng([seed, arg_index])` (the convention of
src/mosaicist/verify/suites.py:53), so every capture sees identical data.
"""

from __future__ import annotations

import numpy as np

from ._common import drop_artifacts, from_env

L, M, K, N = 8, 512, 2048, 2048
SEED = 0

#: the space the tuner walks, first value = default (knobs.py:57-58)
KNOBS = {
    "tile_n": [0, 128, 256],
    "stages": [0, 2, 3, 4, 5, 6],
    "raster": [0, 1],
    "max_ctas": [0, 128, 74],
    "cta_pair": [0, 1, 2],
}
#: knobs that swap the tile shape rather than retune it
STRUCTURAL = ("tile_n", "cta_pair")
DEFAULTS = {"tile_n": 0, "stages": 0, "raster": 0, "max_ctas": 0, "cta_pair": 0}


def _host_inputs():
    a = np.random.default_rng([SEED, 0]).standard_normal((L, M, K)).astype(np.float32)
    b = (np.random.default_rng([SEED, 1]).standard_normal((L, N, K)) * 0.05).astype(np.float32)
    return a, b


def _inputs():
    """Quantised operands on the device: (a_q, a_sf, b_q, b_sf), scales in the MMA tiling."""
    import torch

    from .. import ops

    a, b = _host_inputs()
    dev = torch.device("cuda", torch.cuda.current_device())
    gs = torch.full((L,), 64.0, dtype=torch.float32, device=dev)
    a_q, a_sf = ops.quantize_nvfp4(torch.from_numpy(a).to(dev), gs)
    b_q, b_sf = ops.quantize_nvfp4(torch.from_numpy(b).to(dev), gs)
    return a_q, a_sf, b_q, b_sf


def reference():
    """float64 oracle: q * repeat(sf, 16) for both operands, contracted in double precision
    (cand_pallas_gemm.py:54-63)."""
    from ..formats import dequant_nvfp4

    a_q, a_sf, b_q, b_sf = (t.cpu().numpy() for t in _inputs())
    out = np.empty((L, M, N), np.float64)
    for g in range(L):
        out[g] = dequant_nvfp4(a_q[g], a_sf[g]) @ dequant_nvfp4(b_q[g], b_sf[g]).T
    return out


def build():
    import torch

    from .. import ops

    k = from_env(DEFAULTS)
    cfg = ops.GemmConfig(tile_n=int(k["tile_n"]), stages=int(k["stages"]), raster=int(k["raster"]),
                         max_ctas=int(k["max_ctas"]), cta_pair=int(k["cta_pair"]))
    a_q, a_sf, b_q, b_sf = _inputs()
    alpha = torch.ones((L,), dtype=torch.float32, device=a_q.device)
    masked_m = torch.full((L,), M, dtype=torch.int32, device=a_q.device)
    out = torch.empty((L, M, N), dtype=torch.bfloat16, device=a_q.device)
    single = int(k["cta_pair"]) == 2 or int(k["tile_n"]) != 0
    # mangled template arguments: <kind, stages, ...> of the pair kernel, <kind, tile_n, stages> of the other
    pair_stages = min(max(int(k["stages"]) or 5, 2), 5)
    tile = int(k["tile_n"]) or 128
    single_stages = min(int(k["stages"]) or 9, 5 if tile == 128 else 3)
    drop_artifacts("single" if single else "pair",
                   f"gemm_blockscaled_kernelILi0ELi{tile}ELi{single_stages}E" if single
                   else f"gemm_pair_kernelILi0ELi{pair_stages}ELb0ELb0ELb0E")

    def fn():
        return ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, alpha, masked_m, cfg, out=out)

    return fn, ()
