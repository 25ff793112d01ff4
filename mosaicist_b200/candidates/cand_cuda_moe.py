"""Capture module for the CUDA masked MoE path (drop-in for the reference's
experiments/loop/cand_pallas_moe.py): quantise -> GEMM1 -> SiLU*up + quantise -> GEMM2 at
l=8 experts, m=512 rows each, k=2048 hidden, n=1024 intermediate, the shape the reference
times end to end (experiments/flashinfer-megamoe-sm100a/README.md:45-51).

Weights ~ 0.05 N(0,1) quantised with their own global scales, alphas ~ U[0.5, 1.5], the
second global scale taken from one forward pass of the activation (the recipe of
make_moe_inputs, moe.py:82-115).  Time this module with `--measure all`: the path is four
kernels, not one (src/mosaicist/capture.py:127-140).
"""

from __future__ import annotations

import numpy as np

from ._common import drop_artifacts, from_env

L, M, K, N = 8, 512, 2048, 1024
SEED = 0

KNOBS = {
    "tile_n": [0, 128, 256],
    "stages": [0, 2, 3, 4],
    "cta_pair": [0, 1, 2],
}
STRUCTURAL = ("tile_n", "cta_pair")
DEFAULTS = {"tile_n": 0, "stages": 0, "cta_pair": 0}


def _inputs():
    """Device tensors in the order moe_masked takes them."""
    import torch

    from .. import ops

    dev = torch.device("cuda", torch.cuda.current_device())
    rng = [np.random.default_rng([SEED, i]) for i in range(4)]
    hidden = torch.from_numpy(rng[0].standard_normal((L, M, K)).astype(np.float32)).to(dev).to(torch.bfloat16)
    w1 = torch.from_numpy((rng[1].standard_normal((L, 2 * N, K)) * 0.05).astype(np.float32)).to(dev)
    w2 = torch.from_numpy((rng[2].standard_normal((L, K, N)) * 0.05).astype(np.float32)).to(dev)
    alphas = torch.from_numpy(rng[3].uniform(0.5, 1.5, (2, L)).astype(np.float32)).to(dev)

    def gs_for(x):                                   # global_scale_for, nvfp4.py:29-36
        return ops.global_scale_for(x.contiguous())

    w1_gs, w2_gs, in_gs = gs_for(w1), gs_for(w2), gs_for(hidden)
    w1_q, w1_sf = ops.quantize_nvfp4(w1, w1_gs)
    w2_q, w2_sf = ops.quantize_nvfp4(w2, w2_gs)
    masked_m = torch.full((L,), M, dtype=torch.int32, device=dev)
    # a2 global scale from one pass of the activation (moe.py:101-106)
    a_q, a_sf = ops.quantize_nvfp4(hidden, in_gs)
    gateup = ops.masked_grouped_gemm(a_q, a_sf, w1_q, w1_sf,
                                     (alphas[0] / (in_gs * w1_gs)).contiguous(), masked_m)
    g, u = gateup.float().chunk(2, dim=-1)
    a2_gs = gs_for((torch.sigmoid(g) * g * u).contiguous())
    return (hidden, w1_q, w1_sf, w1_gs, alphas[0].contiguous(), w2_q, w2_sf, w2_gs,
            alphas[1].contiguous(), masked_m, in_gs, a2_gs)


def reference():
    """float64 opinion on the same inputs, computed on the host from the raw inputs alone: no
    kernel of this library takes part.  The layer's own definition is followed where it rounds
    (experiments/flashinfer-megamoe-sm100a/nvfp4.py:91-108): the tokens are quantised to NVFP4
    (nvfp4.py:39-57), GEMM1's result is a bf16 tensor, SiLU(gate) * up is fp32 (nvfp4.py:81-88)
    and is quantised again; the two contractions are carried out in float64."""
    from ..formats import bf16_round, dequant_nvfp4, quantize_nvfp4_values

    (hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, masked_m, in_gs,
     a2_gs) = (t.float().cpu().numpy() if t.is_floating_point() else t.cpu().numpy() for t in _inputs())
    a_q, a_sf = quantize_nvfp4_values(hidden, in_gs)
    a = a_q * np.repeat(a_sf, 16, axis=-1)
    alpha1 = w1_alpha.astype(np.float64) / (in_gs.astype(np.float64) * w1_gs)
    alpha2 = w2_alpha.astype(np.float64) / (a2_gs.astype(np.float64) * w2_gs)
    out = np.empty((L, M, K), np.float64)
    for g in range(L):
        gateup = bf16_round((a[g] @ dequant_nvfp4(w1_q[g], w1_sf[g]).T) * alpha1[g])
        gate, up = gateup[:, :N], gateup[:, N:]
        act = (np.float32(1.0) / (np.float32(1.0) + np.exp(-gate))) * gate * up          # fp32
        d_q, d_sf = quantize_nvfp4_values(act[None], a2_gs[g:g + 1])
        d = d_q[0] * np.repeat(d_sf[0], 16, axis=-1)
        out[g] = (d @ dequant_nvfp4(w2_q[g], w2_sf[g]).T) * alpha2[g]
    return out


def build():
    from .. import ops
    from ..moe import fold_alphas, moe_masked

    k = from_env(DEFAULTS)
    cfg = ops.GemmConfig(tile_n=int(k["tile_n"]), stages=int(k["stages"]), cta_pair=int(k["cta_pair"]))
    args = _inputs()
    (_, _, _, w1_gs, w1_alpha, _, _, w2_gs, w2_alpha, _, in_gs, a2_gs) = args
    folded = fold_alphas(w1_gs, w1_alpha, w2_gs, w2_alpha, in_gs, a2_gs)   # constants of the weights
    single = int(k["cta_pair"]) == 2 or int(k["tile_n"]) != 0
    # mangled template arguments: <kind, stages, ...> of the pair kernel, <kind, tile_n, stages> of the other
    pair_stages = min(max(int(k["stages"]) or 5, 2), 5)
    tile = int(k["tile_n"]) or 128
    single_stages = min(int(k["stages"]) or 9, 5 if tile == 128 else 3)
    drop_artifacts("single" if single else "pair",
                   f"gemm_blockscaled_kernelILi0ELi{tile}ELi{single_stages}E" if single
                   else f"gemm_pair_kernelILi0ELi{pair_stages}ELb0ELb0ELb0E")

    def fn():
        return moe_masked(*args, gemm1_config=cfg, gemm2_config=cfg, folded_alphas=folded)

    return fn, ()
