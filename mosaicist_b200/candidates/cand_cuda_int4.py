"""Capture module for the bf16 x int4 grouped GEMM (benchmark configuration 4): 64 groups with
m ~ U{64..512}, n = 2048, k = 7168, int4 weights uniform in [-8, 7] packed two per byte (low
nibble first), bf16 scales |N(0, 0.02)| per 128 K-elements, fp32 accumulation, bf16 output.
Semantics of ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-87: the weight is
bf16(q) * scale formed in bf16, the product accumulates in fp32; `reference()` is the float64
product with those bf16 weights, computed on the GPU.  $MOSAICIST_SHRINK divides the group
count, n and k (a power of two up to 8) for quick captures.
"""

from __future__ import annotations

import os

from ._common import drop_artifacts, from_env

SHRINK = int(os.environ.get("MOSAICIST_SHRINK", "1"))
GROUPS, N, K, GROUP_SIZE = 64 // SHRINK, 2048 // SHRINK, 7168 // SHRINK, 128
SEED = 0
KNOBS = {"fused": [1, 0], "max_ctas": [0, 128, 74]}
STRUCTURAL = ("fused",)
DEFAULTS = {"fused": 1, "max_ctas": 0}


def _inputs():
    import numpy as np
    import torch

    dev = torch.device("cuda", torch.cuda.current_device())
    rows = np.random.default_rng([SEED, 0]).integers(64, 513, GROUPS).tolist()
    offs, at = [], 0
    for r in rows:
        offs.append(at)
        at += (r + 127) // 128 * 128
    g = torch.Generator(device=dev).manual_seed(SEED)
    a = torch.randn((at, K), device=dev, generator=g).bfloat16()
    b_q = torch.randint(0, 256, (GROUPS, N, K // 2), dtype=torch.uint8, device=dev, generator=g)
    scales = (torch.randn((GROUPS, N, K // GROUP_SIZE), device=dev, generator=g) * 0.02).abs().bfloat16()
    return (a, b_q, scales, torch.tensor(offs, dtype=torch.int32, device=dev),
            torch.tensor(rows, dtype=torch.int32, device=dev))


def reference():
    """(padded rows, n) float64; rows outside every group are zero."""
    import torch

    from .. import ops

    a, b_q, scales, offs, rows = _inputs()
    out = torch.zeros((a.shape[0], N), dtype=torch.float64, device=a.device)
    lo = (b_q & 0xF).to(torch.int8)
    hi = (b_q >> 4).to(torch.int8)
    q = torch.stack([lo, hi], dim=-1).view(GROUPS, N, K)
    q = torch.where(q >= 8, q - 16, q)
    w = (q.bfloat16() * scales.repeat_interleave(GROUP_SIZE, dim=2)).double()   # the product rounds to bf16
    for g, (o, r) in enumerate(zip(offs.tolist(), rows.tolist())):
        out[o:o + r] = a[o:o + r].double() @ w[g].T
    return out.cpu().numpy()


def build():
    import torch

    from .. import ops

    k = from_env(DEFAULTS)
    a, b_q, scales, offs, rows = _inputs()
    out = torch.zeros((a.shape[0], N), dtype=torch.bfloat16, device=a.device)
    drop_artifacts("dense", "gemm_dense_f16_kernelILi5ELb1ELb1E" if int(k["fused"]) else "gemm_dense_f16_kernelILi6ELb1ELb0E")

    def fn():
        return ops.mixed_grouped_gemm_int4(a, b_q, scales, offs, rows, None, GROUP_SIZE, out=out,
                                           fused=bool(int(k["fused"])), max_ctas=int(k["max_ctas"]))

    return fn, ()
