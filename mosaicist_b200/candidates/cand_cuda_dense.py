"""Capture module for the dense fp16 GEMM (benchmark configuration 2): C = A (M, K) * B (K, N)
with B stored (K, N) row-major, fp32 accumulation, fp16 output — the problem of the reference's
dense experiment (experiments/hopper_gemm/gen_inputs.py:26-27), whose oracle is the float64
product computed on the GPU (experiments/hopper_gemm/ref_cutedsl.py:50-74); `reference()` does
the same.  A, B ~ N(0,1) / sqrt(K) rounded to fp16, seeded.  $MOSAICIST_DENSE_DIM overrides
the 8192 (the float64 oracle of the full problem is 4 GB of operands in double and 0.5 GB out).
"""

from __future__ import annotations

import os

from ._common import drop_artifacts, from_env

DIM = int(os.environ.get("MOSAICIST_DENSE_DIM", "8192"))
SEED = 0
KNOBS = {"max_ctas": [0, 128, 74]}
STRUCTURAL = ()
DEFAULTS = {"max_ctas": 0}


def _inputs():
    import torch

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(SEED)
    a = (torch.randn((DIM, DIM), device=dev, generator=g) / DIM ** 0.5).half()
    b = (torch.randn((DIM, DIM), device=dev, generator=g) / DIM ** 0.5).half()
    return a, b


def reference():
    a, b = _inputs()
    return (a.double() @ b.double()).cpu().numpy()


def build():
    import torch

    from .. import ops

    k = from_env(DEFAULTS)
    a, b = _inputs()
    out = torch.empty((DIM, DIM), dtype=torch.float16, device=a.device)
    drop_artifacts("dense", "gemm_dense_f16_kernelILi6ELb0ELb0E")

    def fn():
        return ops.gemm_f16(a, b, out=out, max_ctas=int(k["max_ctas"]))

    return fn, ()
