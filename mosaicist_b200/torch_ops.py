"""The masked grouped GEMM as a torch custom operator, `torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4`,
for callers that build graphs of torch operators (tracing, FakeTensor shape propagation) instead of
calling `ops.masked_grouped_gemm` directly.  Same operands as the reference's masked_grouped_gemm
(masked_gemm.py:104-123) and FlashInfer's grouped_gemm_nt_masked call site
(experiments/loop/ref_flashinfer_gemm.py:25-31); the CUDA implementation is the C-ABI entry point
msc_grouped_gemm_nvfp4.  Importing this module registers the operator; it needs no GPU.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops


@torch.library.custom_op("mosaicist_sm100a::grouped_gemm_nvfp4", mutates_args=(), device_types="cuda")
def grouped_gemm_nvfp4(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor,
                       alpha: Optional[torch.Tensor], masked_m: Optional[torch.Tensor]) -> torch.Tensor:
    """(l, m, k/2) x (l, n, k/2) packed e2m1 with tiled e4m3 scales -> (l, m, n) bf16; rows at or
    beyond masked_m[l] come back as zeros (the operator returns a fresh tensor, so "left
    untouched" has nothing to leave)."""
    l, m = a_q.shape[0], a_q.shape[1]
    out = torch.zeros((l, m, b_q.shape[1]), dtype=torch.bfloat16, device=a_q.device)
    return ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, alpha, masked_m, out=out)


@grouped_gemm_nvfp4.register_fake
def _(a_q, a_sf, b_q, b_sf, alpha, masked_m):
    return a_q.new_empty((a_q.shape[0], a_q.shape[1], b_q.shape[1]), dtype=torch.bfloat16)
