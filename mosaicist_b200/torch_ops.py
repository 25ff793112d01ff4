"""The hot-path operators as torch custom operators (`torch.ops.mosaicist_sm100a.*`), for callers
that build graphs of torch operators (tracing, FakeTensor shape propagation) instead of calling
`mosaicist_b200.ops` directly:

    grouped_gemm_nvfp4         masked grouped GEMM, the operands of the reference's
                               masked_grouped_gemm (masked_gemm.py:104-123) and of FlashInfer's
                               grouped_gemm_nt_masked call site (ref_flashinfer_gemm.py:25-31)
    grouped_gemm_nvfp4_ragged  the same arithmetic over row-concatenated groups
    quantize_nvfp4             quantize_nvfp4 (nvfp4.py:39-57) with scales in the MMA tiling
    silu_mul_quantize_nvfp4    silu_mul (nvfp4.py:81-88) + quantize_nvfp4
    global_scale_for           global_scale_for (nvfp4.py:29-36)
    quantize_mxfp8             e4m3 values + one ue8m0 scale per 32, scales in the MMA tiling
    grouped_gemm_mxfp8_ragged  the MXFP8 grouped GEMM over row-concatenated groups
    gemm_f16                   the dense fp16 / bf16 problem (hopper_gemm/ref_cutedsl.py:50-74)
    grouped_gemm_bf16_int4_ragged   bf16 x int4 grouped GEMM (problems.py:75-87)
    moe_masked                 the masked MoE layer, arguments of the reference's moe_masked
                               (experiments/flashinfer-megamoe-sm100a/moe.py:47-79)

Each is the corresponding C-ABI entry point.  Operators return fresh tensors, so rows a masked
call leaves untouched come back as zeros.  Importing this module registers the operators; it
needs no GPU.
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


@torch.library.custom_op("mosaicist_sm100a::grouped_gemm_nvfp4_ragged", mutates_args=(), device_types="cuda")
def grouped_gemm_nvfp4_ragged(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor,
                              group_offsets: torch.Tensor, group_rows: torch.Tensor,
                              alpha: Optional[torch.Tensor], row_scale: Optional[torch.Tensor]) -> torch.Tensor:
    """(rows_total, k/2) x (l, n, k/2) -> (rows_total, n) bf16, group g owning rows
    [group_offsets[g], + group_rows[g]); rows outside every group come back as zeros."""
    out = torch.zeros((a_q.shape[0], b_q.shape[1]), dtype=torch.bfloat16, device=a_q.device)
    return ops.ragged_grouped_gemm_nvfp4(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha, row_scale, out=out)


@grouped_gemm_nvfp4_ragged.register_fake
def _(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha, row_scale):
    return a_q.new_empty((a_q.shape[0], b_q.shape[1]), dtype=torch.bfloat16)


def _quantized_shapes(l, m, k):
    return (l, m, k // 2), (l, m // 128, k // 64, 32, 16)


@torch.library.custom_op("mosaicist_sm100a::quantize_nvfp4", mutates_args=(), device_types="cuda")
def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor,
                   masked_m: Optional[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """(l, m, k) bf16 / f32 -> packed e2m1 (l, m, k/2) and tiled e4m3 scales (l, m/128, k/64, 32, 16)."""
    q, sf = ops.quantize_nvfp4(x, global_scale, masked_m)
    if masked_m is not None:          # rows the kernel left untouched are uninitialised in q
        rows = torch.arange(x.shape[1], device=x.device)[None, :, None] < masked_m[:, None, None]
        q = torch.where(rows, q, torch.zeros_like(q))
    return q, sf


@quantize_nvfp4.register_fake
def _(x, global_scale, masked_m):
    qs, ss = _quantized_shapes(*x.shape)
    return x.new_empty(qs, dtype=torch.uint8), x.new_empty(ss, dtype=torch.uint8)


@torch.library.custom_op("mosaicist_sm100a::silu_mul_quantize_nvfp4", mutates_args=(), device_types="cuda")
def silu_mul_quantize_nvfp4(gateup: torch.Tensor, global_scale: torch.Tensor,
                            masked_m: Optional[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """(l, m, 2n) bf16 -> NVFP4 of silu(gate) * up: (l, m, n/2) and (l, m/128, n/64, 32, 16)."""
    q, sf = ops.silu_mul_quantize_nvfp4(gateup, global_scale, masked_m)
    if masked_m is not None:
        rows = torch.arange(gateup.shape[1], device=gateup.device)[None, :, None] < masked_m[:, None, None]
        q = torch.where(rows, q, torch.zeros_like(q))
    return q, sf


@silu_mul_quantize_nvfp4.register_fake
def _(gateup, global_scale, masked_m):
    l, m, n2 = gateup.shape
    qs, ss = _quantized_shapes(l, m, n2 // 2)
    return gateup.new_empty(qs, dtype=torch.uint8), gateup.new_empty(ss, dtype=torch.uint8)


@torch.library.custom_op("mosaicist_sm100a::global_scale_for", mutates_args=(), device_types="cuda")
def global_scale_for(x: torch.Tensor) -> torch.Tensor:
    """(l, ...) bf16 / f32 -> (l,) f32 = 2688 / max|x[l]| (a maximum of 0 counted as 1)."""
    return ops.global_scale_for(x)


@global_scale_for.register_fake
def _(x):
    return x.new_empty((x.shape[0],), dtype=torch.float32)


@torch.library.custom_op("mosaicist_sm100a::quantize_mxfp8", mutates_args=(), device_types="cuda")
def quantize_mxfp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(rows, k) bf16 / f32 -> e4m3 bytes (rows, k) and tiled ue8m0 scales (ceil(rows/128), k/128, 32, 16)."""
    return ops.quantize_mxfp8(x)


@quantize_mxfp8.register_fake
def _(x):
    rows, k = x.shape
    return x.new_empty((rows, k), dtype=torch.uint8), x.new_empty(((rows + 127) // 128, k // 128, 32, 16), dtype=torch.uint8)


@torch.library.custom_op("mosaicist_sm100a::grouped_gemm_mxfp8_ragged", mutates_args=(), device_types="cuda")
def grouped_gemm_mxfp8_ragged(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor,
                              group_offsets: torch.Tensor, group_rows: torch.Tensor,
                              alpha: Optional[torch.Tensor], row_scale: Optional[torch.Tensor]) -> torch.Tensor:
    """(rows_total, k) x (l, n, k) e4m3 with tiled ue8m0 scales -> (rows_total, n) bf16; rows outside
    every group come back as zeros."""
    out = torch.zeros((a_q.shape[0], b_q.shape[1]), dtype=torch.bfloat16, device=a_q.device)
    return ops.ragged_grouped_gemm_mxfp8(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha, row_scale, out=out)


@grouped_gemm_mxfp8_ragged.register_fake
def _(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha, row_scale):
    return a_q.new_empty((a_q.shape[0], b_q.shape[1]), dtype=torch.bfloat16)


@torch.library.custom_op("mosaicist_sm100a::gemm_f16", mutates_args=(), device_types="cuda")
def gemm_f16(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """C = A (m, k) @ B (k, n), fp16 or bf16 in and out, fp32 accumulation."""
    return ops.gemm_f16(a, b)


@gemm_f16.register_fake
def _(a, b):
    return a.new_empty((a.shape[0], b.shape[1]))


@torch.library.custom_op("mosaicist_sm100a::grouped_gemm_bf16_int4_ragged", mutates_args=(), device_types="cuda")
def grouped_gemm_bf16_int4_ragged(a: torch.Tensor, b_q: torch.Tensor, scales: torch.Tensor,
                                  group_offsets: torch.Tensor, group_rows: torch.Tensor,
                                  alpha: Optional[torch.Tensor], group_size: int) -> torch.Tensor:
    """bf16 (rows_total, k) x packed int4 (l, n, k/2) with bf16 scales (l, n, k/group_size) ->
    (rows_total, n) bf16; rows outside every group come back as zeros."""
    out = torch.zeros((a.shape[0], b_q.shape[1]), dtype=torch.bfloat16, device=a.device)
    return ops.mixed_grouped_gemm_int4(a, b_q, scales, group_offsets, group_rows, alpha, group_size, out=out)


@grouped_gemm_bf16_int4_ragged.register_fake
def _(a, b_q, scales, group_offsets, group_rows, alpha, group_size):
    return a.new_empty((a.shape[0], b_q.shape[1]), dtype=torch.bfloat16)


@torch.library.custom_op("mosaicist_sm100a::moe_masked", mutates_args=(), device_types="cuda")
def moe_masked(hidden: torch.Tensor, w1_q: torch.Tensor, w1_sf: torch.Tensor, w1_gs: torch.Tensor,
               w1_alpha: torch.Tensor, w2_q: torch.Tensor, w2_sf: torch.Tensor, w2_gs: torch.Tensor,
               w2_alpha: torch.Tensor, masked_m: torch.Tensor, input_global_scale: torch.Tensor,
               a2_global_scale: torch.Tensor) -> torch.Tensor:
    """(l, m, k) bf16 -> (l, m, k) bf16: quantise, GEMM1, SiLU(gate) * up + quantise, GEMM2 per
    expert batch; rows at or beyond masked_m[l] come back as zeros."""
    from . import moe

    out = moe.moe_masked(hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, masked_m,
                         input_global_scale, a2_global_scale)
    rows = torch.arange(hidden.shape[1], device=hidden.device)[None, :, None] < masked_m[:, None, None]
    return torch.where(rows, out, torch.zeros_like(out))


@moe_masked.register_fake
def _(hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, masked_m, input_global_scale,
      a2_global_scale):
    return hidden.new_empty(hidden.shape, dtype=torch.bfloat16)
