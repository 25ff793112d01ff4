"""Host-side operators over torch CUDA tensors, named after the reference functions they
replace (experiments/flashinfer-megamoe-sm100a/*.py).  torch supplies device memory and
the stream; all arithmetic happens in libmosaicist_sm100a.so.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib


@dataclass(frozen=True)
class GemmConfig:
    """Knobs of the persistent block-scaled GEMM.  The reference's GemmConfig
    (masked_gemm.py:52-76) tunes block_k / stages of a one-tile-per-CTA kernel; here K
    staging is fixed at 128 bytes per row and the knobs are the tile width, the ring
    depth, the tile order and the persistent grid size.  Zero means library default."""
    tile_n: int = 0
    stages: int = 0
    raster: int = 0
    max_ctas: int = 0
    cta_pair: int = 0
    sf_warps: int = 0

    def c(self, epilogue: int = _lib.EPI_PLAIN) -> _lib.GemmCfg:
        return _lib.GemmCfg(self.tile_n, self.stages, self.raster, self.max_ctas, epilogue,
                            self.cta_pair, self.sf_warps)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtypes, shape=None):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


_BYTES = (torch.uint8, torch.int8, torch.float8_e4m3fn, torch.float8_e8m0fnu)
if hasattr(torch, "float4_e2m1fn_x2"):
    _BYTES = _BYTES + (torch.float4_e2m1fn_x2,)


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Plan:
    """A validated call with its foreign-function arguments already built: running it costs
    one ctypes call on the current stream.  Holds references to the tensors involved."""

    def __init__(self, fn, args, out, keep):
        self._fn, self._args, self.out, self._keep = fn, args, out, keep

    def __call__(self):
        code = self._fn(*self._args, torch.cuda.current_stream().cuda_stream)
        if code:
            _lib.check(code)
        return self.out


def masked_grouped_gemm(a_q, a_sf, b_q, b_sf, alpha=None, masked_m=None,
                        config: GemmConfig = GemmConfig(), out=None) -> torch.Tensor:
    """See masked_grouped_gemm_plan; validates, launches once and returns `out`."""
    return masked_grouped_gemm_plan(a_q, a_sf, b_q, b_sf, alpha, masked_m, config, out)()


def masked_grouped_gemm_plan(a_q, a_sf, b_q, b_sf, alpha=None, masked_m=None,
                             config: GemmConfig = GemmConfig(), out=None) -> Plan:
    """out[l, m, n] = bf16(alpha[l] * dequant(A)[l] @ dequant(B)[l].T), rows >= masked_m[l]
    left untouched.  Same operands as masked_grouped_gemm (masked_gemm.py:104-123):
    a_q (l, m, k/2) packed e2m1, a_sf (l, m/128, k/64, 32, 16) e4m3 in the MMA tiling,
    b_q (l, n, k/2), b_sf (l, n/128, k/64, 32, 16), alpha (l,) f32, masked_m (l,) i32."""
    _need(a_q, "a_q", _BYTES)
    _need(b_q, "b_q", _BYTES)
    l, m, kh = a_q.shape
    n = b_q.shape[1]
    k = kh * 2
    _need(b_q, "b_q", _BYTES, (l, n, kh))
    _need(a_sf, "a_sf", _BYTES, (l, m // 128, k // 64, 32, 16))
    _need(b_sf, "b_sf", _BYTES, (l, n // 128, k // 64, 32, 16))
    if alpha is not None:
        _need(alpha, "alpha", (torch.float32,), (l,))
    if masked_m is not None:
        _need(masked_m, "masked_m", (torch.int32,), (l,))
    if out is None:
        out = torch.empty((l, m, n), dtype=torch.bfloat16, device=a_q.device)
    else:
        _need(out, "out", (torch.bfloat16,), (l, m, n))
    cfg = config.c()
    args = (_ptr(a_q), _ptr(a_sf), _ptr(b_q), _ptr(b_sf), _ptr(alpha), _ptr(masked_m), _ptr(out),
            l, m, n, k, cfg)
    return Plan(_lib.load().msc_grouped_gemm_nvfp4, args, out,
                (a_q, a_sf, b_q, b_sf, alpha, masked_m, cfg))


def _ragged(fn_name, k, a_q, a_sf, b_q, b_sf, alpha, group_offsets, group_rows, row_scale,
            config, out):
    rows_total = a_q.shape[0]
    l, n = b_q.shape[0], b_q.shape[1]
    _need(group_offsets, "group_offsets", (torch.int32,), (l,))
    _need(group_rows, "group_rows", (torch.int32,), (l,))
    if alpha is not None:
        _need(alpha, "alpha", (torch.float32,), (l,))
    if row_scale is not None:
        _need(row_scale, "row_scale", (torch.float32,), (rows_total,))
    if out is None:
        out = torch.empty((rows_total, n), dtype=torch.bfloat16, device=a_q.device)
    else:
        _need(out, "out", (torch.bfloat16,), (rows_total, n))
    cfg = config.c(_lib.EPI_ROW_SCALE if row_scale is not None else _lib.EPI_PLAIN)
    _lib.check(getattr(_lib.load(), fn_name)(
        _ptr(a_q), _ptr(a_sf), _ptr(b_q), _ptr(b_sf), _ptr(alpha), _ptr(group_offsets),
        _ptr(group_rows), _ptr(row_scale), _ptr(out), l, rows_total, n, k, cfg, _stream()))
    return out


def ragged_grouped_gemm_nvfp4(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha=None,
                              row_scale=None, config: GemmConfig = GemmConfig(), out=None):
    """NVFP4 grouped GEMM over row-concatenated groups: group g owns rows
    [group_offsets[g], +group_rows[g]) of a_q (rows_total, k/2) and out (rows_total, n);
    offsets are multiples of 128.  Per-group arithmetic as masked_grouped_gemm."""
    _need(a_q, "a_q", _BYTES)
    rows_total, kh = a_q.shape
    k = kh * 2
    l, n = b_q.shape[0], b_q.shape[1]
    _need(b_q, "b_q", _BYTES, (l, n, kh))
    _need(a_sf, "a_sf", _BYTES, ((rows_total + 127) // 128, k // 64, 32, 16))
    _need(b_sf, "b_sf", _BYTES, (l, n // 128, k // 64, 32, 16))
    return _ragged("msc_grouped_gemm_nvfp4_ragged", k, a_q, a_sf, b_q, b_sf, alpha,
                   group_offsets, group_rows, row_scale, config, out)


def ragged_grouped_gemm_mxfp8(a_q, a_sf, b_q, b_sf, group_offsets, group_rows, alpha=None,
                              row_scale=None, config: GemmConfig = GemmConfig(), out=None):
    """MXFP8 grouped GEMM (e4m3 values, ue8m0 scale per 32) over row-concatenated groups.
    a_q (rows_total, k) e4m3, a_sf (ceil(rows_total/128), k/128, 32, 16) ue8m0, b_q (l, n, k),
    b_sf (l, n/128, k/128, 32, 16)."""
    _need(a_q, "a_q", _BYTES)
    rows_total, k = a_q.shape
    l, n = b_q.shape[0], b_q.shape[1]
    _need(b_q, "b_q", _BYTES, (l, n, k))
    _need(a_sf, "a_sf", _BYTES, ((rows_total + 127) // 128, k // 128, 32, 16))
    _need(b_sf, "b_sf", _BYTES, (l, n // 128, k // 128, 32, 16))
    return _ragged("msc_grouped_gemm_mxfp8_ragged", k, a_q, a_sf, b_q, b_sf, alpha,
                   group_offsets, group_rows, row_scale, config, out)


def quantize_nvfp4(x, global_scale, masked_m=None, tiled_scales: bool = True):
    """(l, m, k) bf16/f32 -> (q (l, m, k/2) packed e2m1, sf e4m3).  Arithmetic of
    quantize_nvfp4 (nvfp4.py:39-57) / quantize_nvfp4_pallas (quantize_kernels.py:119).
    With tiled_scales the scales come out in the MMA tiling (l, m/128, k/64, 32, 16),
    otherwise row-major (l, m, k/16) as the reference kernel writes them.  Rows at or
    beyond masked_m[l] are left untouched."""
    _need(x, "x", (torch.bfloat16, torch.float32))
    l, m, k = x.shape
    _need(global_scale, "global_scale", (torch.float32,), (l,))
    if masked_m is not None:
        _need(masked_m, "masked_m", (torch.int32,), (l,))
    q = torch.empty((l, m, k // 2), dtype=torch.uint8, device=x.device)
    shape = (l, m // 128, k // 64, 32, 16) if tiled_scales else (l, m, k // 16)
    sf = torch.zeros(shape, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().msc_nvfp4_quantize(
        _ptr(x), 0 if x.dtype == torch.bfloat16 else 1, _ptr(global_scale), _ptr(masked_m),
        _ptr(q), _ptr(sf), 1 if tiled_scales else 0, l, m, k, _stream()))
    return q, sf


def silu_mul_quantize_nvfp4(gateup, global_scale, masked_m=None, tiled_scales: bool = True):
    """(l, m, 2n) bf16 -> NVFP4 of silu(gate) * up, gate = first n columns, activation kept in
    fp32 up to the quantiser (nvfp4.py:81-88; silu_mul_quantize_nvfp4_pallas,
    quantize_kernels.py:162)."""
    _need(gateup, "gateup", (torch.bfloat16,))
    l, m, n2 = gateup.shape
    n = n2 // 2
    _need(global_scale, "global_scale", (torch.float32,), (l,))
    if masked_m is not None:
        _need(masked_m, "masked_m", (torch.int32,), (l,))
    q = torch.empty((l, m, n // 2), dtype=torch.uint8, device=gateup.device)
    shape = (l, m // 128, n // 64, 32, 16) if tiled_scales else (l, m, n // 16)
    sf = torch.zeros(shape, dtype=torch.uint8, device=gateup.device)
    _lib.check(_lib.load().msc_nvfp4_silu_mul_quantize(
        _ptr(gateup), _ptr(global_scale), _ptr(masked_m), _ptr(q), _ptr(sf),
        1 if tiled_scales else 0, l, m, n, _stream()))
    return q, sf


def quantize_nvfp4_ragged(x, global_scale, group_offsets, group_rows, silu: bool = False,
                          out=None):
    """Ragged-layout quantiser: x (rows_total, k) -> q (rows_total, k/2) and tiled scales
    (ceil(rows_total/128), k/64, 32, 16); with silu, x is (rows_total, 2k) gate|up.  `out`
    may carry preallocated (q, sf)."""
    _need(x, "x", (torch.bfloat16, torch.float32))
    rows_total = x.shape[0]
    k = x.shape[1] // 2 if silu else x.shape[1]
    l = global_scale.shape[0]
    _need(global_scale, "global_scale", (torch.float32,), (l,))
    _need(group_offsets, "group_offsets", (torch.int32,), (l,))
    _need(group_rows, "group_rows", (torch.int32,), (l,))
    if out is None:
        q = torch.empty((rows_total, k // 2), dtype=torch.uint8, device=x.device)
        sf = torch.zeros(((rows_total + 127) // 128, k // 64, 32, 16), dtype=torch.uint8,
                         device=x.device)
    else:
        q, sf = out
        _need(q, "q", (torch.uint8,), (rows_total, k // 2))
        _need(sf, "sf", (torch.uint8,), ((rows_total + 127) // 128, k // 64, 32, 16))
    _lib.check(_lib.load().msc_nvfp4_quantize_ragged(
        _ptr(x), 0 if x.dtype == torch.bfloat16 else 1, _ptr(global_scale), _ptr(group_offsets),
        _ptr(group_rows), _ptr(q), _ptr(sf), l, rows_total, k, 1 if silu else 0, _stream()))
    return q, sf


def global_scale_for(x, numerator: float = 2688.0, out=None):
    """(l, ...) bf16/f32 -> (l,) f32: numerator / max|x[l]|, a maximum of 0 counted as 1 -
    global_scale_for (nvfp4.py:29-36; 2688 = 6 * 448)."""
    _need(x, "x", (torch.bfloat16, torch.float32))
    l = x.shape[0]
    per = x.numel() // l
    if out is None:
        out = torch.empty((l,), dtype=torch.float32, device=x.device)
    else:
        _need(out, "out", (torch.float32,), (l,))
    _lib.check(_lib.load().msc_amax_global_scale(_ptr(x), 0 if x.dtype == torch.bfloat16 else 1, l, per,
                                                 float(numerator), _ptr(out), _stream()))
    return out


def quantize_mxfp8(x, tiled_scales: bool = True, group_offsets=None, group_rows=None, out=None):
    """(rows, k) bf16/f32 -> (q (rows, k) e4m3 bytes, sf ue8m0 bytes): one power-of-two scale per
    32 K-elements, the smallest with blockmax / scale <= 448 (structure of the reference's
    block-scaled FP8 quantiser, flashinfer-megamoe-sm90a/quant.py:47-75, with the MX scale rule).
    Scales come out in the MMA tiling (ceil(rows/128), k/128, 32, 16) or row-major (rows, k/32).
    With group_offsets / group_rows only rows inside a group are written (tiled scales)."""
    _need(x, "x", (torch.bfloat16, torch.float32))
    rows, k = x.shape
    ragged = group_offsets is not None
    if ragged and not tiled_scales:
        raise ValueError("the ragged form writes tiled scales")
    if out is None:
        q = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
        shape = ((rows + 127) // 128, k // 128, 32, 16) if tiled_scales else (rows, k // 32)
        sf = torch.zeros(shape, dtype=torch.uint8, device=x.device)
    else:
        q, sf = out
    dt = 0 if x.dtype == torch.bfloat16 else 1
    if ragged:
        l = group_offsets.shape[0]
        _need(group_offsets, "group_offsets", (torch.int32,), (l,))
        _need(group_rows, "group_rows", (torch.int32,), (l,))
        _lib.check(_lib.load().msc_mxfp8_quantize_ragged(_ptr(x), dt, _ptr(group_offsets), _ptr(group_rows),
                                                         _ptr(q), _ptr(sf), l, rows, k, _stream()))
    else:
        _lib.check(_lib.load().msc_mxfp8_quantize(_ptr(x), dt, _ptr(q), _ptr(sf), 1 if tiled_scales else 0,
                                                  rows, k, _stream()))
    return q, sf


def to_mma_scale_layout(sf):
    """(groups, mn, k_scales) row-major scale bytes -> (groups, ceil(mn/128), k_scales/4, 32, 16)
    (a 2-D input is treated as one group and returns 4-D), as to_mma_scale_layout
    (nvfp4.py:121-131)."""
    _need(sf, "sf", _BYTES)
    squeeze = sf.dim() == 2
    if squeeze:
        sf = sf.unsqueeze(0)
    g, mn, ks = sf.shape
    out = torch.empty((g, (mn + 127) // 128, ks // 4, 32, 16), dtype=sf.dtype, device=sf.device)
    _lib.check(_lib.load().msc_sf_swizzle(_ptr(sf), _ptr(out), g, mn, ks, _stream()))
    return out[0] if squeeze else out


def gemm_f16(a, b, out=None, max_ctas: int = 0):
    """C = A @ B for 2-D fp16 or bf16 CUDA tensors, A (m, k) and B (k, n) row-major (rows may be
    strided: a column slice of a wider matrix works as is), fp32 accumulation, output in the
    input dtype.  The reference's dense problem (experiments/hopper_gemm/ref_cutedsl.py:50-74)."""
    if a.dtype != b.dtype or a.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("a and b must both be float16 or both bfloat16")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"shapes {tuple(a.shape)} and {tuple(b.shape)} do not multiply")
    if not (a.is_cuda and b.is_cuda) or a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("a and b must be CUDA tensors with unit stride along their rows")
    m, k = a.shape
    n = b.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    elif out.dtype != a.dtype or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be (m, n) in the input dtype with unit stride along rows")
    _lib.check(_lib.load().msc_gemm_f16(_ptr(a), _ptr(b), _ptr(out), m, n, k, a.stride(0), b.stride(0),
                                        out.stride(0), 0 if a.dtype == torch.float16 else 1, max_ctas,
                                        _stream()))
    return out


def dequant_int4(b_q, scales, group_size: int = 128, out=None):
    """(l, n, k/2) packed int4 + (l, n, k/group_size) bf16 scales -> (l, n, k) bf16, the multiply
    done in bf16 (ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-81)."""
    _need(b_q, "b_q", (torch.uint8, torch.int8))
    l, n, kh = b_q.shape
    k = kh * 2
    _need(scales, "scales", (torch.bfloat16,), (l, n, k // group_size))
    if out is None:
        out = torch.empty((l, n, k), dtype=torch.bfloat16, device=b_q.device)
    _lib.check(_lib.load().msc_int4_dequant_bf16(_ptr(b_q), _ptr(scales), _ptr(out), l, n, k, group_size,
                                                 _stream()))
    return out


def ragged_grouped_gemm_bf16(a, b, group_offsets, group_rows, alpha=None, out=None, max_ctas: int = 0):
    """out[off_g + r] = bf16(alpha_g * a[off_g + r] @ b[g].T), r < group_rows[g]; a (rows_total, k)
    bf16, b (l, n, k) bf16, fp32 accumulation."""
    _need(a, "a", (torch.bfloat16,))
    rows_total, k = a.shape
    l, n = b.shape[0], b.shape[1]
    _need(b, "b", (torch.bfloat16,), (l, n, k))
    _need(group_offsets, "group_offsets", (torch.int32,), (l,))
    _need(group_rows, "group_rows", (torch.int32,), (l,))
    if alpha is not None:
        _need(alpha, "alpha", (torch.float32,), (l,))
    if out is None:
        out = torch.empty((rows_total, n), dtype=torch.bfloat16, device=a.device)
    _lib.check(_lib.load().msc_grouped_gemm_bf16_ragged(_ptr(a), _ptr(b), _ptr(alpha), _ptr(group_offsets),
                                                        _ptr(group_rows), _ptr(out), l, rows_total, n, k,
                                                        max_ctas, _stream()))
    return out


def mixed_grouped_gemm_int4(a, b_q, scales, group_offsets, group_rows, alpha=None, group_size: int = 128,
                            workspace=None, out=None, fused: bool | None = None, max_ctas: int = 0):
    """bf16 activations x int4 weights (ports/hopper_mixed_dtype_grouped_gemm/problems.py:75-87).

    fused (default whenever k and group_size are multiples of 64): one kernel, converter warps
    expand each stage of packed weights to bf16 in shared memory on their way to the tensor
    core; the weights cross HBM once, as int4.  Otherwise two launches: expand the weights to
    bf16 (`workspace`, (l, n, k) bf16, reusable while the weights do not change) and run the
    grouped bf16 GEMM.  Both produce the same bits."""
    _need(b_q, "b_q", (torch.uint8, torch.int8))
    l, n, kh = b_q.shape
    k = kh * 2
    can_fuse = k % 64 == 0 and group_size % 64 == 0 and k % group_size == 0
    if fused is None:
        fused = can_fuse and workspace is None
    if not fused:
        b = dequant_int4(b_q, scales, group_size, out=workspace)
        return ragged_grouped_gemm_bf16(a, b, group_offsets, group_rows, alpha, out=out, max_ctas=max_ctas)
    if not can_fuse:
        raise ValueError("the fused kernel needs k and group_size to be multiples of 64")
    _need(a, "a", (torch.bfloat16,))
    rows_total = a.shape[0]
    _need(a, "a", (torch.bfloat16,), (rows_total, k))
    _need(scales, "scales", (torch.bfloat16,), (l, n, k // group_size))
    _need(group_offsets, "group_offsets", (torch.int32,), (l,))
    _need(group_rows, "group_rows", (torch.int32,), (l,))
    if alpha is not None:
        _need(alpha, "alpha", (torch.float32,), (l,))
    if out is None:
        out = torch.empty((rows_total, n), dtype=torch.bfloat16, device=a.device)
    _lib.check(_lib.load().msc_grouped_gemm_bf16_int4_ragged(
        _ptr(a), _ptr(b_q), _ptr(scales), _ptr(alpha), _ptr(group_offsets), _ptr(group_rows), _ptr(out), l,
        rows_total, n, k, group_size, max_ctas, _stream()))
    return out


def swiglu_interleave_w1(w1_q, w1_sf):
    """w1 (l, 2n, k/2) + tiled scales -> the copy the tokens-on-N fused GEMM1 reads
    (GemmConfig(cta_pair=3)): gate and up rows interleaved in blocks of 64."""
    _need(w1_q, "w1_q", _BYTES)
    l, n2, kh = w1_q.shape
    _need(w1_sf, "w1_sf", _BYTES, (l, n2 // 128, kh // 32, 32, 16))
    out_q, out_sf = torch.empty_like(w1_q), torch.empty_like(w1_sf)
    _lib.check(_lib.load().msc_swiglu_interleave_w1(_ptr(w1_q), _ptr(w1_sf), _ptr(out_q), _ptr(out_sf), l, n2,
                                                    kh * 2, _stream()))
    return out_q, out_sf


def ragged_gemm1_swiglu_quantize(a_q, a_sf, w1_q, w1_sf, group_offsets, group_rows, alpha, out_global_scale,
                                 config: GemmConfig = GemmConfig(), out=None):
    """GEMM1 + SiLU(gate) * up + NVFP4 requantisation in one kernel (the reference's
    gemm1_silu_quantize, gemm1_silu_quantize.py:94): returns (d_q (rows_total, n/2),
    d_sf tiled (rows_total/128, n/64, 32, 16)) with n = w1 rows / 2, bit-identical to the GEMM
    followed by the stand-alone SiLU quantiser."""
    _need(a_q, "a_q", _BYTES)
    rows_total, kh = a_q.shape
    k = kh * 2
    l, n2 = w1_q.shape[0], w1_q.shape[1]
    n = n2 // 2
    _need(w1_q, "w1_q", _BYTES, (l, n2, kh))
    _need(a_sf, "a_sf", _BYTES, ((rows_total + 127) // 128, k // 64, 32, 16))
    _need(w1_sf, "w1_sf", _BYTES, (l, n2 // 128, k // 64, 32, 16))
    _need(group_offsets, "group_offsets", (torch.int32,), (l,))
    _need(group_rows, "group_rows", (torch.int32,), (l,))
    _need(alpha, "alpha", (torch.float32,), (l,))
    _need(out_global_scale, "out_global_scale", (torch.float32,), (l,))
    if out is None:
        d_q = torch.empty((rows_total, n // 2), dtype=torch.uint8, device=a_q.device)
        d_sf = torch.zeros(((rows_total + 127) // 128, n // 64, 32, 16), dtype=torch.uint8, device=a_q.device)
    else:
        d_q, d_sf = out
        _need(d_q, "d_q", (torch.uint8,), (rows_total, n // 2))
        _need(d_sf, "d_sf", (torch.uint8,), ((rows_total + 127) // 128, n // 64, 32, 16))
    _lib.check(_lib.load().msc_grouped_gemm_nvfp4_swiglu_ragged(
        _ptr(a_q), _ptr(a_sf), _ptr(w1_q), _ptr(w1_sf), _ptr(alpha), _ptr(group_offsets), _ptr(group_rows),
        _ptr(out_global_scale), _ptr(d_q), _ptr(d_sf), l, rows_total, n2, k, config.c(), _stream()))
    return d_q, d_sf
