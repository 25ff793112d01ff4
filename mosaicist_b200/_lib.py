"""ctypes binding of libmosaicist_sm100a.so.

The library is the product: if it cannot be loaded every operator raises — there is no
CPU or PyTorch fallback behind these calls.
"""

from __future__ import annotations

import ctypes
import os
import pathlib

PKG = pathlib.Path(__file__).resolve().parent
#: MSC_LIB_PATH selects another build of the same library (e.g. one compiled with -DMSC_DEBUG)
LIB_PATH = pathlib.Path(os.environ.get("MSC_LIB_PATH") or PKG / "libmosaicist_sm100a.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_SMEM, ERR_CUDA, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5
EPI_PLAIN, EPI_ROW_SCALE = 0, 1


class MscError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{message} (libmosaicist_sm100a status {code})")
        self.code = code


class GemmCfg(ctypes.Structure):
    _fields_ = [("tile_n", ctypes.c_int), ("stages", ctypes.c_int), ("raster", ctypes.c_int),
                ("max_ctas", ctypes.c_int), ("epilogue", ctypes.c_int),
                ("cta_pair", ctypes.c_int), ("sf_warps", ctypes.c_int), ("reserved", ctypes.c_int)]


_P, _I = ctypes.c_void_p, ctypes.c_int
_CFG = ctypes.POINTER(GemmCfg)

#: every symbol include/mosaicist_sm100a.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "msc_version": (_I, []),
    "msc_last_error": (ctypes.c_char_p, []),
    "msc_shutdown": (_I, []),
    "msc_ptx_path": (ctypes.c_char_p, []),
    "msc_status_word_read": (_I, [ctypes.POINTER(ctypes.c_int)]),
    "msc_grouped_gemm_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _CFG, _P]),
    "msc_grouped_gemm_nvfp4_ragged": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _CFG, _P]),
    "msc_grouped_gemm_nvfp4_swiglu_ragged": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _CFG, _P]),
    "msc_grouped_gemm_mxfp8_ragged": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _CFG, _P]),
    "msc_nvfp4_quantize": (_I, [_P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "msc_nvfp4_silu_mul_quantize": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "msc_nvfp4_quantize_ragged": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "msc_sf_swizzle": (_I, [_P, _P, _I, _I, _I, _P]),
    "msc_amax_global_scale": (_I, [_P, _I, _I, ctypes.c_longlong, ctypes.c_float, _P, _P]),
    "msc_mxfp8_quantize": (_I, [_P, _I, _P, _P, _I, _I, _I, _P]),
    "msc_mxfp8_quantize_ragged": (_I, [_P, _I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "msc_gemm_f16": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "msc_int4_dequant_bf16": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "msc_grouped_gemm_bf16_ragged": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "msc_grouped_gemm_bf16_int4_ragged": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "msc_swiglu_interleave_w1": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "msc_moe_route_topk": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "msc_moe_plan": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "msc_moe_plan_noalloc": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _P]),
    "msc_moe_permute_quantize": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P, _P]),
    "msc_moe_unpermute": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "msc_peer_alloc": (_I, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), _P]),
    "msc_peer_open": (_I, [_P, ctypes.POINTER(ctypes.c_void_p)]),
    "msc_peer_close": (_I, [_P]),
    "msc_peer_free": (_I, [_P]),
    "msc_ep_offsets": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P]),
    "msc_ep_signal": (_I, [_P, _I, _I, _I, _I, _P, _P, _I, _P]),
    "msc_ep_wait": (_I, [_P, _I, _I, _I, _P]),
    "msc_ep_dispatch_quantize": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P, _P]),
    "msc_ep_presum_push": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "msc_ep_sum_pairs": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "msc_grouped_gemm_nvfp4_scatter_ragged": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _CFG, _P]),
    "msc_ep_combine": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library, with argument types set.  Raises if it is missing."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise MscError(ERR_CUDA, f"{LIB_PATH} is missing: run `python -m mosaicist_b200.build`")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise MscError(code, load().msc_last_error().decode() or "libmosaicist_sm100a call failed")


def status_word() -> int:
    """Reads and clears the device status word (synchronises the device)."""
    out = ctypes.c_int(0)
    check(load().msc_status_word_read(ctypes.byref(out)))
    return out.value
