"""Builds libmosaicist_sm100a.so (and the PTX text beside it) in-tree with nvcc.

    python -m mosaicist_b200.build [--force] [--debug]

`--debug` also builds libmosaicist_sm100a_debug.so with -DMSC_DEBUG: the same kernels plus
per-CTA clock stamps (clock64 and the global nanosecond timer) and pipeline-stage skip flags,
used by `python -m mosaicist_b200.profile_stage --in-kernel-clock`; nothing else loads it.

The library is compiled for sm_100a only.  nvcc cross-compiles without a GPU, so this
runs on a CPU-only machine; the resulting .so is what the GPU machine loads.
"""

from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmosaicist_sm100a.so"
PTX = PKG / "libmosaicist_sm100a.ptx"
#: PTX text per GEMM translation unit; the first is the default kernel and sits where
#: msc_ptx_path() points, the others beside it with a suffix
PTX_UNITS = {"pair": ("gemm_blockscaled_pair.cu", PTX),
             "single": ("gemm_blockscaled.cu", PKG / "libmosaicist_sm100a.single.ptx"),
             "dense": ("gemm_dense_f16.cu", PKG / "libmosaicist_sm100a.dense.ptx")}
PTXAS_LOG = PKG / "libmosaicist_sm100a.ptxas.log"
DEBUG_LIB = PKG / "libmosaicist_sm100a_debug.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo"]


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists() or not all(dst.exists() for _, dst in PTX_UNITS.values()):
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG.parent / "include" / "mosaicist_sm100a.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every .cu under csrc/ into one shared library; returns its path."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not force and not _stale():
        return LIB
    if not pathlib.Path(nvcc).exists():
        if LIB.exists():
            return LIB  # prebuilt library on a machine without the toolkit
        raise RuntimeError("nvcc not found and no prebuilt libmosaicist_sm100a.so")
    srcs = [str(s) for s in sources()]
    cmd = [nvcc, *ARCH, *COMMON, "-Xptxas", "-v", "-shared", "-Xcompiler", "-fPIC",
           "-cudart", "static", "-o", str(LIB), *srcs, "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    PTXAS_LOG.write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stderr[-4000:])
    if verbose:
        print(res.stderr)
    # PTX text of the GEMM kernels: what a capture module hands to the PTX fingerprinter
    for src, dst in PTX_UNITS.values():
        cmd = [nvcc, *ARCH, *COMMON, "-ptx", "-o", str(dst), str(CSRC / src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc -ptx failed:\n" + res.stderr[-4000:])
    return LIB


CUPTI_SHIM = PKG / "cupti_shim" / "libmsc_cupti.so"


def build_cupti_shim(force: bool = False) -> pathlib.Path | None:
    """The small C++ library behind the stand-in `cupti` package (cupti_shim/): kernel activity
    records from libcupti for the reference's tracer, where cupti-python is not installed.
    Returns None (and builds nothing) where the toolkit's CUPTI headers or g++ are missing."""
    src = PKG / "cupti_shim" / "cupti_shim.cpp"
    if not force and CUPTI_SHIM.exists() and CUPTI_SHIM.stat().st_mtime >= src.stat().st_mtime:
        return CUPTI_SHIM
    gxx = shutil.which("g++")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda = pathlib.Path(nvcc).resolve().parents[1]
    if gxx is None or not (cuda / "include" / "cupti.h").exists():
        return CUPTI_SHIM if CUPTI_SHIM.exists() else None
    libdir = cuda / "lib64"
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{cuda / 'include'}", "-o", str(CUPTI_SHIM), str(src),
           f"-L{libdir}", "-lcupti", f"-Wl,-rpath,{libdir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed on the CUPTI shim:\n" + res.stderr[-2000:])
    return CUPTI_SHIM


def build_debug(force: bool = False) -> pathlib.Path:
    """The -DMSC_DEBUG build (clock stamps, skip flags); returns its path."""
    deps = list(CSRC.glob("*")) + [PKG.parent / "include" / "mosaicist_sm100a.h"]
    if not force and DEBUG_LIB.exists() and all(p.stat().st_mtime <= DEBUG_LIB.stat().st_mtime for p in deps):
        return DEBUG_LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *ARCH, *COMMON, "-DMSC_DEBUG", "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
           "-o", str(DEBUG_LIB), *[str(s) for s in sources()], "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stderr[-4000:])
    return DEBUG_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print("built", path)
    print("built", build_cupti_shim(force="--force" in sys.argv))
    if "--debug" in sys.argv:
        print("built", build_debug(force="--force" in sys.argv))
