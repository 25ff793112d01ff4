"""The capture modules driven by the reference's OWN capture stage on a GPU.

`mosaicist.capture.capture()` (src/mosaicist/capture.py:229-271) imports a module, calls its
build(), runs the callable under CUPTI activity tracing, gathers the PTX / ptxas log the module
dropped, saves out0.npy and - from the module's reference() - oracle0.npy, and writes a bundle.
These tests run exactly that, unchanged, on this library's modules and check what the
convergence loop would read next: the PTX fingerprints and its largest entry is the kernel that
ran, the numerics gate passes on the saved arrays, the launch record is the kernel's, and the
CUPTI per-launch time agrees with CUDA-event timing.

Needs the reference's Python package (staged by oracle/stage_reference.py, or $MOSAICIST_REFERENCE)
and a `cupti` module: the cupti-python package, or this repository's stand-in over libcupti
(mosaicist_b200/cupti_shim).  Skipped, with the reason, where either is missing."""

import importlib
import pathlib
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]


@pytest.fixture()
def reference_capture(monkeypatch, tmp_path):
    from oracle.stage_reference import staged_path

    ref = staged_path()
    if ref is None:
        pytest.skip("the reference's package is neither staged (oracle/stage_reference.py) nor in MOSAICIST_REFERENCE")
    monkeypatch.syspath_prepend(str(ref))
    try:
        importlib.import_module("cupti.cupti")
    except ImportError:
        shim = ROOT / "mosaicist_b200" / "cupti_shim"
        if not (shim / "libmsc_cupti.so").exists():
            pytest.skip("no cupti-python and mosaicist_b200/cupti_shim/libmsc_cupti.so is not built")
        for name in [m for m in sys.modules if m == "cupti" or m.startswith("cupti.")]:
            monkeypatch.delitem(sys.modules, name)
        monkeypatch.syspath_prepend(str(shim))
        try:
            importlib.import_module("cupti.cupti")._load()
        except (ImportError, OSError) as exc:
            pytest.skip(f"libcupti cannot be loaded here: {exc}")
    monkeypatch.setenv("MOSAIC_GPU_DUMP_TO", str(tmp_path / "dump"))
    monkeypatch.delenv("MOSAICIST_KNOBS", raising=False)
    from mosaicist import capture as C

    return C, tmp_path / "bundle"


def _event_us(fn, args, reps=30):
    for _ in range(5):
        fn(*args)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn(*args)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / reps


@pytest.mark.parametrize("name,measure,kernel", [("cand_cuda_gemm", "dominant", "gemm_pair_kernel"),
                                                 ("cand_cuda_moe", "all", "gemm_pair_kernel")])
def test_reference_capture_stage_drives_the_module(reference_capture, name, measure, kernel):
    C, out = reference_capture
    from mosaicist.bundle import Bundle
    from mosaicist.ptx.parse import parse
    from mosaicist.verify.numerics import compare_outputs
    from mosaicist.verify.formats import round_to_format

    entry = f"mosaicist_b200.candidates.{name}"
    bundle = C.capture(entry, "pallas", out, reps=30, warmup=5, arch="sm_100a", measure=measure)

    # artifacts: a PTX whose largest entry is the kernel that ran, the ptxas log, a bundle that loads
    ptx = (out / "kernel.ptx").read_text()
    assert kernel in parse(ptx).entry(None).name
    assert (out / "ptxas.log").exists()
    loaded = Bundle.load(out)
    fp = loaded.fingerprint()
    assert fp is not None and loaded.kind == "candidate" and loaded.ptx == "kernel.ptx"

    # launch record of the dominant kernel: a persistent grid of CTA pairs, 320 threads
    assert bundle.launch.block == [320, 1, 1] and bundle.launch.cluster == [2, 1, 1]
    assert bundle.launch.grid[0] % 2 == 0 and 2 <= bundle.launch.grid[0] <= 148
    assert bundle.resources["registers"] > 0

    # outputs and the float64 opinion are saved, and the reference's own gate passes on them
    got, oracle = np.load(out / "out0.npy"), np.load(out / "oracle0.npy")
    assert got.shape == oracle.shape and oracle.dtype == np.float64 and np.count_nonzero(oracle) > oracle.size // 2
    if name == "cand_cuda_gemm":
        rep = compare_outputs(round_to_format(oracle, "bf16"), got, oracle, "bf16")
        assert rep.passed, rep
    else:   # the layer requantises its intermediate: the reference's MoE bounds (test_kernels.py:94-102)
        scale = np.abs(oracle).max()
        assert np.abs(got - oracle).max() / scale < 1e-1 and np.sqrt(np.mean((got - oracle) ** 2)) / scale < 1e-2

    # CUPTI time per repetition against CUDA events around the same callable
    assert len(bundle.timings) == 30 and min(bundle.timings) > 0
    cupti_us = float(np.median(bundle.timings))
    m = importlib.import_module(entry)
    fn, args = m.build()
    event_us = _event_us(fn, args)
    # events around eager launches include the gaps between kernels: a lower bound on the CUPTI
    # figure only makes sense for the single-kernel module (the four-kernel layer is bound by the
    # host's launch rate when it is not replayed from a graph)
    print(f"{name}: CUPTI {cupti_us:.2f} us per repetition ({measure}), CUDA events {event_us:.2f} us")
    assert cupti_us <= event_us * 1.10, (cupti_us, event_us)
    if measure == "dominant":
        assert cupti_us >= event_us * 0.60, (cupti_us, event_us)
