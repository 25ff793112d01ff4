"""The capture modules end to end on a GPU: build() runs, leaves a PTX in the dump
directory, and the result passes the numerics gate against the module's own reference()."""

import numpy as np
import pytest

from oracle import gate, nvfp4 as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,knobs", [("cand_cuda_gemm", {}), ("cand_cuda_gemm", {"cta_pair": 2, "tile_n": 128}),
                                        ("cand_cuda_moe", {})])
def test_capture_module(name, knobs, tmp_path, monkeypatch):
    import importlib
    import json

    import torch

    from mosaicist_b200 import _lib

    monkeypatch.setenv("MOSAIC_GPU_DUMP_TO", str(tmp_path))
    monkeypatch.setenv("MOSAICIST_KNOBS", json.dumps(knobs))
    m = importlib.import_module(f"mosaicist_b200.candidates.{name}")
    fn, args = m.build()
    out = fn(*args)
    torch.cuda.synchronize()
    assert _lib.status_word() == 0
    assert list(tmp_path.rglob("*.ptx")), "no PTX left for collect_artifacts"
    got = out.float().cpu().numpy()
    ref = m.reference(*args)
    ok, worst = O.tolerance_ok(got, ref)
    assert ok, worst
    assert gate.gate_bf16(got, ref).passed
    assert np.count_nonzero(ref) > ref.size // 2
