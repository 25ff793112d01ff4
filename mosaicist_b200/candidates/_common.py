"""Plumbing shared by the capture modules."""

from __future__ import annotations

import json
import os
import pathlib
import shutil

ENV_VAR = "MOSAICIST_KNOBS"          # src/mosaicist/converge/knobs.py:21
DUMP_VAR = "MOSAIC_GPU_DUMP_TO"      # src/mosaicist/capture.py:41-47


def from_env(defaults: dict | None = None) -> dict:
    """The knob setting for this capture: JSON in $MOSAICIST_KNOBS merged over `defaults`
    (same contract as mosaicist.converge.knobs.from_env, knobs.py:25-36)."""
    out = dict(defaults or {})
    raw = os.environ.get(ENV_VAR)
    if raw:
        out.update(json.loads(raw))
    return out


def drop_artifacts() -> None:
    """Copies the library's PTX text and ptxas log into the capture's dump directory, where
    collect_artifacts looks for `*.ptx` and a ptxas-named log (capture.py:81-116).  Without a
    PTX the loop cannot fingerprint the bundle (src/mosaicist/bundle.py:52-55)."""
    dump = os.environ.get(DUMP_VAR)
    if not dump:
        return
    from .. import _lib

    dst = pathlib.Path(dump)
    dst.mkdir(parents=True, exist_ok=True)
    ptx = pathlib.Path(_lib.load().msc_ptx_path().decode())
    if ptx.exists():
        shutil.copy(ptx, dst / "mosaicist_sm100a_gemm.ptx")
    log = ptx.with_suffix(".ptxas.log")
    if log.exists():
        shutil.copy(log, dst / "ptxas_mosaicist_sm100a.log")
