"""Stages the reference project's own Python package for tests that drive this library through it.

    python oracle/stage_reference.py /path/to/reference      # or MOSAICIST_REFERENCE=/path/...

Copies `<reference>/src/mosaicist` (pure Python: capture, verify, ptx, converge ...) to
`oracle/_ref/mosaicist`.  `oracle/_ref/` is git-ignored: nothing of the reference enters this
repository's history; the staged copy only travels with a working tree to the machine that runs
the GPU tests, where the reference checkout itself is not mounted.  Tests that need it
(`tests/test_capture_gpu.py`, two checks in `tests/test_abi.py`) skip when it is absent.

TEST INFRASTRUCTURE ONLY: nothing in `mosaicist_b200/` or `bench.py` imports the staged package.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import sys

HERE = pathlib.Path(__file__).resolve().parent
STAGED = HERE / "_ref"


def stage(reference_root: str | os.PathLike | None = None) -> pathlib.Path | None:
    """Copies the package if the reference is there; returns the directory to put on sys.path
    (the one holding `mosaicist/`), or None when there is neither a reference nor a staged copy."""
    root = reference_root or os.environ.get("MOSAICIST_REFERENCE")
    src = pathlib.Path(root) / "src" / "mosaicist" if root else None
    if src is not None and src.is_dir():
        dst = STAGED / "mosaicist"
        if dst.exists():
            shutil.rmtree(dst)
        shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return STAGED if (STAGED / "mosaicist" / "__init__.py").exists() else None


def staged_path() -> pathlib.Path | None:
    """Where the reference's package can be imported from: $MOSAICIST_REFERENCE/src if set and
    present, else the staged copy, else None."""
    root = os.environ.get("MOSAICIST_REFERENCE")
    if root and (pathlib.Path(root) / "src" / "mosaicist").is_dir():
        return pathlib.Path(root) / "src"
    return STAGED if (STAGED / "mosaicist" / "__init__.py").exists() else None


if __name__ == "__main__":
    where = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print("staged at", where) if where else sys.exit("no reference checkout given and nothing staged")
