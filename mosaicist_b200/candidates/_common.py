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


def only_entry(ptx_text: str, needle: str) -> str:
    """The PTX module reduced to the one `.entry` whose mangled name contains `needle` (the
    preamble, module-scope declarations and every non-entry function are kept); the text
    unchanged if no entry matches.  The fingerprinter looks at the entry with the most
    instructions, which in a translation unit full of template instantiations is rarely the one
    that ran."""
    import re

    heads = list(re.finditer(r"^(?:\.visible |\.weak )?\.entry\s+(\S+?)\(", ptx_text, re.M))
    if not any(needle in h.group(1) for h in heads):
        return ptx_text
    out, pos = [], 0
    for h in heads:
        depth, i = 0, ptx_text.index("{", h.end())
        while True:                                   # the entry's body: match its braces
            ch = ptx_text[i]
            depth += ch == "{"
            depth -= ch == "}"
            i += 1
            if depth == 0:
                break
        out.append(ptx_text[pos:h.start()])
        if needle in h.group(1):
            out.append(ptx_text[h.start():i])
        pos = i
    out.append(ptx_text[pos:])
    return "".join(out)


def drop_artifacts(kernel: str = "pair", entry: str | None = None) -> None:
    """Copies the PTX text of the kernel that will run and the ptxas log into the capture's dump
    directory, where collect_artifacts looks for `*.ptx` and a ptxas-named log
    (capture.py:81-116).  Without a PTX the loop cannot fingerprint the bundle
    (src/mosaicist/bundle.py:52-55), and it fingerprints the entry with the most instructions
    (src/mosaicist/ptx/parse.py:123-146), so only the translation unit of the running kernel is
    dropped: "pair" (CTA-pair block-scaled GEMM, the default), "single" (one CTA per tile) or
    "dense" (16-bit and int4-weight GEMMs) - reduced to the instantiation whose mangled name
    contains `entry` when that is given (see only_entry)."""
    dump = os.environ.get(DUMP_VAR)
    if not dump:
        return
    from .. import _lib

    dst = pathlib.Path(dump)
    dst.mkdir(parents=True, exist_ok=True)
    base = pathlib.Path(_lib.load().msc_ptx_path().decode())
    ptx = base if kernel == "pair" else base.with_suffix(f".{kernel}.ptx")
    if ptx.exists():
        text = ptx.read_text()
        (dst / f"mosaicist_sm100a_{kernel}_gemm.ptx").write_text(only_entry(text, entry) if entry else text)
    log = base.with_suffix(".ptxas.log")
    if log.exists():
        shutil.copy(log, dst / "ptxas_mosaicist_sm100a.log")
