"""Capture modules for Mosaicist's `capture` / `time` / `converge` commands.

Each module follows the candidate-module interface the reference's loop drives
(src/mosaicist/capture.py:9-21, experiments/loop/cand_pallas_gemm.py): `build()` returns
`(callable, args)`, `reference(*args)` returns the float64 oracle over the same inputs,
`KNOBS` / `STRUCTURAL` / `DEFAULTS` describe the search space.  Importing a module touches
neither CUDA nor the shared library (the loop's parent process imports it only to read
KNOBS, src/mosaicist/converge/loop.py:165-177).
"""
