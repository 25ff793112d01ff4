"""Stand-in for the `cupti-python` package where it is not installed: `from cupti import cupti`
gives the five activity calls the reference's tracer uses (src/mosaicist/bench/cupti_trace.py:51-80),
implemented over libcupti by `libmsc_cupti.so` (built from ../cupti_shim.cpp by
`python -m mosaicist_b200.build`).  Put this package's parent directory on sys.path to use it."""
