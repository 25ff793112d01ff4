"""The SM clock a GEMM really runs at, and its throughput against the peak at that clock.

NVML's sampled SM clock stays at the maximum while a power-capped GPU lowers the clock inside
a heavy kernel, so "fraction of the nominal peak" mixes kernel quality with power management.
The debug build of the library stamps every CTA with clock64 (SM cycles) and the global
nanosecond timer at the start and the end of its work; cycles / nanoseconds is the clock the
kernel saw.  The FP4 tensor peak at that clock is SMs x 16384 MAC/clk x 2 x clock (nominal:
9 PFLOP/s dense, i.e. 1.86 GHz on 148 SMs).

    python -m mosaicist_b200.clock_probe        # one JSON line per shape

The timed figure comes from the regular library (CUDA events, 30 launches); only the clock
comes from the debug build, which is slower and never timed.
"""

from __future__ import annotations

import ctypes
import json
import os
import subprocess
import sys

SHAPES = [(1, 8192, 8192, 8192), (8, 2048, 4096, 7168), (8, 512, 2048, 2048)]
MAC_PER_CLK_PER_SM_FP4 = 16384


def _operands(l, m, n, k, dev):
    import torch

    g = torch.Generator(device=dev).manual_seed(0)

    def u8(*shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=dev, generator=g)

    return (u8(l, m, k // 2), u8(l, m // 128, k // 64, 32, 16, lo=0x30, hi=0x40), u8(l, n, k // 2),
            u8(l, n // 128, k // 64, 32, 16, lo=0x30, hi=0x40),
            torch.empty((l, m, n), dtype=torch.bfloat16, device=dev))


def _clock_child():
    """Runs under the debug library: prints {shape: median SM MHz}."""
    import numpy as np
    import torch

    from . import _lib, ops

    lib = _lib.load()
    lib.msc_debug_config.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    res = {}
    for shape in SHAPES:
        a_q, a_sf, b_q, b_sf, out = _operands(*shape, dev)
        cfg = ops.GemmConfig(cta_pair=1)
        trace = torch.zeros(sms * 50 + sms * 32, dtype=torch.int64, device=dev)
        for _ in range(20):                               # reach the steady power state
            ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, None, None, cfg, out=out)
        lib.msc_debug_config(trace.data_ptr(), 0)
        for _ in range(5):                                # the last launch's stamps remain
            ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, None, None, cfg, out=out)
        torch.cuda.synchronize()
        lib.msc_debug_config(None, 0)
        t = trace.cpu().numpy()
        cyc = t[sms * 48: sms * 50].reshape(sms, 2)
        ns = t[sms * 50:].reshape(sms, 32)[:, 30:32]
        dc, dt = (cyc[:, 1] - cyc[:, 0]).astype(float), (ns[:, 1] - ns[:, 0]).astype(float)
        ok = (dt > 0) & (dc > 0)
        res["x".join(map(str, shape))] = float(np.median(dc[ok] / dt[ok] * 1e3))
    print("CLOCKS " + json.dumps(res), flush=True)


def main():
    if "--clock-child" in sys.argv:
        _clock_child()
        return
    import torch

    from . import _lib, build, ops

    debug_lib = build.build_debug()
    env = dict(os.environ, MSC_LIB_PATH=str(debug_lib))
    out = subprocess.run([sys.executable, "-m", "mosaicist_b200.clock_probe", "--clock-child"], env=env,
                         capture_output=True, text=True, check=True).stdout
    clocks = json.loads(next(ln for ln in out.splitlines() if ln.startswith("CLOCKS "))[7:])
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for shape in SHAPES:
        l, m, n, k = shape
        a_q, a_sf, b_q, b_sf, o = _operands(*shape, dev)
        plan = ops.masked_grouped_gemm_plan(a_q, a_sf, b_q, b_sf, None, None, ops.GemmConfig(cta_pair=1), out=o)
        for _ in range(10):
            plan()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(30):
            plan()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1e3 / 30
        tflops = 2.0 * l * m * n * k / us / 1e6
        mhz = clocks["x".join(map(str, shape))]
        peak = sms * MAC_PER_CLK_PER_SM_FP4 * 2 * mhz * 1e6 / 1e12
        print(json.dumps({"shape_l_m_n_k": shape, "us": us, "tflops": tflops, "sm_mhz_in_kernel": mhz,
                          "fp4_peak_at_that_clock_tflops": peak, "frac_of_peak_at_clock": tflops / peak,
                          "frac_of_nominal_9000": tflops / 9000.0}), flush=True)
    assert _lib.status_word() == 0


if __name__ == "__main__":
    main()
