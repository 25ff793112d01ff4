"""The profiling stage: the kernels of the library under Nsight Compute, summarised as
tensor-pipe utilisation and DRAM GB/s per kernel.

The reference pipeline has capture / time / converge stages and no profiling stage
(src/mosaicist/cli.py; its timing comes from CUPTI activity records,
src/mosaicist/bench/cupti_trace.py).  This stage fills that slot for the kernels of this library:

    python -m mosaicist_b200.profile_stage                       # launch list: every kernel's time
    python -m mosaicist_b200.profile_stage --kernel gemm_pair_kernel --json profiles/rows.jsonl
    python -m mosaicist_b200.profile_stage --in-kernel-clock     # SM clock inside the GEMM

Every mode first runs the workload once without the profiler (`--run`, this same module) and
stops unless it exits 0.  Then

* without `--kernel`: one `ncu --clock-control none --metrics gpu__time_duration.sum` pass over
  the library's kernels (a single-pass metric: nothing is replayed) -> launches, total and
  average time per kernel;
* with `--kernel NAME`: the named metrics (duration, DRAM bytes read / written, L2 -> SM bytes,
  DRAM and tensor-pipe utilisation, registers, active warps, ten warp-stall reasons) for that
  ONE kernel and at most `--launches` (default 3, never more than 5) launches of it, over the
  part of the workload that launches it (`--section`, chosen from the name when omitted).  The
  row is folded into `--json` (JSON lines keyed by kernel, the "machine" rows a capture
  bundle can carry) and the markdown table `--out` is rebuilt from all rows collected so far.

Each profiler run has a time limit (`--timeout`, default 600 s).  The workload is sized for
captures that end by themselves: operand sets of 0.1 - 1.5 GB (larger than L2, so DRAM figures
mean something).  Durations under the profiler are serialised and cold-cache; they rank
kernels and feed the GB/s column, they are not benchmark numbers.

`--in-kernel-clock` needs no profiler.  NVML's sampled SM clock stays at the maximum while a
power-capped GPU lowers the clock inside a heavy kernel, so "fraction of the nominal peak"
mixes kernel quality with power management.  The -DMSC_DEBUG build of the library
(`python -m mosaicist_b200.build --debug`) stamps every CTA with clock64 (SM cycles) and the
global nanosecond timer at the start and the end of its work; cycles / nanoseconds is the clock
the kernel saw, and SMs x 16384 MAC/clk x 2 x clock the FP4 tensor peak at that clock (nominal:
9 PFLOP/s dense, i.e. 1.86 GHz on 148 SMs).  The timed figure comes from the regular library
(CUDA events, 30 launches); only the clock comes from the debug build, which is never timed.
"""

from __future__ import annotations

import argparse
import csv
import io
import json
import os
import pathlib
import shutil
import subprocess
import sys
import tempfile

METRICS = [
    "gpu__time_duration.sum",
    "dram__bytes_read.sum",
    "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "launch__registers_per_thread",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "l1tex__m_xbar2l1tex_read_bytes.sum",
]
STALLS = ["long_scoreboard", "barrier", "wait", "short_scoreboard", "math_pipe_throttle", "mio_throttle",
          "lg_throttle", "sleeping", "membar", "branch_resolving"]
STALL_METRICS = [f"smsp__average_warps_issue_stalled_{name}_per_issue_active.ratio" for name in STALLS]
KERNEL_FILTER = "regex:gemm_|quantize|swizzle|moe_|ep_|route_|int4_|amax"
SECTIONS = ("gemm", "mxfp8", "dense", "int4", "quantize", "moe", "ep")
MAX_LAUNCHES = 5


def section_of(kernel: str) -> str:
    """The part of the workload that launches `kernel`."""
    for key, sec in (("dense_f16", "dense"), ("int4", "int4"), ("ep_", "ep"), ("moe_", "moe"), ("route_", "moe"),
                     ("quantize", "quantize"), ("swizzle", "quantize"), ("amax", "quantize"), ("gemm_", "gemm")):
        if key in kernel:
            return sec
    return "all"


def run_workload(section: str = "all"):
    """Launches the library's kernels on small representative cases; `section` limits the run
    to one family (SECTIONS)."""
    import numpy as np
    import torch

    from . import _lib, ops
    from .bench_moe import rand_weights
    from .moe import MegaMoE
    from .parallel import EXCHANGE_BUFFERS, PeerExpertParallelMoE, exchange_layout, exchange_views

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)

    def u8(*shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=dev, generator=g)

    want = lambda name: section in ("all", name)

    # NVFP4 grouped GEMM: the headline shape (pair, single-CTA 128- and 256-column tiles) and a
    # compute-bound shape
    for (l, m, n, k), cfgs in [((8, 512, 2048, 2048), [ops.GemmConfig(), ops.GemmConfig(tile_n=128),
                                                        ops.GemmConfig(tile_n=256)]),
                               ((1, 4096, 4096, 8192), [ops.GemmConfig()])]:
        if not want("gemm"):
            break
        a_q, b_q = u8(l, m, k // 2), u8(l, n, k // 2)
        a_sf = u8(l, m // 128, k // 64, 32, 16, lo=0x30, hi=0x40)
        b_sf = u8(l, n // 128, k // 64, 32, 16, lo=0x30, hi=0x40)
        for cfg in cfgs:
            ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, None, None, cfg)

    # NVFP4 over row-concatenated groups of 240 - 305 rows (a routed layer's experts): the
    # row-major pair kernel with short tiles, and the tokens-on-N kernel
    if want("gemm"):
        rows = [272, 240, 305, 256, 257, 250, 288, 264]
        pad = [(r + 127) // 128 * 128 for r in rows]
        offs = np.concatenate([[0], np.cumsum(pad)[:-1]]).astype(np.int32)
        tot, nn, kk = int(sum(pad)), 4096, 7168
        a_q, a_sf = u8(tot, kk // 2), u8(tot // 128, kk // 64, 32, 16, lo=0x30, hi=0x40)
        b_q, b_sf = u8(len(rows), nn, kk // 2), u8(len(rows), nn // 128, kk // 64, 32, 16, lo=0x30, hi=0x40)
        for pair in (1, 3):
            ops.ragged_grouped_gemm_nvfp4(a_q, a_sf, b_q, b_sf, torch.from_numpy(offs).to(dev),
                                          torch.tensor(rows, dtype=torch.int32, device=dev), None, None,
                                          ops.GemmConfig(cta_pair=pair))

    # MXFP8 grouped GEMM, ragged rows
    rows = [1024, 512, 256, 128, 640, 384, 896, 256]
    offs = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    tot, nn, kk = int(sum(rows)), 4096, 7168
    if want("mxfp8"):
        ops.ragged_grouped_gemm_mxfp8(u8(tot, kk) & 0x77, u8(tot // 128, kk // 128, 32, 16, lo=120, hi=130),
                                      u8(len(rows), nn, kk) & 0x77,
                                      u8(len(rows), nn // 128, kk // 128, 32, 16, lo=120, hi=130),
                                      torch.from_numpy(offs).to(dev),
                                      torch.tensor(rows, dtype=torch.int32, device=dev))

    # dense fp16 GEMM
    if want("dense"):
        a = torch.randn((4096, 4096), device=dev, generator=g).half()
        b = torch.randn((4096, 4096), device=dev, generator=g).half()
        ops.gemm_f16(a, b)

    # bf16 x int4 grouped GEMM (dequantise + bf16 grouped GEMM)
    rows = [256, 128, 384, 512, 128, 256, 256, 128]
    offs = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    tot, nn, kk = int(sum(rows)), 2048, 7168
    if want("int4"):
        x = torch.randn((tot, kk), device=dev, generator=g).bfloat16()
        sc = (torch.randn((len(rows), nn, kk // 128), device=dev, generator=g) * 0.02).abs().bfloat16()
        ops.mixed_grouped_gemm_int4(x, u8(len(rows), nn, kk // 2), sc, torch.from_numpy(offs).to(dev),
                                    torch.tensor(rows, dtype=torch.int32, device=dev))

    # quantiser, SiLU*up quantiser, scale swizzle
    if want("quantize"):
        h = torch.randn((8, 2048, 7168), device=dev, generator=g).bfloat16()
        gs = torch.full((8,), 448.0, dtype=torch.float32, device=dev)
        ops.quantize_nvfp4(h, gs)
        ops.silu_mul_quantize_nvfp4(h[:, :, :4096].contiguous(), gs)
        ops.to_mma_scale_layout(u8(8, 2048, 448))
        ops.global_scale_for(h)
        ops.quantize_mxfp8(h.view(-1, 7168))

    # routed MoE layer: route, plan, gather + quantise, fused GEMM1, GEMM2, combine; then the
    # unfused GEMM1 pair
    if not (want("moe") or want("ep")):
        torch.cuda.synchronize()
        if _lib.status_word() != 0:
            raise RuntimeError("a kernel reported an error status")
        return
    E, k, hid, inter, T = 64, 8, 7168, 2048, 4096
    w = rand_weights(E, inter, hid, dev, 3)
    gs_in = torch.full((E,), 2688.0 / 5.0, dtype=torch.float32, device=dev)
    gs_a2 = torch.full((E,), 2688.0 / 8.0, dtype=torch.float32, device=dev)
    tokens = torch.randn((T, hid), device=dev, generator=g).bfloat16()
    logits = torch.randn((T, E), device=dev, generator=g)
    layer = MegaMoE(*w, gs_in, gs_a2, topk=k, max_tokens=T)
    if want("moe"):
        layer.forward(tokens, logits)
        ops.quantize_nvfp4_ragged(layer.gateup, layer.a2_gs, layer.group_offsets, layer.group_rows, silu=True,
                                  out=(layer.d_q, layer.d_sf))

    # expert-parallel exchange kernels: two ranks' layers on this one device in lockstep, once
    # with the combine pulled from the owners' results and once pushed by the GEMM2 epilogue
    del layer
    world, el, T2 = 2, E // 2, T // 2
    rows_cap = (T2 * k + 127 * el + 127) // 128 * 128
    for push in ((False, True) if want("ep") else ()):
        pairs_cap = T2 // 2 * k if push else 0
        _, total = exchange_layout(rows_cap, hid, pairs_cap, world, E)
        spaces = [exchange_views(torch.zeros(total, dtype=torch.uint8, device=dev), rows_cap, hid, pairs_cap, world, E)
                  for _ in range(world)]
        ptrs = {nm: [s[nm].data_ptr() for s in spaces] for nm in EXCHANGE_BUFFERS}
        ranks = []
        for r in range(world):
            sl = slice(r * el, (r + 1) * el)
            inner = MegaMoE(*[t[sl] for t in w], gs_in[sl], gs_a2[sl], topk=1, max_tokens=1, expert_first=r * el,
                            rows_cap=rows_cap, workspace=spaces[r])
            extra = dict(row_dest=spaces[r]["row_dest"], recv_y=spaces[r]["recv_y"]) if push else {}
            ranks.append(PeerExpertParallelMoE(inner, ptrs, spaces[r]["sf_rows"], gs_in, E, k, T2 // 2, r, world,
                                               **extra))
        parts = [slice(0, T2 // 2), slice(T2 // 2, T2)]
        for ep, sl in zip(ranks, parts):
            ep.count(logits[sl].contiguous())
        counts_all = torch.stack([ep.counts for ep in ranks]).contiguous()
        for ep, sl in zip(ranks, parts):
            ep.place(counts_all)
            ep.dispatch(tokens[sl].contiguous())
        for ep in ranks:
            ep.experts()
        for ep in ranks:
            ep.combine()
        torch.cuda.synchronize()
        del ranks, spaces
    torch.cuda.synchronize()
    if _lib.status_word() != 0:
        raise RuntimeError("a kernel reported an error status")


def kernel_rows(csv_text: str) -> list[dict]:
    """ncu's --csv log (one row per launch and metric) -> one dict per kernel, slowest first."""
    lines = csv_text.splitlines()
    start = next(i for i, ln in enumerate(lines) if ln.startswith('"ID"'))
    per = {}   # kernel -> launch id -> metric -> value
    for row in csv.DictReader(io.StringIO("\n".join(lines[start:]))):
        name = row["Kernel Name"].split("(")[0]
        val = float(row["Metric Value"].replace(",", "")) if row["Metric Value"] not in ("", "n/a") else 0.0
        unit = row["Metric Unit"]
        if row["Metric Name"] == "gpu__time_duration.sum":
            val *= {"ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6}.get(unit, 1.0)          # -> us
        if "bytes" in row["Metric Name"]:
            val *= {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(unit, 1.0)  # -> bytes
        per.setdefault(name, {}).setdefault(row["ID"], {})[row["Metric Name"]] = val
    rows = []
    for name, launches in sorted(per.items(), key=lambda kv: -sum(m.get(METRICS[0], 0) for m in kv[1].values())):
        n = len(launches)
        avg = lambda key: sum(m.get(key, 0.0) for m in launches.values()) / n
        us, rd, wr = avg(METRICS[0]), avg(METRICS[1]), avg(METRICS[2])
        stalls = sorted(((avg(m), nm) for m, nm in zip(STALL_METRICS, STALLS)), reverse=True)
        rows.append({"kernel": name, "launches": n, "avg_us": us, "dram_read_bytes": rd, "dram_write_bytes": wr,
                     "dram_gbs": (rd + wr) / (us * 1e-6) / 1e9 if us > 0 else 0.0,
                     "dram_pct_of_peak": avg(METRICS[3]), "tensor_pipe_pct_of_peak": avg(METRICS[4]),
                     "registers_per_thread": avg(METRICS[5]), "warps_active_pct": avg(METRICS[6]),
                     "l2_to_sm_bytes": avg(METRICS[7]),
                     "top_stalls": [{"reason": nm, "warps_per_issue_active": v} for v, nm in stalls[:3] if v > 0]})
    return rows


def summarise(csv_text: str) -> str:
    """The per-kernel rows as a markdown table."""
    out = ["| kernel | launches | avg us | DRAM read MB | DRAM write MB | DRAM GB/s | DRAM % peak | tensor pipe % | regs | warps active % | L2->SM MB | top stalls (warps per issue-active cycle) |",
           "|---|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in kernel_rows(csv_text):
        stalls = ", ".join(f"{t['reason']} {t['warps_per_issue_active']:.1f}" for t in r["top_stalls"])
        out.append(f"| {r['kernel']} | {r['launches']} | {r['avg_us']:.1f} | {r['dram_read_bytes'] / 1e6:.2f} | "
                   f"{r['dram_write_bytes'] / 1e6:.2f} | {r['dram_gbs']:.0f} | {r['dram_pct_of_peak']:.1f} | "
                   f"{r['tensor_pipe_pct_of_peak']:.1f} | {r['registers_per_thread']:.0f} | {r['warps_active_pct']:.1f} | "
                   f"{r['l2_to_sm_bytes'] / 1e6:.1f} | {stalls} |")
    return "\n".join(out)


def launch_list(csv_text: str) -> str:
    """The single-metric pass as a markdown table: launches, total and average time, share."""
    rows = kernel_rows(csv_text)
    total = sum(r["avg_us"] * r["launches"] for r in rows) or 1.0
    out = ["| kernel | launches | total us | share | avg us |", "|---|---|---|---|---|"]
    for r in rows:
        t = r["avg_us"] * r["launches"]
        out.append(f"| {r['kernel']} | {r['launches']} | {t:.1f} | {100 * t / total:.1f} % | {r['avg_us']:.2f} |")
    return "\n".join(out)


def table_from_rows(rows: list[dict]) -> str:
    out = ["| kernel | launches | avg us | DRAM read MB | DRAM write MB | DRAM GB/s | DRAM % peak | tensor pipe % | regs | warps active % | L2->SM MB | top stalls (warps per issue-active cycle) |",
           "|---|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in sorted(rows, key=lambda r: -r["avg_us"]):
        stalls = ", ".join(f"{t['reason']} {t['warps_per_issue_active']:.1f}" for t in r["top_stalls"])
        out.append(f"| {r['kernel']} | {r['launches']} | {r['avg_us']:.1f} | {r['dram_read_bytes'] / 1e6:.2f} | "
                   f"{r['dram_write_bytes'] / 1e6:.2f} | {r['dram_gbs']:.0f} | {r['dram_pct_of_peak']:.1f} | "
                   f"{r['tensor_pipe_pct_of_peak']:.1f} | {r['registers_per_thread']:.0f} | {r['warps_active_pct']:.1f} | "
                   f"{r['l2_to_sm_bytes'] / 1e6:.1f} | {stalls} |")
    return "\n".join(out)


# ---- the SM clock inside the GEMM (--in-kernel-clock) ------------------------------------------
CLOCK_SHAPES = [(1, 8192, 8192, 8192), (8, 2048, 4096, 7168), (8, 512, 2048, 2048)]
MAC_PER_CLK_PER_SM_FP4 = 16384


def _clock_operands(l, m, n, k, dev):
    import torch

    g = torch.Generator(device=dev).manual_seed(0)

    def u8(*shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=dev, generator=g)

    return (u8(l, m, k // 2), u8(l, m // 128, k // 64, 32, 16, lo=0x30, hi=0x40), u8(l, n, k // 2),
            u8(l, n // 128, k // 64, 32, 16, lo=0x30, hi=0x40),
            torch.empty((l, m, n), dtype=torch.bfloat16, device=dev))


def _clock_child():
    """Runs under the debug library (MSC_LIB_PATH): prints {shape: median SM MHz inside the kernel}."""
    import ctypes

    import numpy as np
    import torch

    from . import _lib, ops

    lib = _lib.load()
    lib.msc_debug_config.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    res = {}
    for shape in CLOCK_SHAPES:
        a_q, a_sf, b_q, b_sf, out = _clock_operands(*shape, dev)
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


def in_kernel_clock():
    import torch

    from . import _lib, build, ops

    debug_lib = build.build_debug()
    env = dict(os.environ, MSC_LIB_PATH=str(debug_lib))
    out = subprocess.run([sys.executable, "-m", "mosaicist_b200.profile_stage", "--clock-child"], env=env,
                         capture_output=True, text=True, check=True, timeout=600).stdout
    clocks = json.loads(next(ln for ln in out.splitlines() if ln.startswith("CLOCKS "))[7:])
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for shape in CLOCK_SHAPES:
        l, m, n, k = shape
        a_q, a_sf, b_q, b_sf, o = _clock_operands(*shape, dev)
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


def _trace_child():
    """Runs under MSC_LIB_PATH = the debug build: per-tile clock stamps of the row-major pair
    kernel and the tokens-on-N kernel on expert-shaped groups (64 groups of 256 or 272 rows,
    plain epilogue).  One JSON line per (shape, rows, kernel) with the median CTA body and, for
    the third and fourth tile of CTA 0, the K loop, the time the epilogue holds the accumulator
    and the epilogue as a whole, all in SM cycles."""
    import ctypes

    import numpy as np
    import torch

    from . import _lib, ops

    lib = _lib.load()
    lib.msc_debug_config.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)

    def u8(*shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=dev, generator=g)

    ncta = torch.cuda.get_device_properties(0).multi_processor_count
    trace = torch.zeros(ncta * 50 + ncta * 32, dtype=torch.int64, device=dev)
    E = 64
    for nn, kk in ((4096, 7168), (7168, 2048)):
        b_q, b_sf = u8(E, nn, kk // 2), u8(E, nn // 128, kk // 64, 32, 16, lo=0x30, hi=0x40)
        for rows_each in (256, 272):
            pad = (rows_each + 127) // 128 * 128
            tot = E * pad
            a_q, a_sf = u8(tot, kk // 2), u8(tot // 128, kk // 64, 32, 16, lo=0x30, hi=0x40)
            offs = torch.arange(E, dtype=torch.int32, device=dev) * pad
            rows = torch.full((E,), rows_each, dtype=torch.int32, device=dev)
            out = torch.empty((tot, nn), dtype=torch.bfloat16, device=dev)
            for pair, name in ((1, "row-major pair"), (3, "tokens on N")):
                cfg = ops.GemmConfig(cta_pair=pair)

                def run():
                    ops.ragged_grouped_gemm_nvfp4(a_q, a_sf, b_q, b_sf, offs, rows, None, None, cfg, out=out)

                lib.msc_debug_config(None, 0)
                run(), run()
                torch.cuda.synchronize()
                trace.zero_()
                lib.msc_debug_config(trace.data_ptr(), 0)
                run()
                torch.cuda.synchronize()
                lib.msc_debug_config(None, 0)
                t = trace.cpu().numpy()
                tiles, ends = t[:ncta * 48].reshape(ncta, 8, 3, 2), t[ncta * 48:ncta * 50].reshape(ncta, 2)
                body = ends[:, 1] - ends[:, 0]
                rec = {"n": nn, "k": kk, "rows_per_group": rows_each, "kernel": name,
                       "cta_body_cycles_median": int(np.median(body)), "tiles": []}
                for tl in (2, 3):
                    r = tiles[0, tl]
                    if r[1, 0] == 0:
                        break
                    rec["tiles"].append({"k_loop": int(r[1, 1] - r[1, 0]), "accumulator_held": int(r[2, 1] - r[2, 0]),
                                         "epilogue": int(r[0, 1] - r[2, 0]) if pair == 3 else None})
                print("TRACE " + json.dumps(rec), flush=True)
            del a_q, a_sf, out
    assert _lib.status_word() == 0


def tile_trace():
    from . import build

    debug_lib = build.build_debug()
    env = dict(os.environ, MSC_LIB_PATH=str(debug_lib))
    out = subprocess.run([sys.executable, "-m", "mosaicist_b200.profile_stage", "--trace-child"], env=env,
                         capture_output=True, text=True, check=True, timeout=600).stdout
    recs = [json.loads(ln[6:]) for ln in out.splitlines() if ln.startswith("TRACE ")]
    print("| n | k | rows per group | kernel | CTA body, median (cycles) | K loop of a tile | accumulator held by the epilogue | whole epilogue |")
    print("|---|---|---|---|---|---|---|---|")
    for r in recs:
        tl = r["tiles"][-1] if r["tiles"] else {"k_loop": None, "accumulator_held": None, "epilogue": None}
        print(f"| {r['n']} | {r['k']} | {r['rows_per_group']} | {r['kernel']} | {r['cta_body_cycles_median']} | "
              f"{tl['k_loop']} | {tl['accumulator_held']} | {tl['epilogue'] if tl['epilogue'] is not None else '-'} |")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", action="store_true", help="only launch the workload (what gets profiled)")
    ap.add_argument("--section", default=None, choices=SECTIONS + ("all",),
                    help="part of the workload to run (default: all, or the one --kernel belongs to)")
    ap.add_argument("--kernel", default=None,
                    help="capture the named metrics for this one kernel (substring of its name)")
    ap.add_argument("--launches", type=int, default=3, help=f"launches of --kernel to capture (at most {MAX_LAUNCHES})")
    ap.add_argument("--out", default=None, help="markdown file to write (default: print only)")
    ap.add_argument("--json", default=None,
                    help="JSON-lines file of per-kernel rows: this call's row replaces the one of the same kernel")
    ap.add_argument("--csv", default=None, help="summarise an existing ncu CSV log instead of profiling")
    ap.add_argument("--raw", default=str(pathlib.Path(tempfile.gettempdir()) / "profile_stage.csv"),
                    help="where ncu's CSV log goes")
    ap.add_argument("--timeout", type=int, default=600, help="seconds each run may take")
    ap.add_argument("--in-kernel-clock", action="store_true", help="SM clock inside the GEMM (debug build, no profiler)")
    ap.add_argument("--clock-child", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--tile-trace", action="store_true",
                    help="per-tile clock stamps of the pair and tokens-on-N kernels (debug build, no profiler)")
    ap.add_argument("--trace-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.clock_child:
        _clock_child()
        return
    if args.trace_child:
        _trace_child()
        return
    if args.tile_trace:
        tile_trace()
        return
    if args.in_kernel_clock:
        in_kernel_clock()
        return
    section = args.section or (section_of(args.kernel) if args.kernel else "all")
    if args.run:
        run_workload(section)
        return
    cmd = [sys.executable, "-m", "mosaicist_b200.profile_stage", "--run", "--section", section]
    if args.kernel:
        launches = max(1, min(args.launches, MAX_LAUNCHES))
        ncu_cmd = ["ncu", "--clock-control", "none", "--metrics", ",".join(METRICS + STALL_METRICS),
                   "-k", f"regex:{args.kernel}", "-c", str(launches)]
    else:
        ncu_cmd = ["ncu", "--clock-control", "none", "--metrics", METRICS[0], "-k", KERNEL_FILTER, "-c", "400"]
    ncu_cmd += ["--print-units", "base", "--csv", "--log-file", args.raw, *cmd]
    if args.csv is None:
        if shutil.which("ncu") is None:
            raise SystemExit("ncu is not on PATH")
        subprocess.run(cmd, check=True, timeout=args.timeout)   # must exit 0 before anything is profiled
        pathlib.Path(args.raw).parent.mkdir(parents=True, exist_ok=True)
        subprocess.run(ncu_cmd, check=True, timeout=args.timeout)
        text = pathlib.Path(args.raw).read_text()
    else:
        text = pathlib.Path(args.csv).read_text()
    shown = " ".join(ncu_cmd[:-len(cmd)]).replace(args.raw, "<log>") + " " + " ".join(["python", *cmd[1:]])
    if not args.kernel:
        body = ("# Launch list of the library's kernels, small cases\n\n"
                "Made by `python -m mosaicist_b200.profile_stage` (plain run first, then\n`" + shown + "`).\n"
                "Times are under the profiler (serialised, cold caches): compare shares, not absolutes.\n\n"
                + launch_list(text) + "\n")
    else:
        rows = kernel_rows(text)
        merged = {}
        if args.json and pathlib.Path(args.json).exists():
            for ln in pathlib.Path(args.json).read_text().splitlines():
                if ln.strip():
                    r = json.loads(ln)
                    merged[r["kernel"]] = r
        for r in rows:
            merged[r["kernel"]] = r
        if args.json:
            pathlib.Path(args.json).write_text("".join(json.dumps(r) + "\n" for r in merged.values()))
        body = ("# Kernels of the library under Nsight Compute, small cases\n\n"
                "Made by `python -m mosaicist_b200.profile_stage --kernel <name>`, one kernel per call (plain run\n"
                "first, then e.g. `" + shown + "`).\n"
                "Durations are under the profiler (serialised, cold caches): use them to rank kernels and for\n"
                "the GB/s column, not as benchmark numbers.  DRAM GB/s = (read + write bytes) / duration.\n\n"
                + table_from_rows(list(merged.values())) + "\n")
    if args.out:
        pathlib.Path(args.out).write_text(body)
    print(body)


if __name__ == "__main__":
    main()
