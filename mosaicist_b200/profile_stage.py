"""The profiling stage: every kernel of the library once under Nsight Compute, summarised as
tensor-pipe utilisation and DRAM GB/s per kernel.

The reference pipeline has capture / time / converge stages and no profiling stage
(src/mosaicist/cli.py; its timing comes from CUPTI activity records,
src/mosaicist/backends/cuda.py).  This stage fills that slot for the kernels of this library:

    python -m mosaicist_b200.profile_stage --out profiles/kernels_small_cases.md

1. runs the workload once without the profiler (`--run`, this same module) and stops unless it
   exits 0;
2. runs it again under `ncu --clock-control none` with named metrics (duration, DRAM bytes
   read / written, L2 -> SM bytes, DRAM and tensor-pipe utilisation, registers, active warps,
   ten warp-stall reasons), limited to this library's kernels and `--launches` launches;
3. folds the CSV into one row per kernel: launches, average duration, DRAM GB/s (bytes /
   duration), DRAM % of peak, tensor pipe % of peak, registers per thread, the three largest
   stall reasons (warps stalled per issue-active cycle) - as a markdown table and, with
   `--json`, as one JSON object per kernel (the "machine" rows a capture bundle can carry).

The workload is sized for a capture that ends by itself within a couple of minutes: operand
sets of 0.1 - 1.5 GB (larger than L2, so DRAM figures mean something), one to three launches per
kernel.  Durations under the profiler are serialised and cold-cache; they rank kernels and
feed the GB/s column, they are not benchmark numbers.
"""

from __future__ import annotations

import argparse
import csv
import io
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
KERNEL_FILTER = "regex:gemm_|quantize|swizzle|moe_|ep_|route_|int4_"


def run_workload():
    """Launches every kernel of the library on a small representative case."""
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

    # NVFP4 grouped GEMM: the headline shape (pair, single-CTA 128- and 256-column tiles) and a
    # compute-bound shape
    for (l, m, n, k), cfgs in [((8, 512, 2048, 2048), [ops.GemmConfig(), ops.GemmConfig(tile_n=128),
                                                        ops.GemmConfig(tile_n=256)]),
                               ((1, 4096, 4096, 8192), [ops.GemmConfig()])]:
        a_q, b_q = u8(l, m, k // 2), u8(l, n, k // 2)
        a_sf = u8(l, m // 128, k // 64, 32, 16, lo=0x30, hi=0x40)
        b_sf = u8(l, n // 128, k // 64, 32, 16, lo=0x30, hi=0x40)
        for cfg in cfgs:
            ops.masked_grouped_gemm(a_q, a_sf, b_q, b_sf, None, None, cfg)

    # MXFP8 grouped GEMM, ragged rows
    rows = [1024, 512, 256, 128, 640, 384, 896, 256]
    offs = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    tot, nn, kk = int(sum(rows)), 4096, 7168
    ops.ragged_grouped_gemm_mxfp8(u8(tot, kk) & 0x77, u8(tot // 128, kk // 128, 32, 16, lo=120, hi=130),
                                  u8(len(rows), nn, kk) & 0x77,
                                  u8(len(rows), nn // 128, kk // 128, 32, 16, lo=120, hi=130),
                                  torch.from_numpy(offs).to(dev), torch.tensor(rows, dtype=torch.int32, device=dev))

    # dense fp16 GEMM
    a = torch.randn((4096, 4096), device=dev, generator=g).half()
    b = torch.randn((4096, 4096), device=dev, generator=g).half()
    ops.gemm_f16(a, b)

    # bf16 x int4 grouped GEMM (dequantise + bf16 grouped GEMM)
    rows = [256, 128, 384, 512, 128, 256, 256, 128]
    offs = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    tot, nn, kk = int(sum(rows)), 2048, 7168
    x = torch.randn((tot, kk), device=dev, generator=g).bfloat16()
    sc = (torch.randn((len(rows), nn, kk // 128), device=dev, generator=g) * 0.02).abs().bfloat16()
    ops.mixed_grouped_gemm_int4(x, u8(len(rows), nn, kk // 2), sc, torch.from_numpy(offs).to(dev),
                                torch.tensor(rows, dtype=torch.int32, device=dev))

    # quantiser, SiLU*up quantiser, scale swizzle
    h = torch.randn((8, 2048, 7168), device=dev, generator=g).bfloat16()
    gs = torch.full((8,), 448.0, dtype=torch.float32, device=dev)
    ops.quantize_nvfp4(h, gs)
    ops.silu_mul_quantize_nvfp4(h[:, :, :4096].contiguous(), gs)
    ops.to_mma_scale_layout(u8(8, 2048, 448))

    # routed MoE layer: route, plan, gather + quantise, fused GEMM1, GEMM2, combine; then the
    # unfused GEMM1 pair
    E, k, hid, inter, T = 64, 8, 7168, 2048, 4096
    w = rand_weights(E, inter, hid, dev, 3)
    gs_in = torch.full((E,), 2688.0 / 5.0, dtype=torch.float32, device=dev)
    gs_a2 = torch.full((E,), 2688.0 / 8.0, dtype=torch.float32, device=dev)
    tokens = torch.randn((T, hid), device=dev, generator=g).bfloat16()
    logits = torch.randn((T, E), device=dev, generator=g)
    layer = MegaMoE(*w, gs_in, gs_a2, topk=k, max_tokens=T)
    layer.forward(tokens, logits)
    ops.quantize_nvfp4_ragged(layer.gateup, layer.a2_gs, layer.group_offsets, layer.group_rows, silu=True,
                              out=(layer.d_q, layer.d_sf))

    # expert-parallel exchange kernels: two ranks' layers on this one device in lockstep, once
    # with the combine pulled from the owners' results and once pushed by the GEMM2 epilogue
    del layer
    world, el, T2 = 2, E // 2, T // 2
    rows_cap = (T2 * k + 127 * el + 127) // 128 * 128
    for push in (False, True):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", action="store_true", help="only launch the workload (what gets profiled)")
    ap.add_argument("--out", default="profiles/kernels_small_cases.md")
    ap.add_argument("--launches", type=int, default=80)
    ap.add_argument("--json", default=None, help="also write the per-kernel rows as JSON lines to this file")
    ap.add_argument("--csv", default=None, help="summarise an existing ncu CSV log instead of profiling")
    ap.add_argument("--raw", default=str(pathlib.Path(tempfile.gettempdir()) / "profile_stage.csv"),
                    help="where ncu's CSV log goes")
    args = ap.parse_args()
    if args.run:
        run_workload()
        return
    cmd = [sys.executable, "-m", "mosaicist_b200.profile_stage", "--run"]
    ncu_cmd = ["ncu", "--clock-control", "none", "--metrics", ",".join(METRICS + STALL_METRICS), "-k", KERNEL_FILTER,
               "-c", str(args.launches), "--print-units", "base", "--csv", "--log-file", args.raw, *cmd]
    if args.csv is None:
        if shutil.which("ncu") is None:
            raise SystemExit("ncu is not on PATH")
        subprocess.run(cmd, check=True)                  # must exit 0 before anything is profiled
        pathlib.Path(args.raw).parent.mkdir(parents=True, exist_ok=True)
        subprocess.run(ncu_cmd, check=True)
        text = pathlib.Path(args.raw).read_text()
    else:
        text = pathlib.Path(args.csv).read_text()
    table = summarise(text)
    if args.json:
        import json

        pathlib.Path(args.json).write_text("".join(json.dumps(r) + "\n" for r in kernel_rows(text)))
    body = ("# Every kernel of the library under Nsight Compute, small cases\n\n"
            "Made by `python -m mosaicist_b200.profile_stage` (plain run first, then\n`"
            + " ".join(ncu_cmd[:-len(cmd)]) + " <same command>`).\n"
            "Durations are under the profiler (serialised, cold caches): use them to rank kernels and for\n"
            "the GB/s column, not as benchmark numbers.  DRAM GB/s = (read + write bytes) / duration.\n\n"
            + table + "\n")
    pathlib.Path(args.out).write_text(body)
    print(body)


if __name__ == "__main__":
    main()
