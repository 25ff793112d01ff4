"""Times the other benchmark configurations on one GPU (the headline NVFP4 grouped GEMM has
its own bench.py at the repository root, the MoE layer bench_moe.py):

  C2  dense fp16 GEMM 8192^3 (also N-sharded: each of `--gpus` ranks takes 8192/N columns)
  C3  MXFP8 grouped GEMM, 32 groups with Zipf(1.2) row counts summing to 16384, n=4096, k=7168
  C4  bf16 x int4 grouped GEMM, 64 groups with m ~ U[64, 512], n=2048, k=7168, group size 128

  C1x the headline NVFP4 grouped GEMM against FlashInfer's CuTeDSL kernel on the same operand
      bytes (`--vs-flashinfer`; needs the third-party flashinfer + nvidia-cutlass-dsl packages)

    python -m mosaicist_b200.bench_configs [--reps 20] [--vs-flashinfer]

Inputs are seeded synthetic data of those shapes; every timed launch is preceded by an L2
flush (a 256 MB memset) outside the CUDA-event window.  One JSON line per configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib

import numpy as np
import torch


def _time(fn, reps, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def _time_graph(fn, launches=20, reps=15):
    """us per launch of `launches` back-to-back calls replayed from one CUDA graph (operands
    stay L2-resident: the warm figure, free of host launch cost for either implementation)."""
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            fn()
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for _ in range(launches):
                fn()
        ts = []
        for _ in range(reps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
            graph.replay()
            e.record(st)
            st.synchronize()
            ts.append(s.elapsed_time(e) * 1e3 / launches)
    ts.sort()
    return ts[len(ts) // 2]


def headline_vs_flashinfer(reps):
    from .candidates import cand_cuda_gemm as cand, ref_flashinfer_gemm as ref

    ours, a1 = cand.build()
    theirs, a2 = ref.build()
    y_ref = theirs(*a2).clone()
    y = ours(*a1)
    torch.cuda.synchronize()
    fl = 2.0 * cand.L * cand.M * cand.N * cand.K
    us_ours, us_ref = _time_graph(lambda: ours(*a1), reps=reps), _time_graph(lambda: theirs(*a2), reps=reps)
    return {"config": "C1 NVFP4 masked grouped GEMM l=8 m=512 n=2048 k=2048, same operand bytes, warm, graph of 20",
            "us": us_ours, "tflops": fl / us_ours / 1e6, "flashinfer_us": us_ref,
            "flashinfer_tflops": fl / us_ref / 1e6,
            "bitwise_equal_fraction": float((y == y_ref).float().mean())}


def masked_moe_path(reps):
    """The masked MoE path at the shape the reference times end to end (l=8 experts, m=512 rows,
    k=2048 hidden, n=1024 intermediate: quantise, GEMM1 + SiLU*up + quantise, GEMM2), warm, as
    the reference times it (sum of kernel times, L2 warm): here one CUDA graph of 20 layers."""
    from . import ops
    from .candidates import cand_cuda_moe as cand
    from .moe import moe_masked

    from .moe import fold_alphas

    args = cand._inputs()
    (hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, masked_m, in_gs, a2_gs) = args
    folded = fold_alphas(w1_gs, w1_alpha, w2_gs, w2_alpha, in_gs, a2_gs)
    us_layer = _time_graph(lambda: moe_masked(*args, folded_alphas=folded), reps=reps)
    us_fused = _time_graph(lambda: moe_masked(*args, folded_alphas=folded, fuse_gemm1=True), reps=reps)
    # the four kernels one by one, for the sum the reference quotes
    a_q, a_sf = ops.quantize_nvfp4(hidden, in_gs, masked_m)
    gateup = ops.masked_grouped_gemm(a_q, a_sf, w1_q, w1_sf, folded[0], masked_m)
    d_q, d_sf = ops.silu_mul_quantize_nvfp4(gateup, a2_gs, masked_m)
    y = torch.empty_like(hidden)
    parts = {
        "quantize": _time_graph(lambda: ops.quantize_nvfp4(hidden, in_gs, masked_m), reps=reps),
        "gemm1": _time_graph(lambda: ops.masked_grouped_gemm(a_q, a_sf, w1_q, w1_sf, folded[0], masked_m, out=gateup),
                             reps=reps),
        "silu_mul_quantize": _time_graph(lambda: ops.silu_mul_quantize_nvfp4(gateup, a2_gs, masked_m), reps=reps),
        "gemm2": _time_graph(lambda: ops.masked_grouped_gemm(d_q, d_sf, w2_q, w2_sf, folded[1], masked_m, out=y),
                             reps=reps),
    }
    fl = 2.0 * cand.L * cand.M * (cand.K * 2 * cand.N + cand.N * cand.K)
    return {"config": "masked MoE path l=8 m=512 k=2048 n=1024 (quantise, GEMM1, SiLU*up+quantise, GEMM2), warm",
            "us_layer_graph_of_20": us_layer, "tflops": fl / us_layer / 1e6, "us_sum_of_kernels": sum(parts.values()),
            "us_per_kernel": parts, "us_layer_with_fused_gemm1": us_fused,
            "reference_flashinfer_us_sum_of_kernels": 46.0,
            "reference_per_kernel_us": {"quantize": 10.9, "gemm1": 13.4, "silu_mul_quantize": 8.7, "gemm2": 9.4},
            "reference_pallas_port_us": 60.8}


def _layout(rows):
    offs, tot = [], 0
    for r in rows:
        offs.append(tot)
        tot += (r + 127) // 128 * 128
    return offs, tot


def zipf_rows(groups=32, total=16384, s=1.2):
    w = 1.0 / np.arange(1, groups + 1) ** s
    rows = np.maximum(1, np.floor(w / w.sum() * total)).astype(int)
    rows[0] += total - rows.sum()
    return rows.tolist()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--vs-flashinfer", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    out = measure(args.reps, rank, world, args.vs_flashinfer)
    if rank == 0:
        for line in out:
            print(json.dumps(line), flush=True)


def measure(reps: int, rank: int = 0, world: int = 1, vs_flashinfer: bool = False, masked_moe: bool = True) -> list:
    """Times the configurations on the current device; returns one record per configuration."""
    import types

    from . import _lib, ops

    args = types.SimpleNamespace(reps=reps, vs_flashinfer=vs_flashinfer)
    dev = torch.device("cuda", torch.cuda.current_device())
    pk = pathlib.Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    bf16_peak = json.loads(pk.read_text())["bf16_tflops"] if pk.exists() else 1590.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(rank)
    out = []
    if args.vs_flashinfer and rank == 0:
        out.append(headline_vs_flashinfer(args.reps))
    if rank == 0 and masked_moe:
        out.append(masked_moe_path(args.reps))

    # C2: dense fp16, this rank's column shard
    n = 8192
    from .parallel import column_range
    cols = column_range(n, world, rank)
    a = (torch.randn((n, n), device=dev, generator=g) / n ** 0.5).half()
    b = (torch.randn((n, n), device=dev, generator=g) / n ** 0.5).half()
    c = torch.empty((n, n), dtype=torch.float16, device=dev)
    bs, cs = b[:, cols.start:cols.stop], c[:, cols.start:cols.stop]
    ms = _time(lambda: ops.gemm_f16(a, bs, out=cs), args.reps, flush)
    ms_lib = _time(lambda: torch.matmul(a, bs, out=cs), args.reps, flush)
    fl = 2.0 * n * n * len(cols)
    out.append({"config": "C2 dense fp16 8192^3", "columns_per_rank": len(cols), "ms": ms,
                "tflops": fl / ms / 1e9, "pct_measured_bf16_peak": 100 * fl / ms / 1e9 / bf16_peak,
                "cublas_ms": ms_lib, "cublas_tflops": fl / ms_lib / 1e9})
    del a, b, c

    # C3: MXFP8 grouped, ragged rows
    rows = zipf_rows()
    offs, tot = _layout(rows)
    nn, kk = 4096, 7168
    a_q = torch.randint(0, 256, (tot, kk), dtype=torch.uint8, device=dev, generator=g) & 0x77      # finite e4m3
    b_q = torch.randint(0, 256, (len(rows), nn, kk), dtype=torch.uint8, device=dev, generator=g) & 0x77
    a_sf = torch.randint(120, 130, (tot // 128, kk // 128, 32, 16), dtype=torch.uint8, device=dev, generator=g)
    b_sf = torch.randint(120, 130, (len(rows), nn // 128, kk // 128, 32, 16), dtype=torch.uint8, device=dev, generator=g)
    o_t = torch.tensor(offs, dtype=torch.int32, device=dev)
    r_t = torch.tensor(rows, dtype=torch.int32, device=dev)
    y = torch.empty((tot, nn), dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: ops.ragged_grouped_gemm_mxfp8(a_q, a_sf, b_q, b_sf, o_t, r_t, out=y), args.reps, flush)
    fl = 2.0 * sum(rows) * nn * kk
    out.append({"config": "C3 MXFP8 grouped 32 groups Zipf(1.2) sum 16384, n=4096 k=7168", "rows": rows,
                "ms": ms, "tflops": fl / ms / 1e9, "pct_2x_measured_bf16_peak": 100 * fl / ms / 1e9 / (2 * bf16_peak),
                "pct_nominal_fp8_4500": 100 * fl / ms / 1e9 / 4500})
    del a_q, b_q, a_sf, b_sf, y

    # C4: bf16 x int4 grouped
    rng = np.random.default_rng(4)
    rows = rng.integers(64, 513, 64).tolist()
    offs, tot = _layout(rows)
    nn, kk = 2048, 7168
    a = torch.randn((tot, kk), device=dev, generator=g).bfloat16()
    bq = torch.randint(0, 256, (64, nn, kk // 2), dtype=torch.uint8, device=dev, generator=g)
    sc = (torch.randn((64, nn, kk // 128), device=dev, generator=g) * 0.02).abs().bfloat16()
    ws = torch.empty((64, nn, kk), dtype=torch.bfloat16, device=dev)
    y = torch.empty((tot, nn), dtype=torch.bfloat16, device=dev)
    o_t = torch.tensor(offs, dtype=torch.int32, device=dev)
    r_t = torch.tensor(rows, dtype=torch.int32, device=dev)
    ms_fused = _time(lambda: ops.mixed_grouped_gemm_int4(a, bq, sc, o_t, r_t, out=y), args.reps, flush)
    ms_two = _time(lambda: ops.mixed_grouped_gemm_int4(a, bq, sc, o_t, r_t, workspace=ws, out=y, fused=False),
                   args.reps, flush)
    ms_gemm = _time(lambda: ops.ragged_grouped_gemm_bf16(a, ws, o_t, r_t, out=y), args.reps, flush)
    fl = 2.0 * sum(rows) * nn * kk
    out.append({"config": "C4 bf16 x int4 grouped 64 groups m~U[64,512], n=2048 k=7168 gs=128", "sum_m": sum(rows),
                "ms": ms_fused, "tflops": fl / ms_fused / 1e9, "kernel": "fused: int4 expanded in shared memory",
                "ms_two_launches": ms_two, "ms_bf16_gemm_only": ms_gemm, "tflops_bf16_gemm_only": fl / ms_gemm / 1e9,
                "pct_measured_bf16_peak": 100 * fl / ms_fused / 1e9 / bf16_peak})
    assert _lib.status_word() == 0
    return out


if __name__ == "__main__":
    main()
