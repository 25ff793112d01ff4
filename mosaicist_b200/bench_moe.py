"""Benchmark of the routed MoE layer at the DeepSeek-V3 shape: 8192 tokens, hidden 7168,
256 experts, top-8 softmax routing, expert intermediate 2048, SwiGLU, NVFP4 weights and
activations.

    python -m mosaicist_b200.bench_moe [--tokens 8192] [--steps 20]
    python -m torch.distributed.run --nproc-per-node N -m mosaicist_b200.bench_moe --gpus N

One GPU runs all 256 experts; N GPUs run expert-parallel (256/N experts and 8192/N tokens per
rank).  `--exchange peer` (default) dispatches NVFP4 rows into, and combines from, the other
ranks' buffers through peer memory; `--exchange nccl` uses all-to-all collectives on bf16 rows.  Weights are random bytes in the NVFP4 layout
(values uniform over the e2m1 codes, block scales in a narrow e4m3 range): the timing does not
depend on their values, and quantising 6 GB of weights from fp32 would dominate set-up.
Prints one JSON line: layer TFLOP/s (2 * routed rows * (hidden * 2n + n * hidden)), time per
layer, and the time of each stage on one GPU.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch


def rand_weights(E, n, h, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    w1_q = torch.randint(0, 256, (E, 2 * n, h // 2), dtype=torch.uint8, device=dev, generator=g)
    w2_q = torch.randint(0, 256, (E, h, n // 2), dtype=torch.uint8, device=dev, generator=g)
    w1_sf = torch.randint(0x28, 0x38, (E, 2 * n // 128, h // 64, 32, 16), dtype=torch.uint8, device=dev, generator=g)
    w2_sf = torch.randint(0x28, 0x38, (E, h // 128, n // 64, 32, 16), dtype=torch.uint8, device=dev, generator=g)
    one = torch.ones((E,), dtype=torch.float32, device=dev)
    return w1_q, w1_sf, one * 64, one, w2_q, w2_sf, one * 64, one


def parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cta-pair", type=int, default=0)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--gemm1-row-major", action="store_true",
                    help="fused GEMM1 on the row-major pair kernel instead of the tokens-on-N kernel (one GPU)")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer")
    ap.add_argument("--sync", choices=["flags", "nccl"], default="flags",
                    help="peer exchange: synchronise through flags in peer memory / NCCL collectives")
    ap.add_argument("--combine", choices=["push", "pull", "presum"], default="push",
                    help="peer exchange: GEMM2 scatters result rows to the home ranks / the home rank pulls them")
    return ap


def main():
    import torch.distributed as dist

    args = parser().parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    out = measure(args, rank, world, local)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure(args, rank: int, world: int, local: int, detail: bool = True) -> dict:
    """One timed run of the layer on `world` ranks (the process group, if any, is the
    caller's); returns the record rank 0 prints.  detail=False leaves out the per-stage /
    per-phase timings."""
    import torch.distributed as dist

    from . import _lib, ops
    from .moe import MegaMoE
    from .parallel import ExpertParallelMoE, PeerBuffers, PeerExpertParallelMoE

    dev = torch.device("cuda", local)
    E, k, h, n = args.experts, args.topk, args.hidden, args.inter
    E_loc, T_loc = E // world, args.tokens // world
    w = rand_weights(E_loc, n, h, dev, 17 + rank)
    gs_in = torch.full((E_loc,), 2688.0 / 5.0, dtype=torch.float32, device=dev)
    gs_a2 = torch.full((E_loc,), 2688.0 / 8.0, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    tokens = torch.randn((T_loc, h), device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn((T_loc, E), device=dev, generator=g)

    cfg = ops.GemmConfig(tile_n=args.tile_n, cta_pair=args.cta_pair)
    if world == 1:
        layer = MegaMoE(*w, gs_in, gs_a2, topk=k, max_tokens=T_loc, config=cfg,
                        gemm1_tokens_on_n=False if args.gemm1_row_major else None)
        run = lambda: layer.forward(tokens, logits)
    elif args.exchange == "nccl":
        # a rank can receive up to 2x its even share before the workspace is exceeded
        inner = MegaMoE(*w, gs_in, gs_a2, topk=1, max_tokens=2 * T_loc * k, expert_first=rank * E_loc,
                        config=cfg)
        layer = ExpertParallelMoE(inner, E, k)
        run = lambda: layer.forward(tokens, logits)
    else:
        rows_cap = (2 * T_loc * k + 127 * E_loc + 127) // 128 * 128
        push = args.combine in ("push", "presum")
        bufs = PeerBuffers(rows_cap, h, T_loc * k if push else 0, E)
        extra = dict(row_dest=bufs.tensors["row_dest"], recv_y=bufs.tensors["recv_y"]) if push else {}
        if args.combine == "presum":
            extra.update(row_next=bufs.tensors["row_next"])
        if args.sync == "flags":
            extra.update(flags=bufs.tensors["flags"], counts_all=bufs.tensors["counts_all"])
        inner = MegaMoE(*w, gs_in, gs_a2, topk=1, max_tokens=1, expert_first=rank * E_loc, config=cfg,
                        rows_cap=rows_cap, workspace=bufs.tensors)
        gs_all = torch.full((E,), 2688.0 / 5.0, dtype=torch.float32, device=dev)
        layer = PeerExpertParallelMoE(inner, bufs.pointers, bufs.tensors["sf_rows"], gs_all, E, k, T_loc, rank, world,
                                      **extra)
        run = lambda: layer.forward(tokens, logits)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        run()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        run()
    e.record()
    barrier()
    ms = s.elapsed_time(e) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert _lib.status_word() == 0
    flop = 2.0 * args.tokens * k * (h * 2 * n + n * h)
    out = {"metric": "megamoe_layer_tflops", "value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "n_gpus": world, "ms_per_layer": ms, "steps": args.steps,
           "config": {"workload": f"MegaMoE tokens={args.tokens} hidden={h} experts={E} top{k} inter={n}",
                      "parallelism": "single GPU" if world == 1 else
                      (f"ep{world}, all-to-all bf16 dispatch + combine" if args.exchange == "nccl" else
                       f"ep{world}, NVFP4 dispatch into peer memory, bf16 results " +
                       ("scattered to the home rank by the GEMM2 epilogue" if args.combine == "push" else
                        "summed per rank after GEMM2, one row per (token, rank) sent home" if args.combine == "presum" else
                        "pulled from peer memory") + f", sync by {args.sync}")}}

    if world == 1 and detail:
        # per-stage device times on one GPU
        lib = _lib.load()
        L = layer
        st = torch.cuda.current_stream().cuda_stream
        stages = {
            "route": lambda: L.route(logits),
            "plan": lambda: _lib.check(lib.msc_moe_plan(L.ids.data_ptr(), T_loc * k, 0, E_loc, L.rank.data_ptr(),
                                                        L.group_rows.data_ptr(), L.group_offsets.data_ptr(),
                                                        L.total_rows.data_ptr(), L.scratch.data_ptr(), st)),
            "gather_quantize": lambda: _lib.check(lib.msc_moe_permute_quantize(
                tokens.data_ptr(), L.ids.data_ptr(), L.weights.data_ptr(), L.rank.data_ptr(),
                L.group_offsets.data_ptr(), L.input_gs.data_ptr(), T_loc, h, k, 0, E_loc, L.a_q.data_ptr(),
                L.a_sf.data_ptr(), L.row_weight.data_ptr(), L.row_token.data_ptr(),
                None if L.sf_rows is None else L.sf_rows.data_ptr(), L.rows_cap, L.total_rows.data_ptr(), st)),
            "gemm1": lambda: ops.ragged_grouped_gemm_nvfp4(L.a_q, L.a_sf, L.w1_q, L.w1_sf, L.group_offsets,
                                                            L.group_rows, L.alpha1, None, L.config, out=L.gateup),
            "silu_mul_quantize": lambda: ops.quantize_nvfp4_ragged(L.gateup, L.a2_gs, L.group_offsets,
                                                                    L.group_rows, silu=True, out=(L.d_q, L.d_sf)),
            "gemm1_swiglu_quantize_fused": lambda: ops.ragged_gemm1_swiglu_quantize(
                L.a_q, L.a_sf, L.w1_q, L.w1_sf, L.group_offsets, L.group_rows, L.alpha1, L.a2_gs,
                L.gemm1_config, out=(L.d_q, L.d_sf)),
            "gemm2": lambda: ops.ragged_grouped_gemm_nvfp4(L.d_q, L.d_sf, L.w2_q, L.w2_sf, L.group_offsets,
                                                            L.group_rows, L.alpha2, L.row_weight, L.config, out=L.y),
            "combine": lambda: _lib.check(lib.msc_moe_unpermute(
                L.y.data_ptr(), L.ids.data_ptr(), L.rank.data_ptr(), L.group_offsets.data_ptr(),
                combined.data_ptr(), T_loc, h, k, 0, E_loc, st)),
        }
        combined = torch.empty((T_loc, h), dtype=torch.bfloat16, device=dev)
        per = {}
        for name, fn in stages.items():
            fn(); torch.cuda.synchronize()
            s.record()
            for _ in range(5):
                fn()
            e.record(); torch.cuda.synchronize()
            per[name] = s.elapsed_time(e) * 1e3 / 5
        out["stage_us"] = per
        out["rows"] = int(L.total_rows[0])
    if world > 1 and args.exchange == "peer" and detail:
        # device time of each phase on this rank (waiting for slower ranks shows up in the barriers)
        L = layer
        from .parallel import SLOT_COUNTS, SLOT_RESULTS_READY, SLOT_ROWS_LANDED

        def bump():
            L.epoch += 1

        if args.sync == "flags":
            phases = [("route_count", lambda: (bump(), L.count(logits))),
                      ("publish_counts", lambda: L.signal(SLOT_COUNTS, with_counts=True)),
                      ("place", lambda: L.place(wait=True)),
                      ("dispatch", lambda: L.dispatch(tokens)),
                      ("barrier_rows_landed", lambda: (L.signal(SLOT_ROWS_LANDED), L.wait(SLOT_ROWS_LANDED))),
                      ("experts", L.experts),
                      ("barrier_results_ready", lambda: (L.signal(SLOT_RESULTS_READY), L.wait(SLOT_RESULTS_READY))),
                      ("combine", L.combine)]
        else:
            phases = [("route_count", lambda: L.count(logits)),
                      ("allgather_counts", lambda: dist.all_gather_into_tensor(L.counts_all, L.counts)),
                      ("place", lambda: L.place(L.counts_all)),
                      ("dispatch", lambda: L.dispatch(tokens)),
                      ("barrier_rows_landed", lambda: dist.all_reduce(L._flag)),
                      ("experts", L.experts),
                      ("barrier_results_ready", lambda: dist.all_reduce(L._flag)),
                      ("combine", L.combine)]
        acc = {name: 0.0 for name, _ in phases}
        reps = 5
        for _ in range(reps):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(phases) + 1)]
            ev[0].record()
            for i, (_, fn) in enumerate(phases):
                fn()
                ev[i + 1].record()
            torch.cuda.synchronize()
            for i, (name, _) in enumerate(phases):
                acc[name] += ev[i].elapsed_time(ev[i + 1]) * 1e3 / reps
        out["phase_us_rank0"] = acc
        out["rows_rank0"] = int(inner.total_rows[0])
        assert _lib.status_word() == 0
    if world > 1 and args.exchange == "peer":
        bufs.close()
    return out


if __name__ == "__main__":
    main()
