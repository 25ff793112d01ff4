"""Expert-parallel MoE on two GPUs (NCCL all-to-all dispatch / combine) against the CPU
oracle of the whole layer.  Needs two devices; skipped otherwise."""

import os
import socket

import ml_dtypes
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from mosaicist_b200 import _lib
    from mosaicist_b200.moe import MegaMoE
    from mosaicist_b200.parallel import ExpertParallelMoE
    from oracle import moe as M, nvfp4 as O
    from tests.test_moe_gpu import _weights

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        E, k, h, n, T_loc = 32, 2, 256, 128, 160
        E_loc = E // world
        w = _weights(E, h, n, seed=5)                       # every rank derives all experts
        rng = np.random.default_rng([7, rank])
        tokens = rng.standard_normal((T_loc, h)).astype(np.float32).astype(ml_dtypes.bfloat16)
        logits = rng.standard_normal((T_loc, E)).astype(np.float32)
        input_gs = np.full(E, 2688.0 / 6.0, np.float32)
        a2_gs = np.full(E, 2688.0 / 4.0, np.float32)
        sl = slice(rank * E_loc, (rank + 1) * E_loc)

        def T(a):
            return torch.from_numpy(np.ascontiguousarray(a)).cuda()

        local = MegaMoE(T(O.pack_e2m1(w["w1_q"][sl])), T(O.e4m3_bytes(O.retile(w["w1_sf"][sl]))),
                        T(w["w1_gs"][sl]), T(w["w1_alpha"][sl]), T(O.pack_e2m1(w["w2_q"][sl])),
                        T(O.e4m3_bytes(O.retile(w["w2_sf"][sl]))), T(w["w2_gs"][sl]), T(w["w2_alpha"][sl]),
                        T(input_gs[sl]), T(a2_gs[sl]), topk=1, max_tokens=world * T_loc * k,
                        expert_first=rank * E_loc)
        ep = ExpertParallelMoE(local, E, k)
        tk = T(np.asarray(tokens, np.float32)).to(torch.bfloat16)
        for _ in range(2):
            got = ep.forward(tk, T(logits)).float().cpu().numpy()
        assert _lib.status_word() == 0
        ids, wts = M.route_topk(logits, k)
        want = M.routed_moe(tokens, ids, wts, w["w1_q"], w["w1_sf"], w["w1_gs"], w["w1_alpha"], w["w2_q"],
                            w["w2_sf"], w["w2_gs"], w["w2_alpha"], input_gs, a2_gs, 0)
        scale = np.abs(want).max()
        rel = np.abs(got - want).max() / scale
        rms = np.sqrt(np.mean((got - want) ** 2)) / scale
        q.put((rank, float(rel), float(rms), int(np.count_nonzero(want)), want.size))
    finally:
        dist.destroy_process_group()


def _peer_worker(rank, world, port, q, push):
    """PeerExpertParallelMoE between real processes: buffers mapped through CUDA IPC, dispatch
    stores and combine loads crossing NVLink.  Checked bit for bit against the single-GPU layer
    run on this rank's tokens with all experts, and against the oracle within tolerance."""
    import torch.distributed as dist

    from mosaicist_b200 import _lib
    from mosaicist_b200.moe import MegaMoE
    from mosaicist_b200.parallel import PeerBuffers, PeerExpertParallelMoE
    from oracle import moe as M, nvfp4 as O
    from tests.test_moe_gpu import _weights

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    bufs = None
    try:
        E, k, h, n, T_loc = 32, 4, 512, 256, 200
        E_loc = E // world
        w = _weights(E, h, n, seed=6)
        rng = np.random.default_rng([8, rank])
        tokens = rng.standard_normal((T_loc, h)).astype(np.float32).astype(ml_dtypes.bfloat16)
        logits = rng.standard_normal((T_loc, E)).astype(np.float32)
        input_gs = np.where(np.arange(E) % 2 == 0, 2688.0 / 6.0, 2688.0 / 5.0).astype(np.float32)
        a2_gs = np.full(E, 2688.0 / 4.0, np.float32)

        def T(a):
            return torch.from_numpy(np.ascontiguousarray(a)).cuda()

        d = dict(w1_q=T(O.pack_e2m1(w["w1_q"])), w1_sf=T(O.e4m3_bytes(O.retile(w["w1_sf"]))),
                 w1_gs=T(w["w1_gs"]), w1_alpha=T(w["w1_alpha"]), w2_q=T(O.pack_e2m1(w["w2_q"])),
                 w2_sf=T(O.e4m3_bytes(O.retile(w["w2_sf"]))), w2_gs=T(w["w2_gs"]), w2_alpha=T(w["w2_alpha"]))
        sl = slice(rank * E_loc, (rank + 1) * E_loc)
        rows_cap = (world * T_loc * k + 127 * E_loc + 127) // 128 * 128
        bufs = PeerBuffers(rows_cap, h, T_loc * k if push else 0, E)
        extra = dict(row_dest=bufs.tensors["row_dest"], recv_y=bufs.tensors["recv_y"]) if push else {}
        if push:     # the pushed combine also runs on flag synchronisation, the pulled one on NCCL
            extra.update(flags=bufs.tensors["flags"], counts_all=bufs.tensors["counts_all"])
        local = MegaMoE(d["w1_q"][sl], d["w1_sf"][sl], d["w1_gs"][sl], d["w1_alpha"][sl], d["w2_q"][sl],
                        d["w2_sf"][sl], d["w2_gs"][sl], d["w2_alpha"][sl], T(input_gs[sl]), T(a2_gs[sl]),
                        topk=1, max_tokens=1, expert_first=rank * E_loc, rows_cap=rows_cap,
                        workspace=bufs.tensors)
        ep = PeerExpertParallelMoE(local, bufs.pointers, bufs.tensors["sf_rows"], T(input_gs), E, k, T_loc, rank,
                                   world, **extra)
        tk = T(np.asarray(tokens, np.float32)).to(torch.bfloat16)
        for _ in range(3):
            got_t = ep.forward(tk, T(logits))
        torch.cuda.synchronize()
        assert _lib.status_word() == 0
        single = MegaMoE(d["w1_q"], d["w1_sf"], d["w1_gs"], d["w1_alpha"], d["w2_q"], d["w2_sf"], d["w2_gs"],
                         d["w2_alpha"], T(input_gs), T(a2_gs), topk=k, max_tokens=T_loc)
        same = bool(torch.equal(got_t, single.forward(tk, T(logits))))
        got = got_t.float().cpu().numpy()
        ids, wts = M.route_topk(logits, k)
        want = M.routed_moe(tokens, ids, wts, w["w1_q"], w["w1_sf"], w["w1_gs"], w["w1_alpha"], w["w2_q"],
                            w["w2_sf"], w["w2_gs"], w["w2_alpha"], input_gs, a2_gs, 0)
        scale = np.abs(want).max()
        rel = np.abs(got - want).max() / scale
        rms = np.sqrt(np.mean((got - want) ** 2)) / scale
        q.put((rank, float(rel), float(rms), int(np.count_nonzero(want)), want.size, same))
    finally:
        if bufs is not None:
            bufs.close()
        dist.destroy_process_group()


@pytest.mark.parametrize("push", [False, True], ids=["pull", "push"])
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_expert_parallel_two_gpus(push):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, q, push)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    for rank, rel, rms, nz, size, same in [q.get(timeout=5) for _ in range(2)]:
        assert same, f"rank {rank}: differs from the single-GPU layer"
        assert rel < 1e-1 and rms < 1e-2, (rank, rel, rms)
        assert nz > size // 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r, port in zip(range(2), [_free_port()] * 2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    results = [q.get(timeout=5) for _ in range(2)]
    for rank, rel, rms, nz, size in results:
        assert rel < 1e-1 and rms < 1e-2, (rank, rel, rms)
        assert nz > size // 2
