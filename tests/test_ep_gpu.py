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
