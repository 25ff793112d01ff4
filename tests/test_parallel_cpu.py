"""world_size-2 gloo tests (CPU) of the multi-GPU host logic: work partitioning and the MoE
dispatch / combine exchange, including a rank that receives nothing."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mosaicist_b200.parallel import TokenExchange, column_range, group_range


def test_partitions_cover_everything_once():
    for n, w in [(8, 1), (8, 2), (8, 8), (5, 2), (3, 4), (256, 8)]:
        got = [g for r in range(w) for g in group_range(n, w, r)]
        assert got == list(range(n))
        sizes = [len(group_range(n, w, r)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1
    cols = [c for r in range(4) for c in (column_range(8192, 4, r).start, column_range(8192, 4, r).stop)]
    assert cols == [0, 2048, 2048, 4096, 4096, 6144, 6144, 8192]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, experts, skew):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        T, k, h = 37 + rank, 3, 8
        tokens = torch.randn((T, h), generator=g)
        if skew:                          # every pair goes to rank 0's experts: rank 1 gets nothing
            ids = torch.randint(0, experts // world, (T, k), generator=g, dtype=torch.int32)
        else:
            ids = torch.randint(0, experts, (T, k), generator=g, dtype=torch.int32)
        weights = torch.rand((T, k), generator=g)
        ex = TokenExchange(experts)
        rows, e_ids, w = ex.dispatch(tokens, ids, weights)
        lo, hi = ex.expert_first, ex.expert_first + ex.experts_local
        assert ((e_ids >= lo) & (e_ids < hi)).all()
        if skew and rank == 1:
            assert rows.shape[0] == 0
        # a stand-in expert: y = row * (expert id + 1) * routing weight
        y = rows * (e_ids.float() + 1)[:, None] * w[:, None]
        back, pos = ex.combine(y)
        got = back[pos.long()].reshape(T, k, h).sum(1)
        want = (tokens[:, None, :] * (ids.float() + 1)[:, :, None] * weights[:, :, None]).sum(1)
        assert torch.allclose(got, want, atol=1e-6), (got - want).abs().max()
        total = torch.tensor([rows.shape[0]])
        dist.all_reduce(total)
        pairs = torch.tensor([T * k])
        dist.all_reduce(pairs)
        assert int(total) == int(pairs)   # every pair arrived somewhere exactly once
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("skew", [False, True])
def test_token_exchange_world2(skew):
    mp.spawn(_worker, args=(2, _free_port(), 8, skew), nprocs=2, join=True)
