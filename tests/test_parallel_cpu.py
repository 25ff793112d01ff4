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


def _placement_worker(rank, world, port, experts):
    """The peer-memory exchange's placement arithmetic, with the counts really all-gathered
    between two processes: every pair gets a distinct row inside its owner's capacity, rows of
    one expert are contiguous and ordered by source rank, then by token."""
    import numpy as np

    from oracle import moe as M

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(50 + rank)
        T, k = 300 + 17 * rank, 4
        ids = np.stack([rng.choice(experts, k, replace=False) for _ in range(T)]).astype(np.int32)
        pos, counts, _, _ = M.plan(ids, 0, experts)
        gathered = [torch.zeros(experts, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts))
        counts_all = torch.stack(gathered).numpy()
        send_base, rows, offs, total = M.ep_placement(counts_all, rank)
        el = experts // world
        dest_rank = ids // el
        dest_row = send_base[ids] + pos
        # publish (owner, row, source, expert, token) of every pair and check globally on rank 0
        mine = np.stack([dest_rank.ravel(), dest_row.ravel(), np.full(T * k, rank), ids.ravel(),
                         np.repeat(np.arange(T), k)], axis=1)
        everything = [None] * world
        dist.all_gather_object(everything, mine)
        tables = [None] * world
        dist.all_gather_object(tables, (rows, offs, total))
        if rank == 0:
            allp = np.concatenate(everything)
            for owner in range(world):
                rws, ofs, tot = tables[owner]
                sel = allp[allp[:, 0] == owner]
                assert len(np.unique(sel[:, 1])) == len(sel)            # no two pairs share a row
                assert sel[:, 1].max(initial=-1) < tot
                for le in range(el):
                    e = owner * el + le
                    grp = sel[sel[:, 3] == e]
                    grp = grp[np.argsort(grp[:, 1])]
                    assert len(grp) == rws[le]
                    assert (grp[:, 1] == ofs[le] + np.arange(len(grp))).all()   # contiguous from the offset
                    key = grp[:, 2] * 10 ** 6 + grp[:, 4]
                    assert (np.diff(key) > 0).all()                           # by source rank, then token
                assert (ofs % 128 == 0).all() and tot % 128 == 0
    finally:
        dist.destroy_process_group()


def test_peer_exchange_placement_world2():
    mp.spawn(_placement_worker, args=(2, _free_port(), 8), nprocs=2, join=True)


def test_exchange_layout_sections_are_aligned_and_disjoint():
    """The exchange allocation: every buffer starts on a 1 KB boundary (TMA maps and bulk copies
    need 16 bytes), no two buffers overlap, and the views have the shapes the kernels expect."""
    from mosaicist_b200.parallel import EXCHANGE_BUFFERS, exchange_layout, exchange_views

    for rows_cap, hidden, pairs_cap, world, experts in [(128, 256, 0, 0, 0), (1280, 7168, 640, 8, 256),
                                                        (384, 512, 96, 2, 32)]:
        offs, total = exchange_layout(rows_cap, hidden, pairs_cap, world, experts)
        assert len(offs) == len(EXCHANGE_BUFFERS) and all(o % 1024 == 0 for o in offs) and total % 1024 == 0
        base = torch.zeros(total, dtype=torch.uint8)
        views = exchange_views(base, rows_cap, hidden, pairs_cap, world, experts)
        assert set(views) == set(EXCHANGE_BUFFERS)
        assert tuple(views["a_q"].shape) == (rows_cap, hidden // 2)
        assert tuple(views["sf_rows"].shape) == (rows_cap, hidden // 16)
        assert tuple(views["y"].shape) == (rows_cap, hidden) and views["y"].dtype == torch.bfloat16
        assert tuple(views["recv_y"].shape) == (pairs_cap, hidden)
        assert tuple(views["counts_all"].shape) == (world, experts) and views["flags"].numel() == 64
        spans = sorted((v.data_ptr() - base.data_ptr(), v.numel() * v.element_size()) for v in views.values())
        for (a0, an), (b0, _) in zip(spans, spans[1:]):
            assert a0 + an <= b0
        assert spans[-1][0] + spans[-1][1] <= total
    with pytest.raises(ValueError):
        exchange_views(torch.zeros(10, dtype=torch.uint8), 128, 256)
