"""Multi-GPU plumbing: one process per GPU, torch.distributed (NCCL over NVLink) for the only
step of the path that really exchanges data — MoE token dispatch and combine.

* Grouped GEMMs shard by group and dense GEMMs along N; neither needs a collective
  (`group_range`, `column_range`).
* The MoE layer is expert-parallel: rank r owns experts [r*E/N, (r+1)*E/N) and a slice of the
  tokens.  `ExpertParallelMoE.forward` routes its tokens, sends every (token, k) pair to the
  rank that owns its expert with `all_to_all_single` (counts first, then rows, expert ids and
  routing weights), runs the local expert layer on what arrived, returns the expert outputs
  with a second all-to-all and sums each token's k contributions.  Received rows always land
  in this GPU's own memory before any kernel reads them.

The reference has no multi-GPU code; this follows the partitioning the benchmark
configuration names (expert-parallel across the GPUs of one box, all-to-all dispatch/combine).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def group_range(groups: int, world: int, rank: int) -> range:
    """Contiguous, balanced share of `groups` independent GEMM groups for `rank`."""
    base, extra = divmod(groups, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def column_range(n: int, world: int, rank: int, multiple: int = 256) -> range:
    """Share of the N columns of a dense GEMM, in units of `multiple` columns."""
    r = group_range(n // multiple, world, rank)
    return range(r.start * multiple, r.stop * multiple)


class TokenExchange:
    """Dispatch / combine of (token, k) pairs between expert-parallel ranks.

    `dispatch` sorts the local pairs by destination rank and exchanges them; `combine` sends
    per-pair results back along the same route and returns them in the local pair order
    (row t*k + j belongs to token t, choice j).  Works on any backend (NCCL on GPUs, gloo on
    CPU for tests)."""

    def __init__(self, experts_total: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts_total % self.world:
            raise ValueError(f"{experts_total} experts do not split over {self.world} ranks")
        self.experts_local = experts_total // self.world
        self.expert_first = self.rank * self.experts_local

    def dispatch(self, tokens, ids, weights):
        """tokens (T, h), ids (T, k) int32 global expert ids, weights (T, k) f32.
        Returns (rows (R, h), expert_ids (R,) int32, row_weights (R,) f32): the pairs this rank's
        experts must process, grouped by source rank."""
        T, k = ids.shape
        flat = ids.reshape(-1).to(torch.int64)
        dest = flat // self.experts_local
        order = torch.sort(dest, stable=True).indices            # pair indices by destination
        self._order = order
        send_counts = torch.bincount(dest, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        self._send = send_counts.tolist()                         # host sync: split sizes
        self._recv = recv_counts.tolist()
        R = sum(self._recv)
        src_rows = tokens.index_select(0, order // k)
        rows = tokens.new_empty((R, tokens.shape[1]))
        dist.all_to_all_single(rows, src_rows, self._recv, self._send, group=self.group)
        e_out = torch.empty((R,), dtype=torch.int32, device=ids.device)
        dist.all_to_all_single(e_out, ids.reshape(-1).index_select(0, order).contiguous(),
                               self._recv, self._send, group=self.group)
        w_out = torch.empty((R,), dtype=torch.float32, device=ids.device)
        dist.all_to_all_single(w_out, weights.reshape(-1).index_select(0, order).contiguous(),
                               self._recv, self._send, group=self.group)
        return rows, e_out, w_out

    def combine(self, y):
        """y (R, h): results for the rows `dispatch` returned, same order.  Returns
        (back (T*k, h) in destination-sorted pair order, position (T*k,) int32) where
        back[position[p]] is the result of local pair p."""
        n_pairs = sum(self._send)
        back = y.new_empty((n_pairs, y.shape[1]))
        dist.all_to_all_single(back, y.contiguous(), self._send, self._recv, group=self.group)
        position = torch.empty_like(self._order)
        position[self._order] = torch.arange(n_pairs, device=self._order.device)
        return back, position.to(torch.int32)


class ExpertParallelMoE:
    """MegaMoE over expert-parallel ranks.  `layer` is this rank's `moe.MegaMoE` holding its
    local experts, built with topk=1, expert_first=rank*E_local and max_tokens >= the most
    rows a rank can receive."""

    def __init__(self, layer, experts_total: int, topk: int, group=None):
        self.layer, self.topk = layer, topk
        self.exchange = TokenExchange(experts_total, group)
        if layer.topk != 1 or layer.expert_first != self.exchange.expert_first:
            raise ValueError("the local layer must be built with topk=1 and this rank's expert_first")
        self._zero = torch.zeros((1,), dtype=torch.int32, device=layer.ids.device)

    def forward(self, tokens, logits):
        """tokens (T_local, h) bf16, logits (T_local, experts_total) f32 -> (T_local, h) bf16."""
        from . import _lib

        lib = _lib.load()
        T, h = tokens.shape
        k = self.topk
        dev = tokens.device
        ids = torch.empty((T, k), dtype=torch.int32, device=dev)
        weights = torch.empty((T, k), dtype=torch.float32, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.msc_moe_route_topk(logits.data_ptr(), ids.data_ptr(), weights.data_ptr(), T,
                                          logits.shape[1], k, st))
        rows, e_ids, w = self.exchange.dispatch(tokens, ids, weights)
        R = rows.shape[0]
        if R > self.layer.max_tokens:
            raise RuntimeError(f"{R} rows arrived, the local layer was built for {self.layer.max_tokens}")
        if R:
            self.layer.ids[:R, 0].copy_(e_ids)
            self.layer.weights[:R, 0].copy_(w)
            y = self.layer.forward(rows, None)
        else:
            y = rows
        back, position = self.exchange.combine(y)
        out = torch.empty((T, h), dtype=torch.bfloat16, device=dev)
        zeros = torch.zeros((T, k), dtype=torch.int32, device=dev)
        _lib.check(lib.msc_moe_unpermute(back.data_ptr(), zeros.data_ptr(), position.data_ptr(),
                                         self._zero.data_ptr(), out.data_ptr(), T, h, k, 0, 1, st))
        return out
