"""Multi-GPU plumbing: one process per GPU, torch.distributed (NCCL over NVLink) for the only
step of the path that really exchanges data — MoE token dispatch and combine.

* Grouped GEMMs shard by group and dense GEMMs along N; neither needs a collective
  (`group_range`, `column_range`).
* The MoE layer is expert-parallel: rank r owns experts [r*E/N, (r+1)*E/N) and a slice of the
  tokens.  `PeerExpertParallelMoE` is the fast path: the ranks map each other's GEMM operand
  and result buffers (CUDA IPC over NVLink); after an all-gather of the per-expert counts the
  dispatch kernel quantises every token once and stores the NVFP4 row straight into the owning
  rank's buffers, and the combine kernel reads the expert outputs from the owners and sums
  them.  Two stream-ordered barriers separate the phases; there is no host synchronisation
  and no row ever crosses NVLink in bf16 on the way in.
* `ExpertParallelMoE` is the plain version on library collectives: it sends every
  (token, k) pair to the rank that owns its expert with `all_to_all_single` (counts first,
  then bf16 rows, expert ids and routing weights), runs the local expert layer on what
  arrived, and returns the outputs with a second all-to-all.  It also runs on gloo.

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
        """tokens (T_local, h) bf16, logits (T_local, experts_total) f32 -> (T_local, h) bf16.
        The result is defined only while the library's status word stays 0 (`_lib.status_word()`):
        a step that overflowed a rank's rows_cap (bit 0x00E00000) drops the pairs that did not fit
        from the sum, one whose wait for a peer ran out (0x00D00000) computed on incomplete data."""
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


class _DeviceBytes:
    """Adapter that lets torch view raw device memory (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


EXCHANGE_BUFFERS = ("a_q", "sf_rows", "row_weight", "y", "row_dest", "recv_y", "flags", "counts_all", "row_next")
FLAG_SLOTS, FLAG_PEERS = 4, 16     # a flag table: slots x peers int32 (msc_ep_signal / msc_ep_wait)
SLOT_COUNTS, SLOT_ROWS_LANDED, SLOT_RESULTS_READY = 0, 1, 2


def exchange_layout(rows_cap: int, hidden: int, pairs_cap: int = 0, world: int = 0, experts_total: int = 0):
    """Byte offsets of the EXCHANGE_BUFFERS inside one rank's exchange allocation, and its total
    size.  Sections start on 1 KB boundaries (TMA maps and bulk copies need 16 bytes).
    pairs_cap = tokens * topk this rank may route: the rows of recv_y, where the other ranks'
    second GEMM delivers this rank's results (0: no such buffer, the combine pulls from y).
    world * experts_total sizes the table the peers write their per-expert counts into."""
    sizes = (rows_cap * (hidden // 2), rows_cap * (hidden // 16), rows_cap * 4, rows_cap * hidden * 2,
             rows_cap * 4, pairs_cap * hidden * 2, FLAG_SLOTS * FLAG_PEERS * 4, world * experts_total * 4,
             rows_cap * 4)
    offs, at = [], 0
    for n in sizes:
        offs.append(at)
        at = (at + n + 1023) // 1024 * 1024
    return offs, at


def exchange_views(base: torch.Tensor, rows_cap: int, hidden: int, pairs_cap: int = 0, world: int = 0,
                   experts_total: int = 0) -> dict:
    """The buffers as tensors over a flat uint8 allocation laid out by exchange_layout."""
    offs, total = exchange_layout(rows_cap, hidden, pairs_cap, world, experts_total)
    if base.dtype != torch.uint8 or base.numel() < total:
        raise ValueError(f"need a uint8 allocation of at least {total} bytes")

    def cut(i, nbytes):
        return base[offs[i]:offs[i] + nbytes]

    return {
        "a_q": cut(0, rows_cap * (hidden // 2)).view(rows_cap, hidden // 2),
        "sf_rows": cut(1, rows_cap * (hidden // 16)).view(rows_cap, hidden // 16),
        "row_weight": cut(2, rows_cap * 4).view(torch.float32),
        "y": cut(3, rows_cap * hidden * 2).view(torch.bfloat16).view(rows_cap, hidden),
        "row_dest": cut(4, rows_cap * 4).view(torch.int32),
        "recv_y": cut(5, pairs_cap * hidden * 2).view(torch.bfloat16).view(pairs_cap, hidden),
        "flags": cut(6, FLAG_SLOTS * FLAG_PEERS * 4).view(torch.int32),
        "counts_all": cut(7, world * experts_total * 4).view(torch.int32).view(world, experts_total),
        "row_next": cut(8, rows_cap * 4).view(torch.int32),
    }


class PeerBuffers:
    """One rank's exchange allocation, mapped into every rank of `group` on the same box.

    `tensors` are this rank's EXCHANGE_BUFFERS (a_q, row_weight and y double as the MegaMoE
    workspace; sf_rows receives scale bytes row-major; row_dest and recv_y serve the push
    combine),
    `pointers[name][r]` is rank r's buffer as seen from this process."""

    def __init__(self, rows_cap: int, hidden: int, pairs_cap: int = 0, experts_total: int = 0, group=None):
        import ctypes

        from . import _lib

        lib = _lib.load()
        self.group, self.rows_cap, self.hidden = group, rows_cap, hidden
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        offs, total = exchange_layout(rows_cap, hidden, pairs_cap, self.world, experts_total)
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _lib.check(lib.msc_peer_alloc(total, ctypes.byref(ptr), handle))
        self._own, self._opened = ptr.value, []
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                bases.append(self._own)
                continue
            q = ctypes.c_void_p()
            _lib.check(lib.msc_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(q)))
            self._opened.append(q.value)
            bases.append(q.value)
        dev = torch.device("cuda", torch.cuda.current_device())
        flat = torch.as_tensor(_DeviceBytes(self._own, total), device=dev)
        flat.zero_()
        self.tensors = exchange_views(flat, rows_cap, hidden, pairs_cap, self.world, experts_total)
        self.tensors["row_dest"].fill_(-1)
        self.pointers = {name: [b + offs[i] for b in bases] for i, name in enumerate(EXCHANGE_BUFFERS)}
        dist.barrier(group=group)   # every rank has zeroed its buffers before anyone writes

    def close(self):
        """Unmaps the peers' buffers and frees this rank's (collective: all ranks call it)."""
        from . import _lib

        lib = _lib.load()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for q in self._opened:
            _lib.check(lib.msc_peer_close(q))
        self._opened = []
        dist.barrier(group=self.group)
        if self._own:
            self.tensors = {}
            _lib.check(lib.msc_peer_free(self._own))
            self._own = None


class PeerExpertParallelMoE:
    """MegaMoE over expert-parallel ranks with dispatch and combine through peer memory.

    `layer` is this rank's `moe.MegaMoE` over its local experts, built with topk=1,
    expert_first=rank * E_local, rows_cap=`rows_cap` and workspace=this rank's exchange buffers;
    `pointers[name][r]` are the device addresses of rank r's a_q / sf_rows / row_weight / y
    (`PeerBuffers.pointers`), `sf_rows` this rank's own (rows_cap, h/16) scale rows; `input_gs_all` (experts_total,) f32 holds every expert's input
    global scale, since the sender quantises.  The phases `count`, `place`, `dispatch`,
    `experts`, `combine` are public so one process can drive several ranks' layers in lockstep
    on one device (each phase for every rank before the next phase)."""

    def __init__(self, layer, pointers: dict, sf_rows, input_gs_all, experts_total: int, topk: int,
                 max_tokens: int, rank: int, world: int, group=None, row_dest=None, recv_y=None,
                 flags=None, counts_all=None, row_next=None):
        """With `row_dest` (rows_cap,) i32 and `recv_y` (>= max_tokens * topk, h) bf16 — this
        rank's buffers of those names, whose addresses on every rank are in `pointers` — the
        combine is pushed: the second GEMM scatters each result row into the home rank's recv_y
        while it runs, and `combine` only sums k local rows per token.  Without them `combine`
        pulls the rows from the owners' y after the GEMM.
        With `row_next` (rows_cap,) i32 as well, a token's result rows that live on the same rank
        are summed there before they cross NVLink (about a third fewer rows under uniform
        routing): the second GEMM stores locally and msc_ep_presum_push sends one row per
        (token, rank).  The sum is then rounded once per rank the token visits, so the result is
        no longer bit-identical to the single-GPU layer, only within the layer's tolerance.
        With `flags` and `counts_all` (this rank's buffers of those names) the ranks synchronise
        through flags in each other's memory (msc_ep_signal / msc_ep_wait) and exchange the
        counts the same way; without them `forward` uses an NCCL all-gather and two all-reduces."""
        import ctypes

        if experts_total % world:
            raise ValueError(f"{experts_total} experts do not split over {world} ranks")
        if layer.topk != 1 or layer.expert_first != rank * (experts_total // world):
            raise ValueError("the local layer must be built with topk=1 and this rank's expert_first")
        self.layer, self.topk, self.E, self.group = layer, topk, experts_total, group
        self.rank, self.world, self.rows_cap, self.max_tokens = rank, world, layer.rows_cap, max_tokens
        self.input_gs_all = input_gs_all.float().contiguous()
        arr = ctypes.c_void_p * world
        if tuple(sf_rows.shape) != (layer.rows_cap, layer.h // 16) or sf_rows.dtype != torch.uint8:
            raise ValueError("sf_rows must be (rows_cap, h/16) uint8")
        if sf_rows.data_ptr() != pointers["sf_rows"][rank]:
            raise ValueError("sf_rows is not the buffer the other ranks were given for this rank")
        self.sf_rows = sf_rows
        self._q, self._sf = arr(*pointers["a_q"]), arr(*pointers["sf_rows"])
        self._rw, self._y = arr(*pointers["row_weight"]), arr(*pointers["y"])
        self.push = row_dest is not None
        if self.push:
            if recv_y is None or recv_y.shape[0] < max_tokens * topk or recv_y.shape[1] != layer.h:
                raise ValueError("recv_y must hold max_tokens * topk rows of h bf16 values")
            if row_dest.data_ptr() != pointers["row_dest"][rank] or recv_y.data_ptr() != pointers["recv_y"][rank]:
                raise ValueError("row_dest / recv_y are not the buffers the other ranks were given")
            self.row_dest, self.recv_y = row_dest, recv_y
            self._rd, self._ry = arr(*pointers["row_dest"]), arr(*pointers["recv_y"])
        else:
            self._rd = None
        self.presum = row_next is not None
        self._rn = None
        if self.presum:
            if not self.push:
                raise ValueError("row_next (the pre-summed combine) needs row_dest and recv_y")
            if row_next.data_ptr() != pointers["row_next"][rank] or tuple(row_next.shape) != (layer.rows_cap,):
                raise ValueError("row_next is not the (rows_cap,) buffer the other ranks were given")
            self.row_next, self._rn = row_next, arr(*pointers["row_next"])
        dev = layer.a_q.device
        i32 = dict(dtype=torch.int32, device=dev)
        T, K = max_tokens, topk
        self.ids = torch.zeros((T, K), **i32)
        self.weights = torch.zeros((T, K), dtype=torch.float32, device=dev)
        self.rank_in_group = torch.zeros((T, K), **i32)
        self.pair_row = torch.full((T, K), -1, **i32)
        self.counts = torch.zeros((experts_total,), **i32)
        self.flag_sync = flags is not None
        if self.flag_sync:
            if counts_all is None or tuple(counts_all.shape) != (world, experts_total):
                raise ValueError("counts_all must be this rank's (world, experts_total) exchange table")
            if flags.data_ptr() != pointers["flags"][rank] or counts_all.data_ptr() != pointers["counts_all"][rank]:
                raise ValueError("flags / counts_all are not the buffers the other ranks were given")
            self.flags, self.counts_all = flags, counts_all
            self._fl, self._ca = arr(*pointers["flags"]), arr(*pointers["counts_all"])
            self.epoch = 0
        else:
            self.counts_all = torch.zeros((world, experts_total), **i32)
        self.send_base = torch.zeros((experts_total,), **i32)
        self._tmp = torch.zeros((experts_total + 8,), **i32)
        self._scratch = torch.zeros((4,), **i32)
        self._flag = torch.zeros((1,), **i32)
        self._T = 0

    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    def count(self, logits):
        """Routes this rank's tokens and counts its pairs per global expert (`counts`)."""
        from . import _lib

        lib = _lib.load()
        T = logits.shape[0]
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed the workspace built for {self.max_tokens}")
        self._T = T
        st = self._stream()
        _lib.check(lib.msc_moe_route_topk(logits.data_ptr(), self.ids.data_ptr(), self.weights.data_ptr(),
                                          T, logits.shape[1], self.topk, st))
        _lib.check(lib.msc_moe_plan(self.ids.data_ptr(), T * self.topk, 0, self.E,
                                    self.rank_in_group.data_ptr(), self.counts.data_ptr(),
                                    self._tmp.data_ptr(), self._tmp[self.E:].data_ptr(),
                                    self._scratch.data_ptr(), st))
        return self.counts

    def signal(self, slot: int, with_counts: bool = False):
        """Raises this rank's flag of `slot` on every rank (after publishing its counts)."""
        from . import _lib

        _lib.check(_lib.load().msc_ep_signal(self._fl, self.world, self.rank, slot, self.epoch,
                                             self.counts.data_ptr() if with_counts else None,
                                             self._ca if with_counts else None, self.E, self._stream()))

    def wait(self, slot: int):
        """Waits (bounded) until every rank has raised its flag of `slot` for this layer call."""
        from . import _lib

        _lib.check(_lib.load().msc_ep_wait(self.flags.data_ptr(), self.world, slot, self.epoch, self._stream()))

    def place(self, counts_all=None, wait: bool = False):
        """From all ranks' counts: where this rank's pairs go, and this rank's group table.
        wait=True (flag synchronisation): the kernel first waits for every rank's counts."""
        from . import _lib

        L = self.layer
        if counts_all is None:
            counts_all = self.counts_all
        _lib.check(_lib.load().msc_ep_offsets(counts_all.data_ptr(), self.world, self.rank, self.E,
                                              self.rows_cap, self.send_base.data_ptr(),
                                              L.group_rows.data_ptr(), L.group_offsets.data_ptr(),
                                              L.total_rows.data_ptr(),
                                              self.flags.data_ptr() if wait else None, SLOT_COUNTS,
                                              self.epoch if wait else 0, self._stream()))

    def dispatch(self, tokens):
        from . import _lib

        T = self._T
        if tokens.shape[0] != T or tokens.dtype != torch.bfloat16 or not tokens.is_contiguous():
            raise ValueError("tokens must be the contiguous bf16 rows the logits were routed for")
        _lib.check(_lib.load().msc_ep_dispatch_quantize(
            tokens.data_ptr(), self.ids.data_ptr(), self.weights.data_ptr(), self.rank_in_group.data_ptr(),
            self.send_base.data_ptr(), self.input_gs_all.data_ptr(), T, self.layer.h, self.topk, self.E,
            self.world, self._q, self._sf, self._rw, self._rd, self._rn, self.rank, self.rows_cap,
            self.pair_row.data_ptr(), self._stream()))

    def experts(self):
        """Tiles the received scale rows for the MMA, then the two grouped GEMMs."""
        from . import _lib

        L = self.layer
        _lib.check(_lib.load().msc_sf_swizzle(self.sf_rows.data_ptr(), L.a_sf.data_ptr(), 1, self.rows_cap,
                                              L.h // 16, self._stream()))
        if not self.push:
            L.run_experts()
            return
        if self.presum:
            L.run_experts()
            _lib.check(_lib.load().msc_ep_presum_push(L.y.data_ptr(), self.row_dest.data_ptr(),
                                                      self.row_next.data_ptr(), self._ry, self.world,
                                                      self.max_tokens * self.topk, self.rows_cap, L.h,
                                                      self._stream()))
            self.row_dest.fill_(-1)
            return
        L.run_gemm1()
        _lib.check(_lib.load().msc_grouped_gemm_nvfp4_scatter_ragged(
            L.d_q.data_ptr(), L.d_sf.data_ptr(), L.w2_q.data_ptr(), L.w2_sf.data_ptr(), L.alpha2.data_ptr(),
            L.group_offsets.data_ptr(), L.group_rows.data_ptr(), L.row_weight.data_ptr(),
            self.row_dest.data_ptr(), self._ry, self.world, self.max_tokens * self.topk, L.E, self.rows_cap,
            L.h, L.n, L.config.c(), self._stream()))
        # rows nobody writes in the next step must not keep this step's destination
        self.row_dest.fill_(-1)

    def combine(self, out=None):
        from . import _lib

        T = self._T
        if out is None:
            out = torch.empty((T, self.layer.h), dtype=torch.bfloat16, device=self.ids.device)
        if self.push:
            _lib.check(_lib.load().msc_ep_sum_pairs(self.recv_y.data_ptr(), self.pair_row.data_ptr(),
                                                    out.data_ptr(), T, self.layer.h, self.topk, self._stream()))
            return out
        _lib.check(_lib.load().msc_ep_combine(self._y, self.ids.data_ptr(), self.pair_row.data_ptr(),
                                              out.data_ptr(), T, self.layer.h, self.topk, self.E,
                                              self.world, self.rows_cap, self._stream()))
        return out

    def forward(self, tokens, logits, out=None):
        """tokens (T_local, h) bf16, logits (T_local, experts_total) f32 -> (T_local, h) bf16.
        The result is defined only while the library's status word stays 0 (`_lib.status_word()`):
        a step that overflowed a rank's rows_cap (bit 0x00E00000) drops the pairs that did not fit
        from the sum, one whose wait for a peer ran out (0x00D00000) computed on incomplete data."""
        self.count(logits)
        if self.flag_sync:
            self.epoch += 1
            self.signal(SLOT_COUNTS, with_counts=True)
            self.place(wait=True)
            self.dispatch(tokens)
            self.signal(SLOT_ROWS_LANDED)
            self.wait(SLOT_ROWS_LANDED)         # every rank's rows have landed
            self.experts()
            self.signal(SLOT_RESULTS_READY)
            self.wait(SLOT_RESULTS_READY)       # every rank's results are complete
            return self.combine(out)
        dist.all_gather_into_tensor(self.counts_all, self.counts, group=self.group)
        self.place(self.counts_all)
        self.dispatch(tokens)
        dist.all_reduce(self._flag, group=self.group)   # every rank's rows have landed
        self.experts()
        dist.all_reduce(self._flag, group=self.group)   # every rank's results are complete
        return self.combine(out)
