"""Routing and the routed MoE layer on numpy (test infrastructure, not product).

PARITY UNPINNED for routing / permutation: the reference has no such code.  The expert
arithmetic is the reference's `moe_reference` (experiments/flashinfer-megamoe-sm100a/
nvfp4.py:91-108) applied to the rows routed to each expert; the routing rule is the one the
benchmark configuration states (softmax over experts, top-k, weights renormalised), and the
routing weight multiplies the second GEMM's fp32 result before its bf16 rounding, which is
where the CUDA path applies it.
"""

from __future__ import annotations

import numpy as np

from . import nvfp4 as O


def route_topk(logits: np.ndarray, topk: int):
    """(T, E) f32 -> ids (T, k) int32 (descending probability, ties to the lower index),
    weights (T, k) f32 renormalised."""
    x = logits.astype(np.float32)
    e = np.exp(x - x.max(axis=1, keepdims=True)).astype(np.float32)
    p = (e / e.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    order = np.argsort(-p, axis=1, kind="stable")[:, :topk]
    w = np.take_along_axis(p, order, axis=1)
    return order.astype(np.int32), (w / w.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)


def plan(ids: np.ndarray, expert_first: int, experts_local: int):
    """rank of every (token, k) pair inside its expert in token order, rows per expert, and
    128-aligned offsets."""
    flat = ids.reshape(-1)
    rank = np.full(flat.shape, -1, np.int32)
    rows = np.zeros(experts_local, np.int32)
    for i, e in enumerate(flat):
        le = e - expert_first
        if 0 <= le < experts_local:
            rank[i] = rows[le]
            rows[le] += 1
    offs = np.zeros(experts_local, np.int32)
    tot = 0
    for g in range(experts_local):
        offs[g] = tot
        tot += (rows[g] + 127) // 128 * 128
    return rank.reshape(ids.shape), rows, offs, tot


def ep_placement(counts_all: np.ndarray, rank: int):
    """Expert-parallel placement from all ranks' per-expert pair counts (world, experts): the
    first row this rank's pairs of every expert take in the owner's buffers (owner's 128-aligned
    group offset + the pairs of lower ranks), and this rank's own rows per expert, group
    offsets and padded total.  The reference is single-GPU; this states the layout the
    expert-parallel kernels agree on so that a rank's rows of one expert are ordered by source
    rank, then token."""
    world, experts = counts_all.shape
    el = experts // world
    total = counts_all.sum(axis=0)
    aligned = (total + 127) // 128 * 128
    send_base = np.zeros(experts, np.int32)
    for e in range(experts):
        first = e // el * el
        send_base[e] = aligned[first:e].sum() + counts_all[:rank, e].sum()
    mine = slice(rank * el, (rank + 1) * el)
    offs = np.concatenate([[0], np.cumsum(aligned[mine])[:-1]]).astype(np.int32)
    return send_base, total[mine].astype(np.int32), offs, int(aligned[mine].sum())


def routed_moe(tokens_bf16, ids, weights, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha,
               input_gs, a2_gs, expert_first: int = 0):
    """out[t] = bf16( sum_k bf16( w_tk * expert_e(t) ) ) over the local experts, each expert
    computed as moe_reference does (quantise with the expert's input scale, GEMM1 -> bf16,
    SiLU*up in fp32, quantise, GEMM2 in fp32)."""
    T, h = tokens_bf16.shape
    E = w1_q.shape[0]
    acc = np.zeros((T, h), np.float32)
    for k in range(ids.shape[1]):                      # k ascending, like the device sum
        yk = np.zeros((T, h), np.float32)
        for le in range(E):
            sel = np.nonzero(ids[:, k] == expert_first + le)[0]
            if sel.size == 0:
                continue
            x = tokens_bf16[sel][None]
            one = slice(le, le + 1)
            a_q, a_sf = O.quantize_nvfp4(x, input_gs[one])
            gateup = O.masked_grouped_gemm_reference(a_q, a_sf, input_gs[one], w1_q[one], w1_sf[one],
                                                     w1_gs[one], w1_alpha[one], [sel.size], O.BF16)
            d_q, d_sf = O.quantize_nvfp4(O.silu_mul(gateup), a2_gs[one])
            a = O.dequantize_nvfp4(d_q, d_sf, a2_gs[one])[0]
            b = O.dequantize_nvfp4(w2_q[one], w2_sf[one], w2_gs[one])[0]
            y = (a @ b.T) * np.float32(w2_alpha[le]) * weights[sel, k][:, None]
            yk[sel] = O.bf16_round(y)
        acc += yk
    return O.bf16_round(acc)
