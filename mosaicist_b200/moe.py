"""The MoE expert layer on the block-scaled grouped GEMM.

`moe_masked` is the reference's layer (experiments/flashinfer-megamoe-sm100a/moe.py:47-79):
per-expert padded batches, quantise -> GEMM1 -> SiLU*up + quantise -> GEMM2, with the two-level
scales folded into each GEMM's alpha (`alpha_eff = alpha / (gs_a * gs_b)`, moe.py:14-16).

`MegaMoE` is the routed layer the benchmark configuration describes (tokens x router logits,
top-k softmax routing, SwiGLU experts): route -> plan -> gather + quantise -> GEMM1 ->
SiLU*up + quantise -> GEMM2 (routing weight folded into its epilogue) -> per-token sum.  It
covers the experts [expert_first, expert_first + experts_local) and returns the partial sum
over those, which is the whole answer on one GPU and one rank's share under expert
parallelism.
"""

from __future__ import annotations

import torch

from . import _lib, ops


_OFFSETS = {}


def _masked_offsets(l: int, m: int, device) -> torch.Tensor:
    """Row offsets g * m of a padded (l, m, ...) batch seen as row-concatenated groups."""
    key = (l, m, str(device))
    if key not in _OFFSETS:
        _OFFSETS[key] = (torch.arange(l, dtype=torch.int32, device=device) * m).contiguous()
    return _OFFSETS[key]


def fold_alphas(w1_gs, w1_alpha, w2_gs, w2_alpha, input_global_scale, a2_global_scale):
    """alpha_eff = alpha / (gs_activation * gs_weight) for the two GEMMs (moe.py:14-16)."""
    return ((w1_alpha / (input_global_scale * w1_gs)).contiguous(),
            (w2_alpha / (a2_global_scale * w2_gs)).contiguous())


def moe_masked(hidden, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, masked_m,
               input_global_scale, a2_global_scale, gemm1_config=ops.GemmConfig(),
               gemm2_config=ops.GemmConfig(), fuse_gemm1: bool | None = None, folded_alphas=None):
    """(l, m, k) bf16 in, (l, m, k) bf16 out; rows >= masked_m[l] are left untouched.
    Same arguments as the reference's moe_masked: w1_q (l, 2n, k/2), w1_sf / w2_sf in the MMA
    tiling, w2_q (l, k, n/2), per-expert global scales and alphas (l,) f32.
    fuse_gemm1: GEMM1, SiLU(gate) * up and the requantisation run as one kernel, as the
    reference's fused variant does (gemm1_silu_quantize.py:94); bit-identical to the three-kernel
    form.  Default: whenever 2n % 256 == 0 (at the reference's l=8 m=512 k=2048 n=1024 the
    layer takes 37.0 us fused against 40.0 us as separate kernels).  folded_alphas = fold_alphas(...) skips the four small elementwise kernels that fold
    the global scales into the GEMM alphas (they only depend on the weights and scales)."""
    a_q, a_sf = ops.quantize_nvfp4(hidden, input_global_scale, masked_m)
    g1_alpha, g2_alpha = folded_alphas if folded_alphas is not None else fold_alphas(
        w1_gs, w1_alpha, w2_gs, w2_alpha, input_global_scale, a2_global_scale)
    l, m_rows, kh = a_q.shape
    n2 = w1_q.shape[1]
    if fuse_gemm1 is None:
        fuse_gemm1 = n2 % 256 == 0
    if fuse_gemm1:
        d_q, d_sf = ops.ragged_gemm1_swiglu_quantize(
            a_q.view(l * m_rows, kh), a_sf.view(l * (m_rows // 128), *a_sf.shape[2:]), w1_q, w1_sf,
            _masked_offsets(l, m_rows, a_q.device), masked_m, g1_alpha, a2_global_scale, gemm1_config)
        d_q = d_q.view(l, m_rows, n2 // 4)
        d_sf = d_sf.view(l, m_rows // 128, *d_sf.shape[1:])
    else:
        gateup = ops.masked_grouped_gemm(a_q, a_sf, w1_q, w1_sf, g1_alpha, masked_m, gemm1_config)
        d_q, d_sf = ops.silu_mul_quantize_nvfp4(gateup, a2_global_scale, masked_m)
    return ops.masked_grouped_gemm(d_q, d_sf, w2_q, w2_sf, g2_alpha, masked_m, gemm2_config)


class MegaMoE:
    """Routed SwiGLU expert layer with NVFP4 weights and activations.

    w1_q (E, 2n, h/2) gate rows first, w1_sf (E, 2n/128, h/64, 32, 16), w2_q (E, h, n/2),
    w2_sf (E, h/128, n/64, 32, 16), w*_gs / w*_alpha / input_gs / a2_gs (E,) f32, where E is
    the number of LOCAL experts.  Workspaces are sized for `max_tokens` once."""

    def __init__(self, w1_q, w1_sf, w1_gs, w1_alpha, w2_q, w2_sf, w2_gs, w2_alpha, input_gs, a2_gs,
                 topk: int, max_tokens: int, expert_first: int = 0,
                 config: ops.GemmConfig = ops.GemmConfig(), fuse_gemm1: bool = True,
                 rows_cap: int | None = None, workspace: dict | None = None,
                 gemm1_tokens_on_n: bool | None = None):
        """`rows_cap` overrides the row capacity of the grouped buffers (default: room for
        max_tokens * topk rows plus 127 padding rows per expert); `workspace` may provide the
        buffers other GPUs access under expert parallelism (a_q, a_sf, row_weight, y)."""
        self.E, n2, hh = w1_q.shape
        self.h, self.n, self.topk = hh * 2, n2 // 2, topk
        self.expert_first, self.config = expert_first, config
        # GEMM1 + SiLU*up + requantise as one kernel (needs 2n % 256 == 0); bit-identical to the
        # two-kernel path, which stays available for comparison
        self.fuse_gemm1 = fuse_gemm1 and (n2 % 256 == 0)
        self.w1_q, self.w1_sf, self.w2_q, self.w2_sf = w1_q, w1_sf, w2_q, w2_sf
        # the fused GEMM1 with the tokens on the MMA's N side (GemmConfig(cta_pair=3)) reads w1
        # with gate and up rows interleaved in blocks of 64: the layer then keeps that copy only
        self.gemm1_config = ops.GemmConfig()
        if gemm1_tokens_on_n and not self.fuse_gemm1:
            raise ValueError("gemm1_tokens_on_n needs the fused GEMM1 (2n % 256 == 0)")
        if gemm1_tokens_on_n is None:      # the default wherever the fused GEMM1 runs
            gemm1_tokens_on_n = self.fuse_gemm1
        if gemm1_tokens_on_n:
            self.w1_q, self.w1_sf = ops.swiglu_interleave_w1(w1_q, w1_sf)
            self.gemm1_config = ops.GemmConfig(cta_pair=3)
        self.input_gs, self.a2_gs = input_gs.contiguous(), a2_gs.contiguous()
        self.alpha1 = (w1_alpha / (input_gs * w1_gs)).float().contiguous()
        self.alpha2 = (w2_alpha / (a2_gs * w2_gs)).float().contiguous()
        dev = w1_q.device
        T, K, E = max_tokens, topk, self.E
        self.max_tokens = T
        cap = rows_cap if rows_cap is not None else (T * K + 127 * E + 127) // 128 * 128
        if cap <= 0 or cap % 128:
            raise ValueError(f"rows_cap={cap} must be a positive multiple of 128")
        self.rows_cap = cap
        ws = workspace or {}
        i32 = dict(dtype=torch.int32, device=dev)
        self.ids = torch.empty((T, K), **i32)
        self.weights = torch.empty((T, K), dtype=torch.float32, device=dev)
        self.rank = torch.zeros((T, K), **i32)
        self.group_rows = torch.zeros((E,), **i32)
        self.group_offsets = torch.zeros((E,), **i32)
        self.total_rows = torch.zeros((1,), **i32)
        self.scratch = torch.zeros((4,), **i32)

        def buf(name, shape, dtype, zero):
            t = ws.get(name)
            if t is None:
                return (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=dev)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype or not t.is_contiguous():
                raise ValueError(f"workspace[{name!r}] must be a contiguous {dtype} tensor of shape {shape}")
            return t

        self.a_q = buf("a_q", (cap, self.h // 2), torch.uint8, False)
        self.a_sf = buf("a_sf", (cap // 128, self.h // 64, 32, 16), torch.uint8, True)
        self.row_weight = buf("row_weight", (cap,), torch.float32, True)
        # row-major staging for the dispatch's scale bytes (the tiled layout is written by a
        # re-tiling pass); layers fed by an expert-parallel exchange never dispatch themselves
        self.sf_rows = (torch.zeros((cap, self.h // 16), dtype=torch.uint8, device=dev)
                        if workspace is None and self.h % 256 == 0 else None)
        self.row_token = torch.zeros((cap,), **i32)
        self.gateup = torch.empty((cap, 2 * self.n), dtype=torch.bfloat16, device=dev)
        self.d_q = torch.empty((cap, self.n // 2), dtype=torch.uint8, device=dev)
        self.d_sf = torch.zeros((cap // 128, self.n // 64, 32, 16), dtype=torch.uint8, device=dev)
        self.y = buf("y", (cap, self.h), torch.bfloat16, False)

    def route(self, logits):
        """logits (T, experts_total) f32 -> fills ids / weights; returns them."""
        T, experts = logits.shape
        lib = _lib.load()
        _lib.check(lib.msc_moe_route_topk(logits.data_ptr(), self.ids.data_ptr(),
                                          self.weights.data_ptr(), T, experts, self.topk,
                                          torch.cuda.current_stream().cuda_stream))
        return self.ids[:T], self.weights[:T]

    def forward(self, tokens, logits=None, out=None):
        """tokens (T, h) bf16; logits (T, experts_total) f32, or None to reuse the routing
        already in self.ids / self.weights.  Returns (T, h) bf16."""
        T = tokens.shape[0]
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed the workspace built for {self.max_tokens}")
        lib = _lib.load()
        st = torch.cuda.current_stream().cuda_stream
        if logits is not None:
            self.route(logits)
        K, E = self.topk, self.E
        _lib.check(lib.msc_moe_plan(self.ids.data_ptr(), T * K, self.expert_first, E,
                                    self.rank.data_ptr(), self.group_rows.data_ptr(),
                                    self.group_offsets.data_ptr(), self.total_rows.data_ptr(),
                                    self.scratch.data_ptr(), st))
        _lib.check(lib.msc_moe_permute_quantize(
            tokens.data_ptr(), self.ids.data_ptr(), self.weights.data_ptr(), self.rank.data_ptr(),
            self.group_offsets.data_ptr(), self.input_gs.data_ptr(), T, self.h, K,
            self.expert_first, E, self.a_q.data_ptr(), self.a_sf.data_ptr(),
            self.row_weight.data_ptr(), self.row_token.data_ptr(),
            None if self.sf_rows is None else self.sf_rows.data_ptr(), self.rows_cap,
            self.total_rows.data_ptr(), st))
        self.run_experts()
        if out is None:
            out = torch.empty((T, self.h), dtype=torch.bfloat16, device=tokens.device)
        _lib.check(lib.msc_moe_unpermute(self.y.data_ptr(), self.ids.data_ptr(), self.rank.data_ptr(),
                                         self.group_offsets.data_ptr(), out.data_ptr(), T, self.h, K,
                                         self.expert_first, E, st))
        return out

    def run_experts(self):
        """GEMM1 -> SiLU*up + quantise -> GEMM2 over the grouped rows in a_q / a_sf (layout in
        group_offsets / group_rows), result rows times row_weight into y."""
        self.run_gemm1()
        ops.ragged_grouped_gemm_nvfp4(self.d_q, self.d_sf, self.w2_q, self.w2_sf, self.group_offsets,
                                      self.group_rows, self.alpha2, self.row_weight, self.config,
                                      out=self.y)

    def run_gemm1(self):
        """a_q / a_sf -> d_q / d_sf: GEMM1 with SiLU(gate) * up and the NVFP4 requantisation."""
        if self.fuse_gemm1:
            ops.ragged_gemm1_swiglu_quantize(self.a_q, self.a_sf, self.w1_q, self.w1_sf,
                                             self.group_offsets, self.group_rows, self.alpha1,
                                             self.a2_gs, self.gemm1_config, out=(self.d_q, self.d_sf))
        else:
            ops.ragged_grouped_gemm_nvfp4(self.a_q, self.a_sf, self.w1_q, self.w1_sf, self.group_offsets,
                                          self.group_rows, self.alpha1, None, self.config, out=self.gateup)
            ops.quantize_nvfp4_ragged(self.gateup, self.a2_gs, self.group_offsets, self.group_rows,
                                      silu=True, out=(self.d_q, self.d_sf))
