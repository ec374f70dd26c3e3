"""Mixture-of-experts feed-forward block of the hybrid MoE variant: 512 routed experts (top-10, softmax
router, renormalised) + one sigmoid-gated shared expert, experts stored as stacked trellis tensors.

Single rank: router -> device plan (pairs sorted by expert) -> grouped gate_up -> grouped down with the
SwiGLU in its prologue -> deterministic combine.  Nothing about the routing is read back by the host
(the reference's host-routed block does one D2H of ids per call:
reference src/model/qwen4exp/include/r4dx/model/qwen4exp/moe_block.h:1-20, grouped decode
src/model/qwen4exp/kernels/moe_trellis_decode.hip:86-416).  Under expert parallelism (``parallel/ep.py``)
the same grouped kernels run on each rank's expert slice and the combine sums across ranks.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..ops import kernels as K
from ..quant.trellis import TrellisWeight

BF = torch.bfloat16
GROUPED_MIN_ROWS = int(os.environ.get("R4DXB_MOE_GROUPED_MIN_ROWS", "16"))   # above: the grouped tensor-core path


@dataclass
class ExpertStack:
    """E experts' packed weights back to back: words [E * per_expert], suh [E, K], svh [E, N]."""
    words: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor
    E: int
    N: int
    K: int
    kb: int

    @staticmethod
    def from_list(ws) -> "ExpertStack":
        w0 = ws[0]
        assert all(w.kb == w0.kb and w.N == w0.N and w.K == w0.K for w in ws), "experts of a stack share shape and bit width"
        return ExpertStack(torch.cat([w.words for w in ws]).contiguous(), torch.stack([w.suh for w in ws]).contiguous(),
                           torch.stack([w.svh for w in ws]).contiguous(), len(ws), w0.N, w0.K, w0.kb)

    @property
    def nbytes(self) -> int:
        return self.words.numel() * 4 + self.suh.numel() * 2 + self.svh.numel() * 2


class MoeBlock:
    """One layer's routed + shared experts.  ``e_begin/e_count``: the expert slice this rank holds."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, object], layer: int, device, max_rows: int, e_begin: int = 0,
                 e_count: Optional[int] = None, tmax: int = 2, share_from: Optional["MoeBlock"] = None):
        self.cfg = cfg
        p = f"text.layers.{layer}.moe."
        self.e_begin = e_begin
        self.e_count = e_count if e_count is not None else cfg.num_experts
        if share_from is not None:      # another block object of the same layer already stacked the experts
            self.gate_up, self.down = share_from.gate_up, share_from.down
        else:
            self.gate_up = ExpertStack.from_list([weights[p + f"experts.{e}.gate_up"] for e in range(e_begin, e_begin + self.e_count)])
            self.down = ExpertStack.from_list([weights[p + f"experts.{e}.down"] for e in range(e_begin, e_begin + self.e_count)])
        self.router = weights[p + "router"]
        self.has_shared = cfg.shared_expert_intermediate_size > 0
        self.shared_gate = weights[p + "shared_gate"] if self.has_shared else None
        self.shared_gu: Optional[TrellisWeight] = weights[p + "shared.gate_up"] if self.has_shared else None
        self.shared_down: Optional[TrellisWeight] = weights[p + "shared.down"] if self.has_shared else None
        self.expert_bias = weights.get(p + "expert_bias")          # sigmoid router only: moves the selection
        self.tmax = tmax
        self.k = cfg.num_experts_per_tok
        H, I = cfg.hidden_size, cfg.moe_intermediate_size
        R, k, E = max_rows, self.k, cfg.num_experts
        z = lambda *s, dtype=BF: torch.zeros(*s, dtype=dtype, device=device)
        self.logits = z(R, E, dtype=torch.float32)
        self.ids = z(R, k, dtype=torch.int32)
        self.wts = z(R, k, dtype=torch.float32)
        self.offsets = z(self.e_count + 1, dtype=torch.int32)
        self.perm = z(R * k, dtype=torch.int32)
        self.gu_pairs = z(R * k, 2 * I)
        self.y_pairs = z(R * k, H)
        self.sh_gu = z(R, 2 * cfg.shared_expert_intermediate_size) if self.has_shared else None
        self.sh_out = z(R, H) if self.has_shared else None
        self.sh_gate = z(R, 1, dtype=torch.float32) if self.has_shared else None
        # many rows: the grouped tensor-core path; rows of the pairs in expert order, and the plan's token tiles
        self.max_rows = R
        if R > GROUPED_MIN_ROWS:
            self.xh_pairs = z(R * k, max(H, I), dtype=torch.float16)
            self.tiles = z(2 * (R * k // 16 + self.e_count + 1), dtype=torch.int32)
            self.ntiles = z(1, dtype=torch.int32)
        self.ks_gu = K.pick_ksplit(self.gate_up.N, self.gate_up.K, target_ctas=1)
        self.ks_dn = K.pick_ksplit(self.down.N, self.down.K, target_ctas=1)
        # one or two rows in flight touch at most k experts each: k * N/128 CTAs leave most of the 148 SMs idle (4 experts of
        # the short-conv MoE geometry: 96 CTAs), so those calls split K over a cluster until about two CTAs per SM exist
        few = int(os.environ.get("R4DXB_MOE_KSPLIT_TARGET", "296"))
        per_expert = max(1, (few + self.k - 1) // self.k)
        self.ks_gu_few = K.pick_ksplit(self.gate_up.N, self.gate_up.K, target_ctas=per_expert)
        self.ks_dn_few = K.pick_ksplit(self.down.N, self.down.K, target_ctas=per_expert)

    compact_grid = os.environ.get("R4DXB_MOE_COMPACT_GRID", "1") != "0"
    fused_route = os.environ.get("R4DXB_MOE_FUSED_ROUTE", "1") != "0"

    def route(self, h: torch.Tensor, T: int) -> None:
        if T > 8:
            K.linear_tc(self.router, h[:T], out=self.logits[:T])      # many rows: the router is a tensor-core product
        else:
            K.bf16_gemv(self.router, h, out=self.logits[:T])
            if self.fused_route:
                # up to 8 rows: selection and plan in one launch (a decode step spent ~25 us per layer in the two)
                sig = self.cfg.moe_router == "sigmoid"
                K.moe_route_plan(self.logits[:T], self.expert_bias if sig else None, self.k, self.cfg.norm_topk_prob, sig,
                                 self.cfg.routed_scaling_factor if sig else 1.0, self.ids, self.wts, self.e_begin, self.e_count,
                                 self.offsets, self.perm)
                return
        if self.cfg.moe_router == "sigmoid":
            K.moe_router_sigmoid(self.logits[:T], self.expert_bias, self.k, self.cfg.norm_topk_prob,
                                 self.cfg.routed_scaling_factor, self.ids, self.wts)
        else:
            K.moe_router(self.logits[:T], self.k, self.cfg.norm_topk_prob, self.ids, self.wts)
        K.moe_plan(self.ids, T * self.k, self.cfg.num_experts, self.e_begin, self.e_count, self.offsets, self.perm)

    def experts(self, h: torch.Tensor, T: int, max_rows: Optional[int] = None) -> None:
        """y_pairs[pair] = down_e(silu(gate_e h) * up_e h) for every pair routed to a local expert.
        ``max_rows``: the largest per-expert row count of the current plan when the caller knows it."""
        g, d = self.gate_up, self.down
        if T > GROUPED_MIN_ROWS:
            return self._experts_grouped(h, T)
        # few rows in flight: 2-row passes (an expert rarely sees more than one); more: 8-row passes.  An expert can
        # receive every row of the call, so the passes cover T rows unless the caller knows the plan's maximum.
        tmax = self.tmax if T <= 4 else 8
        n_pass = ((max_rows if max_rows is not None else T) + tmax - 1) // tmax
        ks_gu, ks_dn = (self.ks_gu_few, self.ks_dn_few) if T <= 2 else (self.ks_gu, self.ks_dn)
        P = T * self.k
        if P < g.E and self.compact_grid:
            # fewer routed pairs than local experts (a decode step: 10 of 512): launch CTAs for the named experts only
            K.trellis_gemv_grouped_pairs(g.words, g.suh, g.svh, h, self.gu_pairs, self.offsets, self.perm, self.ids, P, self.e_begin,
                                         self.k, n_pass, tmax, K.PRO_NONE, g.E, g.N, g.K, g.kb, ks_gu)
            K.trellis_gemv_grouped_pairs(d.words, d.suh, d.svh, self.gu_pairs, self.y_pairs, self.offsets, self.perm, self.ids, P,
                                         self.e_begin, 1, n_pass, tmax, K.PRO_SILU_MUL, d.E, d.N, d.K, d.kb, ks_dn)
            return
        K.trellis_gemv_grouped(g.words, g.suh, g.svh, h, self.gu_pairs, self.offsets, self.perm, self.k, n_pass, tmax,
                               K.PRO_NONE, g.E, g.N, g.K, g.kb, ks_gu)
        K.trellis_gemv_grouped(d.words, d.suh, d.svh, self.gu_pairs, self.y_pairs, self.offsets, self.perm, 1, n_pass, tmax,
                               K.PRO_SILU_MUL, d.E, d.N, d.K, d.kb, ks_dn)

    def _experts_grouped(self, h: torch.Tensor, T: int) -> None:
        """More rows than the weight-streaming passes serve well: every expert's rows in one tensor-core launch per
        projection.  The pairs are transformed in expert order (each expert has its own input signs), a token tile is
        one expert's next ``tn`` rows, and the results land at their pair index.  No row count is read back and no
        expert's rows are capped."""
        g, d = self.gate_up, self.down
        P = T * self.k
        avg = max(1, P // max(1, min(self.e_count, self.cfg.num_experts)))
        # the weights of an expert are decoded once per token tile, so a tile should hold all of an expert's rows
        tn = 16 if avg <= 12 else (32 if avg <= 24 else (64 if avg <= 48 else (128 if avg <= 100 else 256)))
        K.moe_tiles(self.offsets, self.e_count, tn, self.tiles, self.ntiles)
        xh = self.xh_pairs.view(-1)[:P * g.K].view(P, g.K)
        K.trellis_input_grouped(h, g.suh, xh, self.offsets, self.perm, P, self.k, 0)
        K.trellis_gemm_grouped(g.words, g.svh, xh, self.gu_pairs, self.offsets, self.perm, self.tiles, self.ntiles, P, g.E,
                               g.N, g.K, g.kb, tn)
        xh2 = self.xh_pairs.view(-1)[:P * d.K].view(P, d.K)
        K.trellis_input_grouped(self.gu_pairs, d.suh, xh2, self.offsets, self.perm, P, 1, 1)
        K.trellis_gemm_grouped(d.words, d.svh, xh2, self.y_pairs, self.offsets, self.perm, self.tiles, self.ntiles, P, d.E,
                               d.N, d.K, d.kb, tn)

    def shared(self, h: torch.Tensor, T: int) -> None:
        if not self.has_shared:
            return
        if T > 16:
            # many rows: the tensor-core path (input transform + GEMM), SwiGLU fused into the second transform
            xh = K.trellis_input(h[:T], self.shared_gu.suh)
            K.trellis_gemm(self.shared_gu, xh, out=self.sh_gu[:T])
            xh2 = K.trellis_input(self.sh_gu[:T], self.shared_down.suh, fused_silu_mul=True)
            K.trellis_gemm(self.shared_down, xh2, out=self.sh_out[:T])
            K.bf16_gemv(self.shared_gate, h, out=self.sh_gate[:T])
            return
        for s in range(0, T, 8):
            e = min(T, s + 8)
            K.trellis_gemv(self.shared_gu, h[s:e], out=self.sh_gu[s:e])
            K.trellis_gemv(self.shared_down, self.sh_gu[s:e], out=self.sh_out[s:e], prologue=K.PRO_SILU_MUL)
        K.bf16_gemv(self.shared_gate, h, out=self.sh_gate[:T])

    def forward(self, h: torch.Tensor, x: torch.Tensor, T: int, exact_rows: bool = False, residual: bool = True) -> None:
        """x[T, H] += moe(h) (h = post-attention RMSNorm of x).  ``exact_rows``: read the plan's largest per-expert row
        count back (one small copy) and run exactly as many weight-streaming passes as it needs; calls with more than
        ``GROUPED_MIN_ROWS`` rows take the grouped tensor-core path and read nothing back."""
        self.route(h, T)
        self.experts(h, T, self.max_rows_of_an_expert() if exact_rows and T <= GROUPED_MIN_ROWS else None)
        self.shared(h, T)
        K.moe_combine(self.y_pairs, self.ids, self.wts, self.sh_out, self.sh_gate, x if residual else None, x, T,
                      self.cfg.hidden_size, self.k)

    def max_rows_of_an_expert(self) -> int:
        """Largest per-expert row count of the latest plan (one device read)."""
        o = self.offsets.cpu()
        return int((o[1:] - o[:-1]).max().item())

    @property
    def nbytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes + (self.shared_gu.nbytes + self.shared_down.nbytes if self.has_shared else 0)
