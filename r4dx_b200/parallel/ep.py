"""Expert parallelism: tokens sharded by rank (data-parallel attention), experts sharded by rank, and the
all-to-all dispatch / combine issued from inside the kernels over NVLink peer memory
(``native/src/cuda/ep.cu`` + the grouped mode of ``trellis_gemv.cu``).

Per MoE layer: route -> dispatch (rows land in the expert owner's receive buffer) -> plan (from the routing
tables every rank broadcast) -> grouped gate_up reading the received rows -> grouped down whose epilogue stores
into the token owner's combine buffer -> combine (+ shared expert + residual).  ``NcclEpBaseline`` does the same
exchange with library all-to-alls between plain kernels and is what the fused path is measured against.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import native
from ..native import c_int, c_ptr, register_cuda_sig
from ..ops import kernels as K

c_ll = ctypes.c_longlong
register_cuda_sig("r4dxb_ep_dispatch", c_int, [c_ptr] * 6 + [c_int] * 7 + [c_ptr])
register_cuda_sig("r4dxb_ep_plan", c_int, [c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr])
register_cuda_sig("r4dxb_ep_combine", c_int, [c_ptr] * 8 + [c_int] * 6 + [c_ptr, c_ptr])
register_cuda_sig("r4dxb_trellis_gemv_grouped_ep", c_int,
                  [c_ptr] * 7 + [c_int] * 9 + [c_ptr, c_ptr, c_ll, c_ll, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr, c_ptr])

BF = torch.bfloat16


class _LocalBuffer:
    """World-1 stand-in for SymmBuffer (the whole exchange then happens inside one GPU)."""

    def __init__(self, nbytes: int, device):
        self.local = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.world, self.rank = 1, 0
        self.ptrs = [self.local.data_ptr()]

    def ptr_table(self, offset: int = 0):
        arr = (ctypes.c_void_p * 1)()
        arr[0] = self.ptrs[0] + offset
        return arr


class EpComm:
    mode = "fused"

    def __init__(self, world: int, rank: int, device, cfg, max_rows: int, spin_limit: int = 1 << 22,
                 max_rows_per_expert: Optional[int] = None, tmax: Optional[int] = None):
        self.world, self.rank, self.device = world, rank, torch.device(device)
        self.cfg = cfg
        self.k = cfg.num_experts_per_tok
        self.R = max_rows
        self.P = max_rows * self.k
        self.H = cfg.hidden_size
        self.e_per = cfg.num_experts // world
        self.expert_range = (rank * self.e_per, self.e_per)
        self.spin_limit = spin_limit
        # one expert can receive every row of every rank: the passes cover that worst case unless the caller bounds it
        self.cap = max_rows_per_expert or world * max_rows
        self.tmax = tmax or (2 if self.cap <= 4 else 8)       # rows of one expert per grouped launch
        W, P, H = world, self.P, self.H
        a = lambda n: (n + 255) // 256 * 256
        self.off_meta = 0
        self.off_x = a(2 * W * P * 8)
        self.off_xflag = self.off_x + a(2 * W * P * H * 2)
        self.off_comb = self.off_xflag + a(2 * W * P * 4)
        self.off_cnt = self.off_comb + a(2 * P * H * 2)
        total = self.off_cnt + a(2 * P * 4)
        if world > 1:
            from .symm import SymmBuffer
            self.buf = SymmBuffer(total, self.device)
        else:
            self.buf = _LocalBuffer(total, self.device)
        self.t_meta, self.t_x, self.t_xflag = self.buf.ptr_table(self.off_meta), self.buf.ptr_table(self.off_x), self.buf.ptr_table(self.off_xflag)
        self.t_comb, self.t_cnt = self.buf.ptr_table(self.off_comb), self.buf.ptr_table(self.off_cnt)
        base = self.buf.local.data_ptr()
        self.p_meta, self.p_x, self.p_xflag = base + self.off_meta, base + self.off_x, base + self.off_xflag
        self.p_comb, self.p_cnt = base + self.off_comb, base + self.off_cnt
        self.seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.offsets = torch.zeros(self.e_per + 1, dtype=torch.int32, device=self.device)
        self.perm = torch.zeros(W * P, dtype=torch.int32, device=self.device)
        I = cfg.moe_intermediate_size
        self.gu = torch.zeros(W * P, 2 * I, dtype=BF, device=self.device)
        self._L = native.cuda()

    def _s(self):
        return torch.cuda.current_stream().cuda_stream

    def moe_forward(self, block, h: torch.Tensor, x: torch.Tensor, T: int) -> None:
        """x[T, H] += moe(h) with the routed experts spread over the ranks."""
        L, W, P, H, k = self._L, self.world, self.P, self.H, self.k
        K.bf16_gemv(block.router, h, out=block.logits[:T])
        K.moe_router(block.logits[:T], k, self.cfg.norm_topk_prob, block.ids, block.wts)
        rc = L.r4dxb_ep_dispatch(self.t_meta, self.t_x, self.t_xflag, h.data_ptr(), block.ids.data_ptr(), self.seq.data_ptr(),
                                 T, k, H, P, W, self.rank, self.e_per, self._s())
        assert rc == 0, rc
        rc = L.r4dxb_ep_plan(self.p_meta, self.seq.data_ptr(), W, P, self.expert_range[0], self.e_per, self.offsets.data_ptr(),
                             self.perm.data_ptr(), self.spin_limit, self.status.data_ptr(), self._s())
        assert rc == 0, rc
        n_pass = (self.cap + self.tmax - 1) // self.tmax
        g, d = block.gate_up, block.down
        for p_ in range(n_pass):
            rc = L.r4dxb_trellis_gemv_grouped_ep(
                g.words.data_ptr(), g.suh.data_ptr(), g.svh.data_ptr(), self.p_x, self.gu.data_ptr(), self.offsets.data_ptr(),
                self.perm.data_ptr(), 1, p_, self.tmax, K.PRO_NONE, g.E, g.N, g.K, g.kb, block.ks_gu, self.seq.data_ptr(),
                self.p_xflag, W * P * H, W * P, None, None, 0, W, self.spin_limit, self.status.data_ptr(), self._s())
            assert rc == 0, rc
        for p_ in range(n_pass):
            rc = L.r4dxb_trellis_gemv_grouped_ep(
                d.words.data_ptr(), d.suh.data_ptr(), d.svh.data_ptr(), self.gu.data_ptr(), None, self.offsets.data_ptr(),
                self.perm.data_ptr(), 1, p_, self.tmax, K.PRO_SILU_MUL, d.E, d.N, d.K, d.kb, block.ks_dn, self.seq.data_ptr(),
                None, 0, 0, self.t_comb, self.t_cnt, P, W, self.spin_limit, self.status.data_ptr(), self._s())
            assert rc == 0, rc
        block.shared(h, T)
        rc = L.r4dxb_ep_combine(self.p_comb, self.p_cnt, self.seq.data_ptr(), block.ids.data_ptr(), block.wts.data_ptr(),
                                block.sh_out.data_ptr(), block.sh_gate.data_ptr(), x.data_ptr(), T, H, k, P, H // 128,
                                self.spin_limit, self.status.data_ptr(), self._s())
        assert rc == 0, rc

    def check_healthy(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"expert-parallel exchange timed out (code {code})")

    # the dense parts of the model run data-parallel: no tensor-parallel collectives
    def merge_argmax(self, ids, vals) -> None:
        pass

    def row_parallel_linear(self, lin, x, res, prologue: int = 0) -> None:
        lin(x, out=res, residual=res, prologue=prologue)


class NcclEpBaseline(EpComm):
    """Same layer with library collectives: all-gather the routing and the rows, local grouped experts,
    all-reduce of the per-token expert sums.  The number the fused path has to beat."""
    mode = "nccl"

    def moe_forward(self, block, h, x, T):
        W, k, H = self.world, self.k, self.H
        K.bf16_gemv(block.router, h, out=block.logits[:T])
        K.moe_router(block.logits[:T], k, self.cfg.norm_topk_prob, block.ids, block.wts)
        if W == 1:
            K.moe_plan(block.ids, T * k, self.cfg.num_experts, 0, self.e_per, block.offsets, block.perm)
            block.experts(h, T)
            block.shared(h, T)
            K.moe_combine(block.y_pairs, block.ids, block.wts, block.sh_out, block.sh_gate, x, x, T, H, k)
            return
        hs = torch.empty(W, T, H, dtype=BF, device=self.device)
        idsg = torch.empty(W, T, k, dtype=torch.int32, device=self.device)
        dist.all_gather_into_tensor(hs, h.contiguous())
        dist.all_gather_into_tensor(idsg, block.ids[:T].contiguous())
        npairs = W * T * k
        perm = torch.zeros(npairs, dtype=torch.int32, device=self.device)
        K.moe_plan(idsg.view(-1), npairs, self.cfg.num_experts, self.expert_range[0], self.e_per, self.offsets, perm)
        gu = torch.zeros(npairs, block.gate_up.N, dtype=BF, device=self.device)
        y = torch.zeros(npairs, H, dtype=BF, device=self.device)
        n_pass = (self.cap + self.tmax - 1) // self.tmax
        g, d = block.gate_up, block.down
        K.trellis_gemv_grouped(g.words, g.suh, g.svh, hs.view(-1, H), gu, self.offsets, perm, k, n_pass, self.tmax, K.PRO_NONE,
                               g.E, g.N, g.K, g.kb, block.ks_gu)
        K.trellis_gemv_grouped(d.words, d.suh, d.svh, gu, y, self.offsets, perm, 1, n_pass, self.tmax, K.PRO_SILU_MUL,
                               d.E, d.N, d.K, d.kb, block.ks_dn)
        dist.all_reduce(y)                       # rows of foreign experts are zero here
        mine = y.view(W, T * k, H)[self.rank].contiguous()
        block.shared(h, T)
        K.moe_combine(mine, block.ids, block.wts, block.sh_out, block.sh_gate, x, x, T, H, k)
