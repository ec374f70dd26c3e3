"""Tensor-parallel communicator whose collectives are issued from inside the compute kernels.

Decode / verify rows (T <= 8): ``r4dxb_trellis_gemv_allreduce`` -- the row-parallel trellis linear
pushes its fp32 partial blocks into every peer's receive slots over NVLink, exchanges per-block
flags at system scope and sums in rank order, so the all-reduce costs one NVLink round inside the
kernel's tail instead of a separate collective launch.  Prefill chunks: ``r4dxb_trellis_gemm_rs`` -- the tensor-core product stores its partial rows straight into the
receive buffer of the rank that owns each token row (reduce-scatter in the GEMM epilogue, tile by tile);
``r4dxb_tp_reduce_push`` on the owner sums them in rank order on top of the residual row and stores the result
into every rank's residual stream (the all-gather half, pushed by the kernel that made the rows);
``r4dxb_tp_wait`` holds the stream until all rows of the call have arrived.  The vocabulary-parallel greedy pick and the
all-reduce of bare row blocks are one push kernel each (``tp_collectives.cu``).  Every device wait is bounded and sticky:
after the first one that runs out, no later call waits until ``recover()`` has run.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import native
from ..native import c_int, c_ptr, register_cuda_sig
from ..ops import kernels as K
from ..quant.trellis import TrellisWeight
from .symm import SymmBuffer
from .tp_comm import NcclComm

register_cuda_sig("r4dxb_trellis_gemv_allreduce", c_int,
                  [c_ptr] * 6 + [c_int] * 6 + [c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr])
register_cuda_sig("r4dxb_trellis_gemv_mma_allreduce", c_int,
                  [c_ptr] * 6 + [c_int] * 6 + [c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr, c_ptr])
register_cuda_sig("r4dxb_tp_allreduce_rows", c_int, [c_ptr, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr])
register_cuda_sig("r4dxb_tp_argmax_merge", c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr])
register_cuda_sig("r4dxb_trellis_gemm_rs", c_int, [c_ptr, c_ptr, c_ptr] + [c_int] * 5 + [c_ptr, c_ptr, c_ptr] + [c_int] * 3 + [c_ptr])
register_cuda_sig("r4dxb_tp_reduce_push", c_int, [c_ptr, c_ptr, c_ptr, c_ptr, ctypes.c_uint32] + [c_int] * 6 + [c_ptr, c_ptr])
register_cuda_sig("r4dxb_tp_wait", c_int, [c_ptr, ctypes.c_uint32, c_int, c_int, c_ptr, c_ptr])

MAX_ROWS = 8


class TpTimeoutError(RuntimeError):
    pass


class FusedComm(NcclComm):
    mode = "fused"

    def __init__(self, world: int, rank: int, device: str, n: int = 5120, spin_limit: int = 1 << 22, group=None):
        """``n``: the width of the all-reduced rows (hidden size); the receive layout is sized for exactly this N."""
        super().__init__(world, rank, device, group)
        self.n = n
        max_n = n
        self.spin_limit = spin_limit
        self.recv_bytes = 2 * world * MAX_ROWS * max_n * 8      # (fp32 value, u32 sequence) pairs
        self.am_bytes = 2 * world * MAX_ROWS * 2 * 8            # argmax merge: (value, seq) + (id, seq) per row and source rank
        self.symm = SymmBuffer(self.recv_bytes + self.am_bytes, self.device, group)
        self.recv_tab = self.symm.ptr_table(0)
        self.am_tab = self.symm.ptr_table(self.recv_bytes)
        self.block_seq = torch.zeros(max_n // 128, dtype=torch.int32, device=self.device)
        self.am_seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._lib = native.cuda()

    # ---- collectives that are one kernel each -----------------------------------------------------------
    def all_reduce_rows(self, t: torch.Tensor) -> None:
        """In-place sum over the ranks; T <= 8 rows of the hidden width go through the push kernel (same receive buffer
        and counters as the fused products), anything else through the library."""
        if t.dim() != 2 or t.shape[0] > MAX_ROWS or t.shape[1] != self.n or t.dtype != torch.bfloat16 or not t.is_contiguous():
            return super().all_reduce_rows(t)
        rc = self._lib.r4dxb_tp_allreduce_rows(t.data_ptr(), t.shape[0], self.n, self.recv_tab, self.block_seq.data_ptr(),
                                               self.status.data_ptr(), self.world, self.rank, self.spin_limit,
                                               torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"tp_allreduce_rows failed with code {rc}")
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += t.numel() * 4

    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        """In place: every rank ends with the global (max value, lowest id) per row; one kernel, pairs pushed to every peer."""
        T = ids.numel()
        if T > MAX_ROWS:
            return super().merge_argmax(ids, vals)
        rc = self._lib.r4dxb_tp_argmax_merge(ids.data_ptr(), vals.data_ptr(), T, self.am_tab, self.am_seq.data_ptr(),
                                             self.status.data_ptr(), self.world, self.rank, self.spin_limit,
                                             torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"tp_argmax_merge failed with code {rc}")
        self.stats.argmax_merges += 1

    # ---- failure handling ---------------------------------------------------------------------------------
    def recover(self) -> None:
        """After a wait ran out (sticky status word) or a step was abandoned: drain this rank's stream, agree with the other
        ranks on the host that everybody has drained, zero every counter, receive slot and flag, clear the status word and
        prove the path with one all-reduce whose answer is known (reference: src/model/tp/tp_group.h:198 does the same for
        its mailbox: drain, rebase sequence numbers, zero, self-test)."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                 # nobody is still pushing into anybody's slots
        self.symm.local.zero_()
        self.block_seq.zero_()
        self.am_seq.zero_()
        if getattr(self, "pf_symm", None) is not None:
            self.pf_symm.local[self.pf_off_recv:].zero_()     # receive halves, arrival counter, row flags (not the residual stream)
            self.pf_calls = 0
            self.pf_cnt_target = 0
            self.pf_xflag_target = 0
        self.status.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                 # every rank's buffers are clean before the first push
        self.self_test()

    def self_test(self) -> None:
        """One all-reduce and one argmax merge with known answers; raises TpTimeoutError / KernelError otherwise."""
        x = torch.full((2, self.n), float(self.rank + 1), dtype=torch.bfloat16, device=self.device)
        self.all_reduce_rows(x)
        ids = torch.tensor([self.rank * 10 + 3, 7], dtype=torch.int32, device=self.device)
        vals = torch.tensor([float(self.rank), 1.0], dtype=torch.float32, device=self.device)
        self.merge_argmax(ids, vals)
        torch.cuda.synchronize(self.device)
        self.check_healthy()
        want = self.world * (self.world + 1) / 2
        if not bool((x.float() == want).all()):
            raise K.KernelError(f"rank {self.rank}: all-reduce self-test gave {x.float().unique().tolist()}, expected {want}")
        if ids.tolist() != [(self.world - 1) * 10 + 3, 7] or vals.tolist() != [float(self.world - 1), 1.0]:
            raise K.KernelError(f"rank {self.rank}: argmax-merge self-test gave {ids.tolist()} {vals.tolist()}")

    def row_parallel_linear(self, lin, x: torch.Tensor, res: torch.Tensor, prologue: int = 0) -> None:
        w = lin.w
        if not isinstance(w, TrellisWeight) or w.N != self.n:
            return super().row_parallel_linear(lin, x, res, prologue)
        T = res.shape[0]
        if K.use_mma_gemv(T, w.N, w.K, lin.ksplit):
            rc = self._lib.r4dxb_trellis_gemv_mma_allreduce(
                w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(), res.data_ptr(),
                prologue, T, w.N, w.K, w.kb, lin.ksplit, self.recv_tab, self.block_seq.data_ptr(),
                self.status.data_ptr(), self.world, self.rank, self.spin_limit, K.gemm_status(self.device).data_ptr(),
                torch.cuda.current_stream().cuda_stream)
        else:
            rc = self._lib.r4dxb_trellis_gemv_allreduce(
                w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(), res.data_ptr(),
                prologue, T, w.N, w.K, w.kb, lin.ksplit, self.recv_tab, self.block_seq.data_ptr(),
                self.status.data_ptr(), self.world, self.rank, self.spin_limit, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"trellis_gemv_allreduce failed with code {rc}")
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += T * w.N * 4

    # ---- prefill chunks: reduce-scatter in the GEMM epilogue, all-gather pushed by the reducing kernel ----
    def alloc_chunk_x(self, C: int, H: int) -> torch.Tensor:
        """The residual stream of a prefill chunk, in symmetric memory so that owners can push rows into it."""
        taken = getattr(self, "pf_x", None) is not None and C <= self.pf_C     # a second model on this communicator
        if os.environ.get("R4DXB_TP_PREFILL", "fused") != "fused" or H != self.n or taken:
            return torch.empty(C, H, dtype=torch.bfloat16, device=self.device)
        W = self.world
        if getattr(self, "pf_symm", None) is not None:      # a larger chunk replaces the old buffers: drop them first
            self.pf_x = self.pf_symm = self.pf_x_tab = self.pf_recv_tab = self.pf_cnt_tab = self.pf_xflag_tab = None
        self.pf_C, self.pf_H = C, H
        self.pf_rpr_max = (C + W - 1) // W
        a = lambda v: (v + 255) // 256 * 256
        self.pf_off_recv = a(C * H * 2)
        self.pf_recv_bytes = a(W * self.pf_rpr_max * H * 2)
        self.pf_off_cnt = self.pf_off_recv + 2 * self.pf_recv_bytes
        self.pf_off_xflag = self.pf_off_cnt + 256
        self.pf_symm = SymmBuffer(self.pf_off_xflag + 256, self.device, self.group)
        self.pf_x_tab = self.pf_symm.ptr_table(0)
        self.pf_recv_tab = [self.pf_symm.ptr_table(self.pf_off_recv + p * self.pf_recv_bytes) for p in (0, 1)]
        self.pf_cnt_tab = self.pf_symm.ptr_table(self.pf_off_cnt)
        self.pf_xflag_tab = self.pf_symm.ptr_table(self.pf_off_xflag)
        self.pf_calls = 0
        self.pf_cnt_target = 0          # arrivals this rank's counter has been promised so far
        self.pf_xflag_target = 0
        self.pf_x = self.pf_symm.local_view(0, C * H * 2, torch.bfloat16).view(C, H)
        return self.pf_x

    def row_parallel_chunk(self, lin, inp: torch.Tensor, x: torch.Tensor, cb: dict, fused_silu_mul: bool = False) -> None:
        w = lin.w
        pf_x = getattr(self, "pf_x", None)
        if (pf_x is None or x.data_ptr() != pf_x.data_ptr() or not isinstance(w, TrellisWeight) or w.N != self.n):
            return super().row_parallel_chunk(lin, inp, x, cb, fused_silu_mul)
        L, W, rank = self._lib, self.world, self.rank
        T, H = x.shape[0], self.n
        rpr = (T + W - 1) // W
        tn = K.pick_token_tile(T, w.N)
        xh = cb["xh"].view(-1)[:T * w.K].view(T, w.K)
        K.trellis_input(inp, w.suh, out=xh, fused_silu_mul=fused_silu_mul)
        st = torch.cuda.current_stream().cuda_stream
        par = self.pf_calls & 1
        rc = L.r4dxb_trellis_gemm_rs(w.words.data_ptr(), w.svh.data_ptr(), xh.data_ptr(), T, w.N, w.K, w.kb, tn,
                                     K.gemm_status(self.device).data_ptr(), self.pf_recv_tab[par], self.pf_cnt_tab, W, rank, rpr, st)
        if rc != 0:
            raise K.KernelError(f"trellis_gemm_rs failed with code {rc}")
        # arrivals promised to this rank's counter: every CTA (all ranks) whose token tile touches my rows
        lo, hi = rank * rpr, min(T, (rank + 1) * rpr)
        rows_own = max(0, hi - lo)
        tiles = 0 if rows_own == 0 else (hi - 1) // tn - lo // tn + 1
        self.pf_cnt_target = (self.pf_cnt_target + W * (w.N // 128) * tiles) & 0xFFFFFFFF
        base = self.pf_symm.local.data_ptr()
        rc = L.r4dxb_tp_reduce_push(self.pf_x_tab, self.pf_xflag_tab, base + self.pf_off_recv + par * self.pf_recv_bytes,
                                    base + self.pf_off_cnt, self.pf_cnt_target, W, rank, rpr, rows_own, H, self.spin_limit,
                                    self.status.data_ptr(), st)
        if rc != 0:
            raise K.KernelError(f"tp_reduce_push failed with code {rc}")
        self.pf_xflag_target = (self.pf_xflag_target + T) & 0xFFFFFFFF
        rc = L.r4dxb_tp_wait(base + self.pf_off_xflag, self.pf_xflag_target, self.spin_limit, 300 + rank, self.status.data_ptr(), st)
        if rc != 0:
            raise K.KernelError(f"tp_wait failed with code {rc}")
        self.pf_calls += 1
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += T * H * 2

    def check_healthy(self) -> None:
        """Reads the sticky status word (one small device-to-host copy); raises TpTimeoutError naming the wait that ran out."""
        code = int(self.status.item())
        if code == 0:
            return
        if code == 390:
            what = "a split-K hand-off inside a fused product never completed"
        elif code >= 300:
            what = f"the all-gather of a prefill chunk did not arrive (code {code})"
        elif code >= 200:
            what = f"a prefill reduce-scatter wait ran out (code {code})"
        elif code >= 150:
            what = f"no answer from rank {code - 150} inside the vocabulary argmax merge"
        else:
            what = f"no answer from rank {code - 100} inside a fused all-reduce"
        raise TpTimeoutError(f"rank {self.rank}: {what}; the communicator needs recover()")
