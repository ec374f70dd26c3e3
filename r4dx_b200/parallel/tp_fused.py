"""Tensor-parallel communicator whose collectives are issued from inside the compute kernels.

Decode / verify rows (T <= 8): ``r4dxb_trellis_gemv_allreduce`` -- the row-parallel trellis linear
pushes its fp32 partial blocks into every peer's receive slots over NVLink, exchanges per-block
flags at system scope and sums in rank order, so the all-reduce costs one NVLink round inside the
kernel's tail instead of a separate collective launch.  Long prefill chunks and the vocab merge
still use the NCCL baseline inherited from ``NcclComm``.
"""
from __future__ import annotations

import ctypes

import torch

from .. import native
from ..native import c_int, c_ptr, register_cuda_sig
from ..ops import kernels as K
from ..quant.trellis import TrellisWeight
from .symm import SymmBuffer
from .tp_comm import NcclComm

register_cuda_sig("r4dxb_trellis_gemv_allreduce", c_int,
                  [c_ptr] * 6 + [c_int] * 6 + [c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr])

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
        self.symm = SymmBuffer(self.recv_bytes, self.device, group)
        self.recv_tab = self.symm.ptr_table(0)
        self.block_seq = torch.zeros(max_n // 128, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._lib = native.cuda()

    def row_parallel_linear(self, lin, x: torch.Tensor, res: torch.Tensor, prologue: int = 0) -> None:
        w = lin.w
        if not isinstance(w, TrellisWeight) or w.N != self.n:
            return super().row_parallel_linear(lin, x, res, prologue)
        T = res.shape[0]
        rc = self._lib.r4dxb_trellis_gemv_allreduce(
            w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(), res.data_ptr(),
            prologue, T, w.N, w.K, w.kb, lin.ksplit, self.recv_tab, self.block_seq.data_ptr(),
            self.status.data_ptr(), self.world, self.rank, self.spin_limit, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"trellis_gemv_allreduce failed with code {rc}")
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += T * w.N * 4

    def check_healthy(self) -> None:
        code = int(self.status.item())
        if code:
            raise TpTimeoutError(f"rank {self.rank}: no answer from rank {code - 100} inside a fused all-reduce")
