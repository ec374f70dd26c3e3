"""Tensor-parallel communicator: one process per GPU, torch.distributed (NCCL) for bootstrap.

Two data paths implement the same interface:

* ``nccl``  -- the baseline: every row-parallel linear is a local GEMM followed by an NCCL
  all-reduce and a residual add; vocab-parallel argmax is an all-gather of (value, id) pairs.
* ``fused`` -- the product path: the all-reduce is issued from inside the row-parallel GEMM
  kernel over NVLink peer memory (``parallel/symm.py``, ``parallel/tp_fused.py``, the epilogue in
  ``native/src/cuda/tp_push.cuh``); the argmax merge is a kernel that pushes every rank's pair to
  every peer (``native/src/cuda/tp_collectives.cu``).

The reference engine has one all-reduce primitive (bf16 rows, fp32 add, identical bits on every
rank) plus host all-gathers for the vocab merges (reference: src/core/include/r4dx/core/tp_comm.hpp:58-106,
src/model/tp/tp_vocab.h:38-160); the call sites are the same three per layer.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K

BF = torch.bfloat16


class TpStats:
    def __init__(self):
        self.all_reduces = 0
        self.all_reduce_bytes = 0
        self.argmax_merges = 0

    def line(self) -> str:
        return f"[r4dxb-tp] all_reduces={self.all_reduces} bytes={self.all_reduce_bytes} argmax_merges={self.argmax_merges}"


class NcclComm:
    """Baseline communicator: library collectives between kernels."""

    mode = "nccl"

    def __init__(self, world: int, rank: int, device: str, group=None):
        self.world, self.rank, self.device = world, rank, torch.device(device)
        self.group = group
        self.stats = TpStats()
        self._tmp = {}
        self._pair = torch.zeros(8, 2, dtype=torch.float32, device=self.device)
        self._pairs = torch.zeros(world, 8, 2, dtype=torch.float32, device=self.device)

    def _scratch(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        t = self._tmp.get(key)
        if t is None:
            t = torch.empty(*shape, dtype=dtype, device=self.device)
            self._tmp[key] = t
        return t

    # ---- row-parallel linears -----------------------------------------------------------------
    def row_parallel_linear(self, lin, x: torch.Tensor, res: torch.Tensor, prologue: int = 0) -> None:
        """res += all_reduce(lin(act(x))) for T <= 8 rows."""
        tmp = self._scratch(res.shape, BF)
        lin(x, out=tmp, prologue=prologue)
        dist.all_reduce(tmp, group=self.group)
        K.residual_add(res, tmp)
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += tmp.numel() * 2

    def row_parallel_chunk(self, lin, inp: torch.Tensor, x: torch.Tensor, cb: dict, fused_silu_mul: bool = False) -> None:
        tmp = self._scratch(x.shape, BF)
        lin.chunk(inp, cb["xh"], tmp, fused_silu_mul=fused_silu_mul)
        dist.all_reduce(tmp, group=self.group)
        K.residual_add(x, tmp)
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += tmp.numel() * 2

    def all_reduce_rows(self, t: torch.Tensor) -> None:
        """In-place sum of a bf16 row block over the ranks (the families whose block output is normalised before it joins the
        residual stream cannot fold the add into the product's epilogue, so they reduce the bare product)."""
        dist.all_reduce(t, group=self.group)
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += t.numel() * t.element_size()

    # ---- vocab-parallel greedy pick -------------------------------------------------------------
    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        """In place: every rank ends with the global (max value, lowest id) per row."""
        T = ids.numel()
        pair = self._pair                              # always 8 rows: fixed-size, contiguous exchange
        pair[:T, 0] = vals
        pair[:T, 1] = ids.to(torch.float32)            # exact only below 2^24: every supported vocabulary is (the fused
        #                                                communicator's kernel carries the ids as raw 32-bit patterns instead)
        dist.all_gather_into_tensor(self._pairs, pair, group=self.group)
        v, i = self._pairs[:, :T, 0], self._pairs[:, :T, 1]
        best = v.max(dim=0, keepdim=True).values
        cand = torch.where(v == best, i, torch.full_like(i, 3.0e38))
        ids.copy_(cand.min(dim=0).values.to(torch.int32))
        vals.copy_(best[0])
        self.stats.argmax_merges += 1

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def check_healthy(self) -> None:
        """Raises if a device-side wait of this communicator ran out (the library path has none)."""

    def recover(self) -> None:
        """Bring the communicator back to a known state after a failed step (drain + host barrier here)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def check_lockstep(self, *ints: int) -> None:
        """All ranks must be making the same call with the same sizes (fingerprint exchange on the host)."""
        # host-side comparison through an object all-gather keeps this off the device stream
        objs = [None] * self.world
        dist.all_gather_object(objs, tuple(ints), group=self.group)
        if any(o != objs[0] for o in objs):
            raise TpDivergenceError(f"ranks disagree on the call fingerprint: {objs}")


class TpDivergenceError(RuntimeError):
    pass


def make_comm(world: int, rank: int, device: str, mode: Optional[str] = None, hidden: int = 5120,
              spin_limit: Optional[int] = None):
    """``mode``: fused (collectives inside the compute kernels), nccl (library collectives between kernels), noop (no
    exchange: timing aid, wrong results).  Emulated ranks on one device come from ``tp_emulated.EmulatedWorld``."""
    mode = mode or os.environ.get("R4DXB_TP_MODE", "fused")
    if world == 1:
        return None
    if mode == "fused":
        from .tp_fused import FusedComm
        kw = {} if spin_limit is None else {"spin_limit": spin_limit}
        return FusedComm(world, rank, device, n=hidden, **kw)
    if mode == "noop":
        from .tp_emulated import NoopComm
        return NoopComm(world, rank, device)
    if mode != "nccl":
        raise ValueError(f"unknown tensor-parallel mode {mode!r}")
    return NcclComm(world, rank, device)


def spin_limit_for_ms(ms: int) -> int:
    """Poll count of a device wait that should give up after about ``ms`` milliseconds: a poll of peer-written memory
    with its back-off sleep takes roughly 100 ns."""
    return max(1 << 12, int(ms) * 10000)
