"""Communicators that need no second GPU: N emulated ranks on one device, and a no-op.

``EmulatedWorld`` runs N ranks of a tensor-parallel model as N Python threads of one process on ONE device.
A collective is a host-side rendezvous: every rank launches its local product on the shared stream, the
threads meet at a barrier, and each rank then sums all ranks' partials in rank order (stream order makes the
partials visible: they were all enqueued before any sum).  No kernel ever waits for another kernel, so nothing
here depends on two launches being co-resident on the device.  What this exercises is everything around the
wire: the sharding of every tensor for 2 / 4 / 8 ranks (KV-head replication included), the per-rank call
sequence, the vocabulary-parallel pick.  The device protocol of the fused kernels is covered separately (scripted
peer on one GPU, real peers on several).

``NoopComm`` skips the exchange altogether: every rank keeps its own partial.  Results are wrong by
construction; it exists to time a rank's kernels without any communication in the way.

(reference: src/model/tp/tp_comm_emulated.cpp:1-40,74 and src/model/tp/tp_comm_noop.cpp serve the same two
purposes; there the emulated ranks are threads of the engine process as well.)
"""
from __future__ import annotations

import threading
from typing import Callable, List

import torch

from ..ops import kernels as K
from .tp_comm import NcclComm

BF = torch.bfloat16


class EmulatedWorld:
    def __init__(self, world: int, device: str = "cuda:0"):
        self.world, self.device = world, device
        self._barrier = threading.Barrier(world)
        self._slots: List[object] = [None] * world

    def comm(self, rank: int) -> "EmulatedComm":
        return EmulatedComm(self, rank)

    def exchange(self, rank: int, payload):
        """Every rank's payload, in rank order (two barrier phases: publish, read)."""
        self._slots[rank] = payload
        self._barrier.wait(timeout=120)
        got = list(self._slots)
        self._barrier.wait(timeout=120)
        return got

    def run(self, fn: Callable[[int, "EmulatedComm"], object]) -> list:
        """Runs ``fn(rank, comm)`` on one thread per rank; returns the results in rank order, re-raising the first error."""
        out: List[object] = [None] * self.world
        err: List[BaseException] = []

        def body(r):
            try:
                torch.cuda.set_device(torch.device(self.device))
                out[r] = fn(r, self.comm(r))
            except BaseException as e:       # noqa: BLE001
                err.append(e)
                self._barrier.abort()         # the other ranks must not wait for a rank that is gone

        th = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for t in th:
            t.start()
        for t in th:
            t.join()
        if err:
            first = next((e for e in err if not isinstance(e, threading.BrokenBarrierError)), err[0])
            raise first
        return out


class EmulatedComm(NcclComm):
    mode = "emulate"

    def __init__(self, world: EmulatedWorld, rank: int):
        super().__init__(world.world, rank, world.device, None)
        self.w = world

    def _sum_into(self, mine: torch.Tensor, out: torch.Tensor, add_to_out: bool) -> None:
        parts = self.w.exchange(self.rank, mine)
        acc = parts[0].float()
        for p in parts[1:]:                   # rank order, identical on every rank
            acc = acc + p.float()
        if add_to_out:
            acc = acc + out.float()
        out.copy_(acc.to(out.dtype))
        self.w.exchange(self.rank, None)      # nobody overwrites its partial before every rank has read it
        self.stats.all_reduces += 1
        self.stats.all_reduce_bytes += mine.numel() * 2

    def row_parallel_linear(self, lin, x: torch.Tensor, res: torch.Tensor, prologue: int = 0) -> None:
        tmp = self._scratch(res.shape, BF)
        lin(x, out=tmp, prologue=prologue)
        self._sum_into(tmp, res, True)

    def row_parallel_chunk(self, lin, inp: torch.Tensor, x: torch.Tensor, cb: dict, fused_silu_mul: bool = False) -> None:
        tmp = self._scratch(x.shape, BF)
        lin.chunk(inp, cb["xh"], tmp, fused_silu_mul=fused_silu_mul)
        self._sum_into(tmp, x, True)

    def all_reduce_rows(self, t: torch.Tensor) -> None:
        self._sum_into(t.clone(), t, False)

    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        got = self.w.exchange(self.rank, (ids.clone(), vals.clone()))
        v = torch.stack([g[1] for g in got])              # [world, T]
        i = torch.stack([g[0] for g in got])
        best = v.max(dim=0, keepdim=True).values
        cand = torch.where(v == best, i, torch.full_like(i, 2**31 - 1))
        ids.copy_(cand.min(dim=0).values)
        vals.copy_(best[0])
        self.w.exchange(self.rank, None)
        self.stats.argmax_merges += 1

    def barrier(self) -> None:
        self.w.exchange(self.rank, None)

    def recover(self) -> None:
        torch.cuda.synchronize(self.device)

    def check_lockstep(self, *ints: int) -> None:
        got = self.w.exchange(self.rank, tuple(ints))
        if any(g != got[0] for g in got):
            from .tp_comm import TpDivergenceError
            raise TpDivergenceError(f"ranks disagree on the call fingerprint: {got}")


class NoopComm(NcclComm):
    """No exchange at all: every rank keeps its own partial sums (timing aid, wrong results by design)."""

    mode = "noop"

    def row_parallel_linear(self, lin, x: torch.Tensor, res: torch.Tensor, prologue: int = 0) -> None:
        lin(x, out=res, residual=res, prologue=prologue)

    def row_parallel_chunk(self, lin, inp: torch.Tensor, x: torch.Tensor, cb: dict, fused_silu_mul: bool = False) -> None:
        lin.chunk(inp, cb["xh"], x, residual=x, fused_silu_mul=fused_silu_mul)

    def all_reduce_rows(self, t: torch.Tensor) -> None:
        pass

    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        pass

    def barrier(self) -> None:
        pass

    def recover(self) -> None:
        torch.cuda.synchronize(self.device)

    def check_lockstep(self, *ints: int) -> None:
        pass
