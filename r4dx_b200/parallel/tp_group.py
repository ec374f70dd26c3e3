"""Rank-group control plane: one process per GPU, a leader that broadcasts commands, lockstep checks,
result comparison, a progress watchdog, host-side fault injection and recovery.

All of it runs on the host (gloo / TCP store), never on the device stream, so it is testable with CPU
ranks; the device side contributes only status words that the fused kernels set when a bounded wait runs
out.  State machine and error types follow the reference's (reference: docs/tp.md:263-346,
src/core/include/r4dx/core/tp_comm.hpp:24-41, src/model/tp/tp_rank_worker.h:219-296,
src/model/tp_model.h:317-351); threads became processes, the host mailbox became a store.
"""
from __future__ import annotations

import enum
import os
import threading
import time
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Sequence

import torch.distributed as dist


class TpAborted(RuntimeError): pass
class TpTimeout(RuntimeError): pass
class TpDivergence(RuntimeError): pass
class TpStateError(RuntimeError): pass


class TpState(enum.Enum):
    READY = "ready"
    NEEDS_RECOVERY = "needs_recovery"
    FATAL = "fatal"


def fnv1a(tokens: Sequence[int]) -> int:
    h = 0xcbf29ce484222325
    for t in tokens:
        for b in int(t).to_bytes(4, "little", signed=True):
            h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h


@dataclass
class FaultSpec:
    """``rank:n:kind`` -- on `rank`, at the n-th collective command: throw | stall | exit."""
    rank: int = -1
    at: int = -1
    kind: str = ""

    @staticmethod
    def parse(text: str) -> "FaultSpec":
        if not text:
            return FaultSpec()
        r, n, k = text.split(":")
        if k not in ("throw", "stall", "exit"):
            raise ValueError(f"unknown fault kind {k}")
        return FaultSpec(int(r), int(n), k)


class RankGroup:
    """Host-side group of ``world`` ranks over a gloo process group."""

    def __init__(self, rank: int, world: int, group=None, timeout_s: float = 30.0, fault: Optional[FaultSpec] = None,
                 stall_s: float = 0.7, clock: Callable[[], float] = time.monotonic):
        self.rank, self.world, self.group = rank, world, group
        self.timeout_s = timeout_s
        self.state = TpState.READY
        self.fault = fault or FaultSpec.parse(os.environ.get("R4DXB_TP_FAULT", ""))
        self.stall_s = stall_s
        self.commands = 0
        self.clock = clock
        self.heartbeat = clock()
        self.stats = {"commands": 0, "lockstep_checks": 0, "recoveries": 0}
        self.last_error: Optional[str] = None

    # ---- state ----
    def require_ready(self) -> None:
        if self.state is TpState.NEEDS_RECOVERY:
            raise TpStateError("the group needs recovery: call reset() first")
        if self.state is TpState.FATAL:
            raise TpStateError(f"the group is in a fatal state ({self.last_error}); restart the process")

    # ---- collectives on the host ----
    def all_gather(self, obj: Any) -> List[Any]:
        out = [None] * self.world
        try:
            dist.all_gather_object(out, obj, group=self.group)
        except Exception as e:                      # a peer went away or the group timed out
            self.state = TpState.FATAL
            self.last_error = f"host all-gather failed: {e}"
            raise TpTimeout(self.last_error) from e
        return out

    def check_lockstep(self, kind: str, rows: int, pos: int, tokens: Sequence[int]) -> None:
        """Every rank must be about to run the same call on the same tokens."""
        fp = (kind, rows, pos, fnv1a(tokens))
        self.stats["lockstep_checks"] += 1
        got = self.all_gather(fp)
        if any(g != got[0] for g in got):
            self.state = TpState.NEEDS_RECOVERY
            self.last_error = f"lockstep fingerprints differ: {got}"
            raise TpDivergence(self.last_error)

    def require_all_equal(self, value: Any, what: str = "result") -> Any:
        got = self.all_gather(value)
        if any(g != got[0] for g in got):
            self.state = TpState.NEEDS_RECOVERY
            self.last_error = f"{what} differs across ranks: {got}"
            raise TpDivergence(self.last_error)
        return got[0]

    # ---- commands ----
    def run_collective(self, fn: Callable[[], Any], kind: str = "cmd", rows: int = 0, pos: int = 0,
                       tokens: Sequence[int] = ()) -> Any:
        """Runs ``fn`` on every rank (each rank calls this with the same arguments).  A failure anywhere leaves
        every rank in NEEDS_RECOVERY and re-raises the root cause with its type on the rank that had it,
        TpAborted on the others."""
        self.require_ready()
        self.check_lockstep(kind, rows, pos, tokens)
        self.commands += 1
        self.stats["commands"] += 1
        err: Optional[BaseException] = None
        result = None
        try:
            self._maybe_fault()
            result = fn()
        except BaseException as e:                  # noqa: BLE001 -- reported to the group below
            err = e
        self.heartbeat = self.clock()
        flags = self.all_gather(None if err is None else f"{type(err).__name__}: {err}")
        if any(f is not None for f in flags):
            self.state = TpState.NEEDS_RECOVERY
            first = next(i for i, f in enumerate(flags) if f is not None)
            self.last_error = f"rank {first}: {flags[first]}"
            if err is not None:
                raise err
            raise TpAborted(self.last_error)
        return result

    def _maybe_fault(self) -> None:
        f = self.fault
        if f.rank == self.rank and f.at == self.commands - 1:      # n counts commands from 0
            self.fault = FaultSpec()                                # one shot: the count restarts after a recovery
            if f.kind == "throw":
                raise RuntimeError("injected fault (throw before enqueue)")
            if f.kind == "stall":
                time.sleep(self.stall_s)
            if f.kind == "exit":
                os._exit(17)

    # ---- recovery ----
    def recover(self, reset_fn: Optional[Callable[[], None]] = None, self_test: Optional[Callable[[], Any]] = None) -> None:
        """Drain, reset device-side counters / status through ``reset_fn``, re-check lockstep, self-test."""
        if self.state is TpState.FATAL:
            raise TpStateError("fatal state: restart the process")
        self.all_gather("recover")                  # rendezvous; raises TpTimeout (-> FATAL) if a rank is gone
        if reset_fn is not None:
            reset_fn()
        self.commands = 0
        self.state = TpState.READY
        self.check_lockstep("recover", 0, 0, ())
        if self_test is not None:
            self.require_all_equal(self_test(), "self-test")
        self.stats["recoveries"] += 1
        self.last_error = None

    def stats_line(self) -> str:
        return (f"[r4dxb-tp] rank {self.rank}/{self.world} state={self.state.value} commands={self.stats['commands']} "
                f"lockstep={self.stats['lockstep_checks']} recoveries={self.stats['recoveries']}")


class ProgressWatchdog:
    """Declares the group fatal when the heartbeat has not moved for ``limit_s`` (injectable clock)."""

    def __init__(self, group: RankGroup, limit_s: float = 60.0, clock: Callable[[], float] = time.monotonic):
        self.group, self.limit_s, self.clock = group, limit_s, clock

    def check(self, busy: bool) -> bool:
        if busy and self.clock() - self.group.heartbeat > self.limit_s:
            self.group.state = TpState.FATAL
            self.group.last_error = f"no progress for {self.limit_s} s"
            return False
        return True
