"""Rank-group control plane with CPU ranks (gloo): lockstep, divergence, injected faults, recovery, watchdog.
Failures are made on the host only: a rank that raises, stalls or exits between steps."""
import os
import socket
import sys

import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, scenario, q):
    sys.path.insert(0, ROOT)
    import datetime
    import torch.distributed as dist
    from r4dx_b200.parallel.tp_group import (FaultSpec, RankGroup, TpAborted, TpDivergence, TpState, TpStateError, TpTimeout)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=6))
    out = {}
    try:
        if scenario == "ok":
            g = RankGroup(rank, world)
            r = g.run_collective(lambda: 41 + 1, "decode", 1, 5, [7])
            out["result"] = g.require_all_equal(r)
            out["state"] = g.state.value
        elif scenario == "divergence":
            g = RankGroup(rank, world)
            try:
                g.check_lockstep("decode", 1, 5, [7 if rank == 0 else 8])
                out["raised"] = False
            except TpDivergence:
                out["raised"] = True
            out["state"] = g.state.value
            try:
                g.run_collective(lambda: 0)
                out["blocked"] = False
            except TpStateError:
                out["blocked"] = True
            g.recover(self_test=lambda: 123)
            out["after"] = g.state.value
        elif scenario == "throw":
            g = RankGroup(rank, world, fault=FaultSpec.parse("1:1:throw"))
            g.run_collective(lambda: 0)
            try:
                g.run_collective(lambda: 0)
                out["err"] = None
            except TpAborted as e:
                out["err"] = "aborted"
            except RuntimeError as e:
                out["err"] = "root:" + str(e)
            out["state"] = g.state.value
            g.recover()
            out["ok_after"] = g.run_collective(lambda: 5)
        elif scenario == "exit":
            g = RankGroup(rank, world, fault=FaultSpec.parse("1:1:exit"))
            g.run_collective(lambda: 0)
            try:
                g.run_collective(lambda: 0)
                out["err"] = None
            except TpTimeout:
                out["err"] = "timeout"
            out["state"] = g.state.value
    finally:
        q.put((rank, out))


def _run(world, scenario):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = {}
    alive = world - (1 if scenario == "exit" else 0)
    for _ in range(alive):
        r, o = q.get(timeout=60)
        res[r] = o
    for p in ps:
        p.join(timeout=20)
    return res


def test_commands_run_in_lockstep():
    res = _run(2, "ok")
    assert all(o == {"result": 42, "state": "ready"} for o in res.values())


def test_divergence_blocks_until_recovered():
    res = _run(2, "divergence")
    for o in res.values():
        assert o["raised"] and o["state"] == "needs_recovery" and o["blocked"] and o["after"] == "ready"


def test_injected_throw_reaches_every_rank_with_its_type_on_the_faulty_one():
    res = _run(3, "throw")
    assert res[1]["err"].startswith("root:injected fault")
    assert res[0]["err"] == "aborted" and res[2]["err"] == "aborted"
    assert all(o["state"] == "needs_recovery" and o["ok_after"] == 5 for o in res.values())


def test_rank_that_exits_between_steps_makes_the_rest_fatal():
    res = _run(2, "exit")
    assert res[0]["err"] == "timeout" and res[0]["state"] == "fatal"


def test_watchdog_with_a_fake_clock():
    sys.path.insert(0, ROOT)
    from r4dx_b200.parallel.tp_group import ProgressWatchdog, RankGroup, TpState, fnv1a
    now = [0.0]
    g = RankGroup(0, 1, clock=lambda: now[0])
    w = ProgressWatchdog(g, limit_s=60, clock=lambda: now[0])
    now[0] = 59.0
    assert w.check(busy=True)
    now[0] = 61.0
    assert w.check(busy=False) and g.state is TpState.READY
    assert not w.check(busy=True) and g.state is TpState.FATAL
    assert fnv1a([1, 2, 3]) != fnv1a([1, 2, 4])
