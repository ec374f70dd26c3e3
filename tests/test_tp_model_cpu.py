"""The tensor-parallel model facade with CPU ranks (gloo) and the host-only stand-in model: the leader serves
requests through the ordinary engine, followers run the command loop; faults are made on the host only."""
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
    from r4dx_b200.parallel.tp_group import FaultSpec, RankGroup
    from r4dx_b200.runtime.sampler import SampleParams
    from r4dx_b200.runtime.text_model import FakeTextModel
    from r4dx_b200.runtime.tokenizer import ByteTokenizer
    from r4dx_b200.runtime.tp_model import TpTextModel
    from r4dx_b200.server.engine import Engine, EngineFatal, GenRequest
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    fault = {"throw": "1:4:throw", "exit": "1:4:exit"}.get(scenario, "")
    group = RankGroup(rank, world, fault=FaultSpec.parse(fault))
    tm = TpTextModel(FakeTextModel(vocab=64), group)
    out = {}
    if rank != 0:
        tm.follow()
        out["state"] = group.state.value
        q.put((rank, out))
        return
    eng = Engine(tm, ByteTokenizer(300))
    try:
        def gen(params=None):
            return eng.generate(GenRequest(prompt_ids=[5, 9, 11], max_tokens=10, params=params or SampleParams(temperature=0.0)), timeout=30)
        if scenario == "ok":
            solo = Engine(FakeTextModel(vocab=64), ByteTokenizer(300))
            want = solo.generate(GenRequest(prompt_ids=[5, 9, 11], max_tokens=10, params=SampleParams(temperature=0.0)), timeout=30)
            want_s = solo.generate(GenRequest(prompt_ids=[5, 9, 11], max_tokens=10, params=SampleParams(temperature=0.9, seed=5)), timeout=30)
            solo.shutdown()
            r = gen()
            rs = gen(SampleParams(temperature=0.9, seed=5))
            out.update(error=r.error, same=r.token_ids == want.token_ids, same_sampled=rs.token_ids == want_s.token_ids,
                       commands=group.stats["commands"], lockstep=group.stats["lockstep_checks"])
        elif scenario == "throw":
            r1 = gen()                      # rank 1 raises at its fifth command: the request fails on every rank
            r2 = gen()                      # the next request starts with reset(): recovery, then it is served
            out.update(first_error=r1.error, second_error=r2.error, second_len=len(r2.token_ids),
                       recoveries=group.stats["recoveries"], fatal=eng.fatal)
        elif scenario == "exit":
            r1 = gen()                      # rank 1 leaves between steps: the host exchange fails, the group is fatal
            try:
                eng.submit(GenRequest(prompt_ids=[1], max_tokens=2))
                refused = False
            except EngineFatal:
                refused = True
            out.update(first_error=r1.error, refused=refused, fatal=eng.fatal, state=group.state.value)
    finally:
        eng.shutdown()
        tm.shutdown()
    q.put((rank, out))


def _run(scenario, world=3):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in ps:
        p.start()
    got = {}
    try:
        for _ in range(world if scenario != "exit" else world - 1):
            r, out = q.get(timeout=90)
            got[r] = out
    finally:
        for p in ps:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    return got


def test_leader_serves_through_the_engine_and_followers_replay_every_command():
    got = _run("ok")
    lead = got[0]
    assert lead["error"] is None and lead["same"] and lead["same_sampled"]
    assert lead["commands"] > 10 and lead["lockstep"] >= lead["commands"]
    assert all(got[r]["state"] == "ready" for r in (1, 2))


def test_a_rank_that_raises_fails_the_request_everywhere_and_the_next_request_recovers():
    got = _run("throw")
    lead = got[0]
    assert lead["first_error"] and "TpAborted" in lead["first_error"]
    assert lead["second_error"] is None and lead["second_len"] == 10
    assert lead["recoveries"] == 1 and lead["fatal"] is None


def test_a_rank_that_leaves_makes_the_group_fatal_and_the_engine_refuses_new_work():
    got = _run("exit")
    lead = got[0]
    assert lead["first_error"] is not None
    assert lead["state"] == "fatal" and lead["refused"] and lead["fatal"]
