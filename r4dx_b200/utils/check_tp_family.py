"""Tensor-parallel self-check of a model family: every rank shards a small synthetic model, runs small-batch rows, a
chunked prefill, single-row steps and a short graph decode, and rank 0 compares the logits with the unsharded model.
Progress is printed stage by stage (flushed), so a run that stops shows where.

    R4DXB_UNVALIDATED_TP=1 python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m r4dx_b200.utils.check_tp_family --family lfm2

Families: ``lfm2`` (short-conv + attention MoE: conv channel blocks, experts sliced by inner width), ``gemma``
(sandwich norms + GeGLU: bare products reduced before the norm), ``hybrid`` (the default dense hybrid).  The first two sit
behind ``R4DXB_UNVALIDATED_TP`` in the model until this check has passed on GPUs."""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="lfm2", choices=["lfm2", "gemma", "hybrid"])
    ap.add_argument("--tolerance", type=float, default=0.06, help="max |logit error| as a fraction of the largest |logit|")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    t0 = time.perf_counter()

    def say(msg: str) -> None:
        print(f"[rank {rank} +{time.perf_counter() - t0:6.1f}s] {msg}", flush=True)

    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    say("process group up")
    from r4dx_b200.config import gemma_config, lfm2_moe_config, small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_comm import make_comm
    from r4dx_b200.quant.weights import moe_kb_rule, synthetic_weight_set
    if a.family == "lfm2":
        gcfg = lfm2_moe_config(hidden=512, layers=4, heads=8, kv_heads=4, head_dim=64, intermediate=1024, experts=8, top_k=2,
                               moe_intermediate=256, dense_layers=1, vocab=8192, attention_layers=(2,))
        full = synthetic_weight_set(gcfg, device=dev, seed=5, sigma=0.05, kb_rule=moe_kb_rule)
        # selection bias two units apart: which experts run does not hinge on rounding (a sigmoid score lives in (0, 1))
        for i in range(gcfg.num_dense_layers, gcfg.num_hidden_layers):
            full[f"text.layers.{i}.moe.expert_bias"] = torch.roll(torch.arange(8, dtype=torch.float32, device=dev) * 2.0, i)
    elif a.family == "gemma":
        gcfg = gemma_config(hidden=512, layers=4, heads=8, kv_heads=4, head_dim=64, intermediate=1024, vocab=8192, window=24)
        gcfg.sliding_global_every = 2
        full = synthetic_weight_set(gcfg, device=dev, seed=5, sigma=0.05)
    else:
        gcfg = small_hybrid_config(layers=4)
        full = synthetic_weight_set(gcfg, device=dev, seed=5, sigma=0.05)
    say(f"synthetic {a.family} weights built")
    comm = make_comm(world, rank, dev, hidden=gcfg.hidden_size)
    cfg = gcfg.shard(world, rank)
    model = HybridModel(cfg, shard_weight_set(gcfg, full, world, rank), max_ctx=256, device=dev, comm=comm)
    say(f"sharded model built ({comm.mode} communicator)")
    V = cfg.vocab_shard_size
    ids = torch.randint(0, gcfg.vocab_size, (41,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    model.feed(ids[:8])
    small = model.buf.logits[:8].float().clone()
    torch.cuda.synchronize()
    say("8 rows through the small-batch path")
    model.reset()
    model.prefill(ids[:40], chunk=32)
    torch.cuda.synchronize()
    say("chunked prefill of 40 tokens")
    step = model.decode_step_logits(int(ids[40])).float().clone()
    torch.cuda.synchronize()
    say("one single-row step")
    model.reset()
    toks = model.generate_greedy(ids, 6, use_graph=True)
    torch.cuda.synchronize()
    say(f"graph decode: {toks}")
    if hasattr(comm, "check_healthy"):
        comm.check_healthy()
    gathered = [None] * world
    dist.all_gather_object(gathered, toks)
    ok = all(g == gathered[0] for g in gathered)
    if not ok:
        say(f"FAIL: ranks disagree on the decoded tokens: {gathered}")
    if rank == 0:
        ref = HybridModel(gcfg, full, max_ctx=256, device=dev)
        ref.feed(ids[:8])
        rs = ref.buf.logits[:8, :V].float()
        e1 = (small - rs).abs().max().item() / rs.abs().max().item()
        ref.reset()
        ref.prefill(ids[:40], chunk=32)
        rstep = ref.decode_step_logits(int(ids[40])).float()[:V]
        e2 = (step - rstep).abs().max().item() / rstep.abs().max().item()
        say(f"logit error vs the unsharded model: small-batch {e1:.4f}, prefill + step {e2:.4f} (tolerance {a.tolerance})")
        ok = ok and e1 < a.tolerance and e2 < a.tolerance
        print("TP_FAMILY_OK" if ok else "TP_FAMILY_FAIL", a.family, flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
