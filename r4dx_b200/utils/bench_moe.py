"""MoE layer benchmark at the hybrid-MoE geometry (hidden 2048, 512 experts, top-10, intermediate 512):
one decode step's MoE block for ``--tokens`` concurrent requests spread over the ranks, fused in-kernel
all-to-all vs the NCCL baseline.  Device-timed with CUDA events, max over ranks.

    python -m torch.distributed.run --nproc-per-node 8 -m r4dx_b200.utils.bench_moe --tokens 64
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--layers", type=int, default=4, help="distinct layers cycled through so weights do not sit in L2")
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    from r4dx_b200.config import qwen_hybrid_moe_config
    from r4dx_b200.models.moe import MoeBlock
    from r4dx_b200.parallel.ep import EpComm, NcclEpBaseline
    from r4dx_b200.quant.weights import moe_kb_rule, synthetic_weight_set
    cfg = qwen_hybrid_moe_config(a.layers)
    e_per = cfg.num_experts // world
    w = synthetic_weight_set(cfg, device=dev, seed=0, kb_rule=moe_kb_rule, expert_range=(rank * e_per, e_per))
    T = a.tokens // world
    blocks = [MoeBlock(cfg, w, i, dev, max(T, 8), rank * e_per, e_per) for i in range(a.layers)]
    g = torch.Generator(device=dev).manual_seed(rank)
    h = torch.randn(T, cfg.hidden_size, device=dev, generator=g).to(torch.bfloat16)
    x = torch.zeros(T, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
    out = {}
    for name, cls in (("fused", EpComm), ("nccl", NcclEpBaseline)):
        ep = cls(world, rank, dev, cfg, max_rows=max(T, 8))
        for i in range(6):
            ep.moe_forward(blocks[i % a.layers], h, x, T)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.iters):
            ep.moe_forward(blocks[i % a.layers], h, x, T)
        e1.record()
        torch.cuda.synchronize()
        ep.check_healthy()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name + "_us_per_layer"] = float(t[0]) * 1e3
    if rank == 0:
        pairs = a.tokens * cfg.num_experts_per_tok
        # bytes that must cross NVLink per rank per layer: its tokens' rows out and the expert outputs back, (W-1)/W remote
        nv = 2 * (pairs / world) * cfg.hidden_size * 2 * (world - 1) / max(world, 1)
        out.update({"tokens": a.tokens, "world": world, "pairs": pairs, "nvlink_bytes_per_rank": nv,
                    "nvlink_floor_us_at_770GBs": nv / 770e9 * 1e6,
                    "expert_bytes_per_rank": blocks[0].gate_up.nbytes + blocks[0].down.nbytes})
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
