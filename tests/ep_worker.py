"""Child of tests/test_tp_gpu.py: one rank of an expert-parallel MoE layer (tokens and experts sharded)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from r4dx_b200.config import tiny_moe_config
    from r4dx_b200.models.moe import MoeBlock
    from r4dx_b200.models.oracle import init_weights
    from r4dx_b200.parallel.ep import EpComm, NcclEpBaseline
    from r4dx_b200.quant.weights import moe_kb_rule, quantize_weight_set
    cfg = tiny_moe_config()
    q = quantize_weight_set(cfg, init_weights(cfg, 0), kb_rule=moe_kb_rule)
    q = {k: (v.to(dev) if hasattr(v, "to") else v) for k, v in q.items()}
    full = MoeBlock(cfg, q, 0, dev, 8)
    e_per = cfg.num_experts // world
    mine = MoeBlock(cfg, q, 0, dev, 8, rank * e_per, e_per)
    for cls in (EpComm, NcclEpBaseline):
        ep = cls(world, rank, dev, cfg, max_rows=8, spin_limit=1 << 21)
        g = torch.Generator().manual_seed(100 + rank)
        for it in range(4):
            # ragged token counts per rank only on the fused path: the library all-gather needs equal shapes
            T = 8 if (it != 2 or cls is NcclEpBaseline) else 3 + rank
            h = torch.randn(T, cfg.hidden_size, generator=g).to(torch.bfloat16).to(dev)
            x0 = torch.randn(T, cfg.hidden_size, generator=g).to(torch.bfloat16).to(dev)
            xa, xb = x0.clone(), x0.clone()
            full.forward(h, xa, T)
            ep.moe_forward(mine, h, xb, T)
            torch.cuda.synchronize()
            ep.check_healthy()
            err = (xa.float() - xb.float()).abs().max().item()
            tol = 0.0 if cls is EpComm else 0.05
            assert err <= tol, (cls.__name__, it, err)
        dist.barrier()
    if rank == 0:
        print("EP_OK", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
