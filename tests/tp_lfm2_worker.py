"""Child of tests/test_tp_gpu.py: one rank of a tensor-parallel run of a small short-conv + attention MoE model.

Conv mixers are split by channel block, experts by inner width (every rank holds a slice of every expert); rank 0 also runs
the unsharded model and compares logits.  The selection bias is spread two units apart so that the routing does not hinge
on rounding (a sigmoid score lives in (0, 1)); token-dependent selection is compared exactly at the kernel level."""
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
    from r4dx_b200.config import lfm2_moe_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_comm import make_comm
    from r4dx_b200.quant.weights import moe_kb_rule, synthetic_weight_set
    gcfg = lfm2_moe_config(hidden=512, layers=4, heads=8, kv_heads=4, head_dim=64, intermediate=1024, experts=8, top_k=2,
                           moe_intermediate=256, dense_layers=1, vocab=8192, attention_layers=(2,))
    full = synthetic_weight_set(gcfg, device=dev, seed=5, sigma=0.05, kb_rule=moe_kb_rule)
    for i in range(gcfg.num_dense_layers, gcfg.num_hidden_layers):
        full[f"text.layers.{i}.moe.expert_bias"] = torch.roll(torch.arange(8, dtype=torch.float32, device=dev) * 2.0, i)
    comm = make_comm(world, rank, dev, hidden=gcfg.hidden_size)
    cfg = gcfg.shard(world, rank)
    model = HybridModel(cfg, shard_weight_set(gcfg, full, world, rank), max_ctx=256, device=dev, comm=comm)
    ids = torch.randint(0, gcfg.vocab_size, (41,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    model.feed(ids[:8])
    V = cfg.vocab_shard_size
    small = model.buf.logits[:8].float().clone()
    model.reset()
    model.prefill(ids[:40], chunk=32)                      # one 32-row chunk (tensor-core path) + 8 rows
    step = model.decode_step_logits(int(ids[40])).float().clone()
    model.reset()
    toks = model.generate_greedy(ids, 6, use_graph=True)
    torch.cuda.synchronize()
    if hasattr(comm, "check_healthy"):
        comm.check_healthy()
    gathered = [None] * world
    dist.all_gather_object(gathered, toks)
    assert all(g == gathered[0] for g in gathered), f"ranks disagree: {gathered}"
    if rank == 0:
        ref = HybridModel(gcfg, full, max_ctx=256, device=dev)
        ref.feed(ids[:8])
        rs = ref.buf.logits[:8, :V].float()
        scale = rs.abs().max().item()
        assert (small - rs).abs().max().item() < 0.06 * scale, ((small - rs).abs().max().item(), scale)
        ref.reset()
        ref.prefill(ids[:40], chunk=32)
        rstep = ref.decode_step_logits(int(ids[40])).float()[:V]
        assert (step - rstep).abs().max().item() < 0.06 * rstep.abs().max().item()
        print("TP_LFM2_OK", toks)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
