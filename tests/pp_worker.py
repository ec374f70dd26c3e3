"""Child of tests/test_tp_gpu.py: PP=2 prefill over NCCL p2p, then reshard into TP=2 decode (hybrid mode)."""
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
    from r4dx_b200.config import small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.pp import LayerSplitDecode, PipelinePrefill, reshard_to_tp
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_comm import make_comm
    from r4dx_b200.quant.weights import synthetic_weight_set
    gcfg = small_hybrid_config(layers=4)
    full = synthetic_weight_set(gcfg, device=dev, seed=3, sigma=0.05)
    split = 2
    rng = (0, split) if rank == 0 else (split, 4)
    stage = HybridModel(gcfg, full, max_ctx=512, device=dev, layer_range=rng)
    ids = torch.randint(0, gcfg.vocab_size, (150,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    pp = PipelinePrefill(stage, rank, split, chunk=64)
    tok = pp.prefill(ids)
    # reference: the whole model on one GPU
    ref = HybridModel(gcfg, full, max_ctx=512, device=dev)
    rtok = ref.prefill(ids, chunk=64)
    assert tok == rtok, (tok, rtok)
    # hybrid: reshard into the tensor-parallel layout and decode there
    comm = make_comm(world, rank, dev, hidden=gcfg.hidden_size)
    tp = HybridModel(gcfg.shard(world, rank), shard_weight_set(gcfg, full, world, rank), max_ctx=512, device=dev, comm=comm)
    reshard_to_tp(gcfg, stage, tp, world, rank, {0: 0, 1: 0, 2: 1, 3: 1})
    out_tp = [tok]
    for _ in range(8):
        out_tp.append(tp.decode_step_greedy(out_tp[-1]))
    out_ref = [rtok]
    for _ in range(8):
        out_ref.append(ref.decode_step_greedy(out_ref[-1]))
    # layer-split decode on the two stages, continuing from the pipelined prefill: same kernels, no sharding, so the
    # tokens equal the single-GPU model's exactly
    ls = LayerSplitDecode(stage, rank)
    out_ls = [tok]
    for _ in range(8):
        out_ls.append(ls.step(out_ls[-1]))
    assert out_ls == out_ref, (out_ls, out_ref)
    same = sum(int(a == b) for a, b in zip(out_tp, out_ref))
    if rank == 0:
        print("pp+reshard tokens", out_tp, "ref", out_ref, flush=True)
    assert same >= 7, (out_tp, out_ref)
    dist.barrier()
    if rank == 0:
        print("PP_OK", flush=True)
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
