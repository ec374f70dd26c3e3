"""Soak test of the fused row-parallel product + all-reduce kernel: many back-to-back calls with changing inputs,
every rank folding its results into a running checksum; the checksums must agree bit for bit across ranks (the
kernel sums in rank order on every rank) and a sample of calls is checked against an NCCL all-reduce of the same
partial products (reference: docs/tp.md:94 reports 12.28 M bit-exact all-reduces for the reference's mailbox path).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m r4dx_b200.utils.stress_allreduce --calls 300000
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--calls", type=int, default=100000)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--k", type=int, default=1024, help="rank-local K")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--check-every", type=int, default=5000)
    a = ap.parse_args()
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from r4dx_b200.models.hybrid import Linear
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.parallel.tp_fused import FusedComm
    from r4dx_b200.quant import trellis
    comm = FusedComm(world, rank, dev, n=a.hidden)
    lin = Linear(trellis.random_weight(a.hidden, a.k, 4, seed=100 + rank, device=dev), "stress")
    T = a.rows
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    xs = torch.randn(64, T, a.k, device=dev, generator=g).to(torch.bfloat16)         # a pool of inputs, cycled
    res = torch.zeros(T, a.hidden, dtype=torch.bfloat16, device=dev)
    check = torch.zeros(1, dtype=torch.int64, device=dev)
    mism = 0
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.time()
    for i in range(a.calls):
        res.zero_()
        comm.row_parallel_linear(lin, xs[i % 64], res)
        # fold the result's bits into the checksum (order-sensitive)
        check.mul_(1000003).add_(res.view(torch.int16).to(torch.int64).sum())
        if (i + 1) % a.check_every == 0:
            part = K.trellis_gemv(lin.w, xs[i % 64]).float()
            dist.all_reduce(part)
            err = (part - res.float()).abs().max().item()
            tol = 0.02 * part.abs().max().item() + 1e-3
            mism += int(err > tol)
            comm.check_healthy()
    torch.cuda.synchronize()
    dt = time.time() - t0
    sums = [torch.zeros_like(check) for _ in range(world)]
    dist.all_gather(sums, check)
    same = all(int(s.item()) == int(sums[0].item()) for s in sums)
    if rank == 0:
        print(json.dumps({"calls": a.calls, "world": world, "rows": T, "hidden": a.hidden, "k_local": a.k, "seconds": dt,
                          "calls_per_second": a.calls / dt, "checksums_equal_across_ranks": same,
                          "sampled_mismatches_vs_nccl": mism, "status": int(comm.status.item())}))
    assert same and mism == 0
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
