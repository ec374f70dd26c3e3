"""Single-GPU stand-in for profiling the fused row-parallel product + all-reduce kernel.

A profiler cannot wrap a multi-rank job, so this runs rank 0's kernel of a 2-rank group on one GPU: the "peer's"
receive buffer is a second local buffer, and the pairs the peer would have pushed are written beforehand with the
sequence numbers the kernel will look for, so no wait ever spins.  The kernel does everything it does in a real
group - the weight stream, the split-K reduction over DSMEM, the (value, sequence) pair stores to the peer buffer,
the acquire polls of its own buffer, the rank-ordered sum - only the stores and polls stay on this GPU.

    python -m r4dx_b200.utils.profile_fused_ar [--shape down] [--launches 2]
"""
from __future__ import annotations

import argparse
import ctypes

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="down", choices=["down", "o"])
    ap.add_argument("--launches", type=int, default=2)
    a = ap.parse_args()
    from r4dx_b200 import native
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.parallel import tp_fused  # noqa: F401  (registers the kernel's signature)
    from r4dx_b200.quant import trellis
    dev = "cuda"
    world, N = 2, 5120
    Kd = {"down": 17408 // 2, "o": 6144 // 2}[a.shape]        # rank-local K of a 2-rank group
    w = trellis.random_weight(N, Kd, 4, seed=1, device=dev)
    T = 1
    x = torch.randn(T, 2 * Kd if a.shape == "down" else Kd, device=dev).to(torch.bfloat16)
    res = torch.randn(T, N, device=dev).to(torch.bfloat16)
    slot_pairs = world * 8 * N
    recv = [torch.zeros(2 * slot_pairs, 2, dtype=torch.float32, device=dev) for _ in range(world)]
    # what rank 1 would have pushed into rank 0's buffer: value 0.5 with sequence s, for the calls s = 1 .. launches
    for s in range(1, a.launches + 1):
        seq_bits = torch.tensor([s], dtype=torch.int32).view(torch.float32).item()
        blk = recv[0][(s & 1) * slot_pairs + (1 * 8) * N:(s & 1) * slot_pairs + (1 * 8 + 8) * N]
        blk[:, 0] = 0.5
        blk[:, 1] = seq_bits
    tab = (ctypes.c_void_p * world)(*[r.data_ptr() for r in recv])
    block_seq = torch.zeros(N // 128, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    L = native.cuda()
    ks = K.pick_ksplit(N, Kd)
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    for s in range(a.launches):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = L.r4dxb_trellis_gemv_allreduce(w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(),
                                            res.data_ptr(), K.PRO_SILU_MUL if a.shape == "down" else K.PRO_NONE, T, N, Kd, 4, ks,
                                            tab, block_seq.data_ptr(), status.data_ptr(), world, 0, 1 << 16,
                                            torch.cuda.current_stream().cuda_stream)
        e1.record()
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0, (rc, int(status.item()))
        print(f"fused {a.shape} + all-reduce stand-in, launch {s}: {e0.elapsed_time(e1) * 1e3:.1f} us (N={N}, K={Kd}, ksplit={ks})")


if __name__ == "__main__":
    main()
