"""Times the tensor-parallel prefill kernels of one rank on ONE GPU, with every peer's buffers in local memory.

    python -m r4dx_b200.utils.profile_fused_prefill --world 8 --rows 2048

The row-parallel GEMM with the reduce-scatter in its epilogue (``r4dxb_trellis_gemm_rs``), the owner-side
reduce + all-gather push (``r4dxb_tp_reduce_push``) and the wait kernel run here for all ``world`` ranks of a down
projection, one rank after the other on one stream: rank r's GEMM stores its partial rows into the "peers'" receive
buffers (all of them local allocations) and bumps their counters; once all ranks' GEMMs have run, every counter has its
full count, so no kernel of this script ever waits for a kernel that has not finished.  Each rank multiplies its own K
slice of one activation matrix, so the gathered result must equal the unsharded product: the script checks that, then
times rank 0's three kernels with CUDA events (the stores go to HBM instead of NVLink: the times are the kernels' cost
without the link) and brackets one more round with cudaProfilerStart/Stop for a profiler.
"""
from __future__ import annotations

import argparse
import ctypes

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--inner", type=int, default=17408, help="unsharded K of the row-parallel product")
    ap.add_argument("--kb", type=int, default=4)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from r4dx_b200 import native
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.parallel import tp_fused  # noqa: F401  (registers the C signatures of the prefill kernels)
    from r4dx_b200.quant import trellis
    L = native.cuda()
    dev = "cuda"
    W, T, H = a.world, a.rows, a.hidden
    Ks = a.inner // W // 128 * 128
    rpr = (T + W - 1) // W
    tn = K.pick_token_tile(T, H)
    ws = [trellis.random_weight(H, Ks, a.kb, seed=r, sigma=0.02, device=dev) for r in range(W)]
    g = torch.Generator(device=dev).manual_seed(0)
    act = (torch.randn(T, Ks * W, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    res = (torch.randn(T, H, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    # per-rank buffers, all local: residual stream copy, receive buffer [W][rpr][H], arrival counter, pushed-rows counter
    xs = [res.clone() for _ in range(W)]
    recv = [torch.zeros(W, rpr, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    cnt = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(W)]
    xflag = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(W)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tab = lambda ts: (ctypes.c_void_p * W)(*[t.data_ptr() for t in ts])
    t_x, t_recv, t_cnt, t_xflag = tab(xs), tab(recv), tab(cnt), tab(xflag)
    xh = [K.trellis_input(act[:, r * Ks:(r + 1) * Ks].contiguous(), ws[r].suh) for r in range(W)]
    st = torch.cuda.current_stream().cuda_stream
    spin = 1 << 16
    rounds = 0

    def gemm(r):
        rc = L.r4dxb_trellis_gemm_rs(ws[r].words.data_ptr(), ws[r].svh.data_ptr(), xh[r].data_ptr(), T, H, Ks, a.kb, tn,
                                     K.gemm_status(dev).data_ptr(), t_recv, t_cnt, W, r, rpr, st)
        assert rc == 0, rc

    def targets(r):
        lo, hi = r * rpr, min(T, (r + 1) * rpr)
        tiles = 0 if hi <= lo else (hi - 1) // tn - lo // tn + 1
        return max(0, hi - lo), W * (H // 128) * tiles

    def push(r):
        own, per_round = targets(r)
        rc = L.r4dxb_tp_reduce_push(t_x, t_xflag, recv[r].data_ptr(), cnt[r].data_ptr(), (per_round * rounds) & 0xFFFFFFFF, W, r,
                                    rpr, own, H, spin, status.data_ptr(), st)
        assert rc == 0, rc

    def wait(r):
        rc = L.r4dxb_tp_wait(xflag[r].data_ptr(), (T * rounds) & 0xFFFFFFFF, spin, 300 + r, status.data_ptr(), st)
        assert rc == 0, rc

    def round_all():
        nonlocal rounds
        rounds += 1
        for r in range(W):
            gemm(r)
        for r in range(W):
            push(r)
        for r in range(W):
            wait(r)

    # ---- correctness: the gathered rows equal residual + the unsharded product ----
    round_all()
    torch.cuda.synchronize()
    K.check_gemm_status(dev)
    assert int(status.item()) == 0, int(status.item())
    ref = res.float()
    for r in range(W):
        ref = ref + K.trellis_gemm(ws[r], xh[r]).float()
    worst = max((xs[r].float() - ref).abs().max().item() for r in range(W))
    scale = ref.abs().max().item()
    print(f"gathered rows vs unsharded sum: max |d| {worst:.4f} of scale {scale:.3f}; every rank's copy equal: "
          f"{all(torch.equal(xs[0], xs[r]) for r in range(1, W))}")

    # ---- timing of rank 0's kernels (the other ranks' launches run between the timed ones) ----
    ev = lambda: torch.cuda.Event(enable_timing=True)
    tg, tp_, tw = 0.0, 0.0, 0.0
    for _ in range(a.iters):
        for x_ in xs:
            x_.copy_(res)
        rounds += 1
        e = [ev() for _ in range(6)]
        e[0].record(); gemm(0); e[1].record()
        for r in range(1, W):
            gemm(r)
        e[2].record(); push(0); e[3].record()
        for r in range(1, W):
            push(r)
        e[4].record(); wait(0); e[5].record()
        for r in range(1, W):
            wait(r)
        torch.cuda.synchronize()
        tg += e[0].elapsed_time(e[1]); tp_ += e[2].elapsed_time(e[3]); tw += e[4].elapsed_time(e[5])
    n = a.iters
    flops = 2.0 * T * H * Ks
    print(f"world {W}, T {T}, H {H}, K/W {Ks}, kb {a.kb}, tile {tn}")
    print(f"  gemm + reduce-scatter stores: {tg / n * 1e3:.1f} us ({flops / (tg / n * 1e-3) / 1e12:.0f} TFLOP/s)")
    print(f"  reduce + push ({targets(0)[0]} rows): {tp_ / n * 1e3:.1f} us "
          f"({(W + 1 + W) * targets(0)[0] * H * 2 / (tp_ / n * 1e-3) / 1e9:.0f} GB/s of row traffic)")
    print(f"  wait kernel: {tw / n * 1e3:.1f} us")
    assert int(status.item()) == 0

    torch.cuda.profiler.start()
    for x_ in xs:
        x_.copy_(res)
    round_all()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


if __name__ == "__main__":
    main()
