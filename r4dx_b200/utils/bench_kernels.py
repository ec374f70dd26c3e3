"""Microbenchmarks of the hot kernels at the 27B geometry's shapes.

    python -m r4dx_b200.utils.bench_kernels [--only trellis_gemv] [--shape gate_up] [--rows 1] [--iters 20]

Each kernel is timed with CUDA events after warm-up; a 256 MiB buffer is rewritten between timed
launches so the weights never sit in L2.  Prints algorithmic bytes / time and the fraction of the
measured copy bandwidth (MEASURED_PEAKS.json beside the repository root, else 6650 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

SHAPES_27B = {            # name: (N, K)
    "in_proj_qkv": (10240, 5120), "in_proj_z": (6144, 5120), "out_proj": (5120, 6144),
    "qg": (12288, 5120), "kv": (1024, 5120), "o": (5120, 6144),
    "gate_up": (34816, 5120), "down": (5120, 17408),
}


def _peak_gbs() -> float:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"])
    except Exception:
        return 6650.0


def timed(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters * 1e3      # us


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--shape", default="")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--kb", type=int, default=0)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--decode-warps", type=int, default=0, help="4, 8 or 16; 0 leaves the library's own choice")
    ap.add_argument("--tn", type=int, default=0)
    ap.add_argument("--ksplit", type=int, default=0, help="override the cluster split of the weight-streaming kernel")
    ap.add_argument("--f8", action="store_true", help="with --only trellis_gemm: also time the 8-bit (e4m3 x e4m3) product")
    ap.add_argument("--impl", default="", help="weight-streaming kernel: mma (tensor memory, default) or simt (CUDA cores)")
    a = ap.parse_args()
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.quant import trellis, w4a16
    if a.impl:
        K.set_gemv_impl(a.impl)
    peak = _peak_gbs()
    dev = "cuda"
    flush = torch.zeros(256 << 18, dtype=torch.float32, device=dev)
    T = a.rows
    BF = torch.bfloat16
    if a.only in ("", "trellis_gemv"):
        for name, (N, Kd) in SHAPES_27B.items():
            if a.shape and a.shape != name:
                continue
            for kb in ((a.kb,) if a.kb else (4, 5)):
                w = trellis.random_weight(N, Kd, kb, seed=1, device=dev)
                x = torch.randn(T, Kd, device=dev).to(BF)
                y = torch.empty(T, N, dtype=BF, device=dev)
                ks = a.ksplit or K.pick_ksplit(N, Kd)
                if (Kd // 128) % ks:
                    continue
                us = timed(lambda: K.trellis_gemv(w, x, out=y, ksplit=ks), a.iters, flush)
                gbs = w.nbytes / us / 1e3
                K.check_gemm_status(dev)
                print(f"trellis_gemv[{K.GEMV_IMPL}] {name:12s} N={N:6d} K={Kd:6d} kb={kb} T={T} ksplit={ks}: {us:8.1f} us  "
                      f"{gbs:7.0f} GB/s  {gbs / peak:5.2f} of measured HBM  {N * Kd / us / 1e6:6.2f} Tweights/s")
    if a.only in ("trellis_gemm",):
        Tg = max(a.rows, 16)
        from r4dx_b200 import native
        native.cuda().r4dxb_set_gemm_decode_warps(a.decode_warps)
        tf_peak = 1699.0
        try:
            tf_peak = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            pass
        for name, (N, Kd) in SHAPES_27B.items():
            if a.shape and a.shape != name:
                continue
            for kb in ((a.kb,) if a.kb else (4,)):
                w = trellis.random_weight(N, Kd, kb, seed=1, device=dev)
                x = torch.randn(Tg, Kd, device=dev).to(BF)
                xh = K.trellis_input(x, w.suh)
                y = torch.empty(Tg, N, dtype=BF, device=dev)
                tn = a.tn or K.pick_token_tile(Tg, N)
                us = timed(lambda: K.trellis_gemm(w, xh, out=y, tn=tn), a.iters, flush)
                K.check_gemm_status(dev)
                tf = 2.0 * N * Kd * Tg / us / 1e6
                print(f"trellis_gemm {name:12s} N={N:6d} K={Kd:6d} kb={kb} T={Tg} tn={tn}: {us:9.1f} us  "
                      f"{tf:7.1f} TFLOP/s  {tf / tf_peak:5.2f} of measured cuBLAS bf16")
                if a.f8:
                    xq, sc = K.quantize_rows_e4m3(xh)
                    tn8 = a.tn or (512 if Tg > 256 else 256)
                    us8 = timed(lambda: K.trellis_gemm_f8(w, xq, sc, out=y, tn=tn8), a.iters, flush)
                    usq = timed(lambda: K.quantize_rows_e4m3(xh, xq, sc), a.iters, flush)
                    K.check_gemm_status(dev)
                    tf8 = 2.0 * N * Kd * Tg / us8 / 1e6
                    print(f"trellis_gemm_f8 {name:9s} N={N:6d} K={Kd:6d} kb={kb} T={Tg} tn={tn8}: {us8:9.1f} us  "
                          f"{tf8:7.1f} TFLOP/s effective  {tf8 / tf_peak:5.2f} of measured cuBLAS bf16  (+ {usq:.1f} us row quantizer)")
    if a.only in ("linear_tc",):
        # plain tensor-core linear: the w4a16 head over a wide batch, a w4a16 drafter product, dense vision-tower products
        Tg = max(a.rows, 16)
        for label, N, Kd, kind in (("head w4a16", 248320, 5120, "w4"), ("drafter gate_up w4a16", 27648, 5120, "w4"),
                                   ("vision qkv bf16", 3456, 1152, "bf16"), ("vision fc1 bf16", 4304, 1152, "bf16")):
            if kind == "w4":
                W = w4a16.random_weight(N, Kd, 64, device=dev)
            else:
                W = (torch.randn(N, Kd, device=dev) * 0.03).to(BF)
            x = torch.randn(Tg, Kd, device=dev).to(BF)
            y = torch.empty(Tg, N, dtype=BF, device=dev)
            us = timed(lambda: K.linear_tc(W, x, out=y), a.iters, flush)
            K.check_gemm_status(dev)
            print(f"linear_tc {label:22s} N={N:6d} K={Kd:5d} T={Tg}: {us:8.1f} us  {2.0 * N * Kd * Tg / us / 1e6:7.1f} TFLOP/s")
    if a.only in ("moe_grouped",):
        # one mixture-of-experts block of the 512-expert geometry on a.rows rows (grouped tensor-core path above 16 rows)
        from r4dx_b200 import native
        from r4dx_b200.config import qwen_hybrid_moe_config
        native.cuda().r4dxb_set_gemm_decode_warps(a.decode_warps)
        from r4dx_b200.models import moe as M
        cfg = qwen_hybrid_moe_config(1)
        H, I, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
        p = "text.layers.0.moe."
        gu0, dn0 = trellis.random_weight(2 * I, H, 3, seed=1, device=dev), trellis.random_weight(H, I, 3, seed=2, device=dev)
        wts = {p + f"experts.{e}.gate_up": gu0 for e in range(E)}
        wts.update({p + f"experts.{e}.down": dn0 for e in range(E)})
        wts[p + "router"] = (torch.randn(E, H, device=dev) * 0.5).to(BF)
        wts[p + "shared_gate"] = (torch.randn(1, H, device=dev) * 0.02).to(BF)
        wts[p + "shared.gate_up"] = trellis.random_weight(2 * cfg.shared_expert_intermediate_size, H, 4, seed=3, device=dev)
        wts[p + "shared.down"] = trellis.random_weight(H, cfg.shared_expert_intermediate_size, 4, seed=4, device=dev)
        Tm = max(a.rows, 17)
        blk = M.MoeBlock(cfg, wts, 0, dev, Tm)
        h = torch.randn(Tm, H, device=dev).to(BF)
        xr = torch.zeros(Tm, H, device=dev, dtype=BF)
        us = timed(lambda: blk.forward(h, xr, Tm), a.iters, flush)
        K.check_gemm_status(dev)
        print(f"moe block (512 experts top-10, hidden {H}, inner {I}) T={Tm}: {us:8.1f} us  "
              f"{2.0 * Tm * cfg.num_experts_per_tok * 3 * I * H / us / 1e6:6.1f} TFLOP/s over the routed experts")
    if a.only in ("", "w4a16"):
        N, Kd = 248320, 5120
        w = w4a16.random_weight(N, Kd, 64, device=dev)
        x = torch.randn(T, Kd, device=dev).to(BF)
        y = torch.empty(T, N, dtype=torch.float32, device=dev)
        us = timed(lambda: K.w4a16_gemv(w, x, out=y), a.iters, flush)
        gbs = w.nbytes / us / 1e3
        print(f"w4a16_gemv lm_head N={N} K={Kd} T={T}: {us:8.1f} us  {gbs:7.0f} GB/s  {gbs / peak:5.2f} of measured HBM")
    if a.only in ("attn_prefill",):
        Hq, Hkv, D = 24, 4, 256
        Tq = max(a.rows, 128)
        ctx = a.ctx
        nblk = (ctx + Tq + 15) // 16 + 1
        cache = torch.randint(0, 120, (nblk, Hkv, 2, 16, D), dtype=torch.uint8, device=dev)
        table = torch.arange(nblk, dtype=torch.int32, device=dev)
        q = torch.randn(Tq, Hq, D, device=dev).to(BF)
        qg = torch.randn(Tq, Hq, 2 * D, device=dev).to(BF)
        ds = torch.full((Hkv,), 1 / 16.0, device=dev)
        out = torch.zeros(Tq, Hq * D, dtype=BF, device=dev)
        flops = 4.0 * Hq * D * Tq * (ctx + (Tq + 1) / 2.0)
        for impl in ("tc", "mma"):
            K.set_attn_prefill_impl(impl)
            us = timed(lambda: K.attn_prefill(q, qg, cache, table, ds, ds, out, Tq, Hq, Hkv, D, ctx, True), a.iters, flush)
            K.check_gemm_status(dev)
            print(f"attn_prefill[{impl}] T={Tq} ctx={ctx}: {us:9.1f} us  {flops / us / 1e6:7.1f} TFLOP/s (causal-effective)")
    if a.only in ("", "attn"):
        Hq, Hkv, D = 24, 4, 256
        ctx = a.ctx
        nblk = (ctx + T + 15) // 16 + 1
        cache = torch.randint(0, 120, (nblk, Hkv, 2, 16, D), dtype=torch.uint8, device=dev)
        table = torch.arange(nblk, dtype=torch.int32, device=dev)
        pos = torch.arange(ctx, ctx + T, dtype=torch.int32, device=dev)
        q = torch.randn(T, Hq, D, device=dev).to(BF)
        qg = torch.randn(T, Hq, 2 * D, device=dev).to(BF)
        ds = torch.full((Hkv,), 1 / 16.0, device=dev)
        splits = 37
        G = Hq // Hkv * T
        pa = torch.zeros(splits * Hkv * G * D, device=dev)
        pm = torch.zeros(splits * Hkv * G * 2, device=dev)
        out = torch.zeros(T, Hq * D, dtype=BF, device=dev)
        us = timed(lambda: K.attn_decode(q, qg, cache, table, pos, ds, ds, pa, pm, out, T, Hq, Hkv, D, splits, True),
                   a.iters, flush)
        nbytes = ctx * Hkv * 2 * D
        print(f"attn_decode ctx={ctx} T={T}: {us:8.1f} us  {nbytes / us / 1e3:7.0f} GB/s  {nbytes / us / 1e3 / peak:5.2f} of measured HBM")


if __name__ == "__main__":
    main()
