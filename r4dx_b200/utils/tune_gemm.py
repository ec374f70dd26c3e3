"""Fills the measured tuning table of the two trellis product kernels.

    python -m r4dx_b200.utils.tune_gemm [--tp 1,2,4,8] [--rows 1,8] [--gemm-rows 256,1024,2048,4096] [--out PATH]

For every linear shape of the 27B hybrid geometry, at every requested tensor-parallel degree's shard shape, the tool
times the weight-streaming kernel at each cluster split (1 / 2 / 4 / 8) and the tcgen05 GEMM at each token tile
(128 / 256 / 512), cold (a buffer larger than L2 is rewritten between launches), and writes the winners to
``r4dx_b200/ops/tuning_table.json``.  ``ops/kernels.py:pick_ksplit`` / ``pick_token_tile`` look a shape up there first
and fall back to their heuristics for shapes the table does not hold.  An entry is only written when its winner beats the
heuristic's choice by more than ``--min-gain`` (default 5 %): the table records measured exceptions, not noise.

(reference: tools/profile/tune_gemm.py fills src/model/gemm_tuning_table*.inc, read by src/model/linear.h:18-140
``PickTuning``.)
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .bench_kernels import SHAPES_27B, timed

COLUMN_PARALLEL = {"in_proj_qkv", "in_proj_z", "qg", "kv", "gate_up"}     # N is split over the ranks; the others split K


def shard_shape(name: str, N: int, K: int, tp: int):
    if name in COLUMN_PARALLEL:
        n = N // tp
        if name == "kv":
            n = max(n, 256)           # KV heads are replicated once the ranks outnumber them
        return (n + 127) // 128 * 128, K
    return N, (K // tp) // 128 * 128


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", default="1,2,4,8")
    ap.add_argument("--rows", default="1")
    ap.add_argument("--gemm-rows", default="256,1024,2048,4096")
    ap.add_argument("--kb", type=int, default=4)
    ap.add_argument("--iters", type=int, default=12)
    ap.add_argument("--min-gain", type=float, default=0.05)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ops", "tuning_table.json"))
    a = ap.parse_args()
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.quant import trellis
    K.TUNING.clear()                    # measure against the heuristics, not against an older table
    dev = "cuda"
    flush = torch.zeros(256 << 18, dtype=torch.float32, device=dev)
    BF = torch.bfloat16
    table = {"gemv": {}, "gemm": {}, "meta": {"device": torch.cuda.get_device_name(0), "kb": a.kb, "min_gain": a.min_gain}}
    seen = set()
    for tp in [int(x) for x in a.tp.split(",")]:
        for name, (N0, K0) in SHAPES_27B.items():
            N, Kd = shard_shape(name, N0, K0, tp)
            if (N, Kd) in seen:
                continue
            seen.add((N, Kd))
            w = trellis.random_weight(N, Kd, a.kb, seed=1, device=dev)
            for T in [int(x) for x in a.rows.split(",")]:
                x = torch.randn(T, Kd, device=dev).to(BF)
                y = torch.empty(T, N, dtype=BF, device=dev)
                base = K.pick_ksplit(N, Kd)
                res = {}
                for ks in (1, 2, 4, 8):
                    if Kd // 128 < ks:
                        continue
                    try:
                        res[ks] = timed(lambda: K.trellis_gemv(w, x, out=y, ksplit=ks), a.iters, flush)
                    except K.KernelError:
                        continue
                best = min(res, key=res.get)
                gain = 1.0 - res[best] / res[base]
                print(f"gemv {name:12s} tp={tp} N={N:6d} K={Kd:6d} T={T}: " + "  ".join(f"ks{k}={v:6.1f}" for k, v in res.items()) +
                      f"  heuristic ks{base}  best ks{best} ({gain * 100:+.1f} %)", flush=True)
                if best != base and gain > a.min_gain:
                    table["gemv"][f"{N}x{Kd}x{'1' if T == 1 else 'n'}"] = {"ksplit": best, "us": round(res[best], 1), "heuristic_us": round(res[base], 1)}
            for T in [int(x) for x in a.gemm_rows.split(",")]:
                x = torch.randn(T, Kd, device=dev).to(BF)
                xh = K.trellis_input(x, w.suh)
                y = torch.empty(T, N, dtype=BF, device=dev)
                base = K.pick_token_tile(T, N)
                res = {}
                for tn in (128, 256, 512):
                    if tn > max(128, T):
                        continue
                    res[tn] = timed(lambda: K.trellis_gemm(w, xh, out=y, tn=tn), max(4, a.iters // 2), flush)
                K.check_gemm_status(dev)
                best = min(res, key=res.get)
                gain = 1.0 - res[best] / res[base] if base in res else 0.0
                print(f"gemm {name:12s} tp={tp} N={N:6d} K={Kd:6d} T={T}: " + "  ".join(f"tn{k}={v:7.1f}" for k, v in res.items()) +
                      f"  heuristic tn{base}  best tn{best} ({gain * 100:+.1f} %)", flush=True)
                if best != base and gain > a.min_gain:
                    table["gemm"][f"{N}x{Kd}x{T}"] = {"tn": best, "us": round(res[best], 1), "heuristic_us": round(res.get(base, 0.0), 1)}
            del w
    with open(a.out, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    print(f"wrote {a.out}: {len(table['gemv'])} weight-streaming entries, {len(table['gemm'])} GEMM entries")


if __name__ == "__main__":
    main()
