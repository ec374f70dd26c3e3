"""Chooses the trellis bit width (3, 4 or 5) of every class of linears under a byte budget.

A class is (layer, projection) - all experts of one layer's gate_up (or down) form one class, because a layer's experts
share one launch and therefore one width.  Every class starts at 3 bits; the tool then promotes, one step at a time, the
class whose promotion removes the most output error per added byte, until the next promotion would exceed the budget.

The error of a class at a width is measured, not modelled: the class's tensors are quantized at that width, and the
error is  sum over its tensors of  ||(W - Q) X||^2 / ||W X||^2  with X the calibration second moments when a Hessian file
is given (tr((W - Q) H (W - Q)^T) / tr(W H W^T)), else the plain relative squared weight error.

    python -m r4dx_b200.utils.alloc_bits --input random:moe --budget-mib 3.0 --out plan.json [--hessians h.safetensors]
    python -m r4dx_b200.cli.convert --input ... --kb-plan-file plan.json ...

(reference: docs/qwen4exp-plan.md 4.4 step 4 and Q14: bits per tensor class chosen by a sweep within a weight-byte cap.)
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from typing import Callable, Dict, List, Optional, Tuple

import torch

WIDTHS = (3, 4, 5)


def class_of(name: str) -> str:
    """text.layers.7.moe.experts.12.gate_up -> text.layers.7.moe.experts.*.gate_up; other linears are their own class."""
    return re.sub(r"\.experts\.\d+\.", ".experts.*.", name)


def class_pattern(cls: str) -> str:
    return "^" + re.escape(cls).replace(r"\*", r"\d+") + "$"


def plan_rule(plan: Dict[str, int], default: int = 4) -> Callable[[str], int]:
    """name -> width from a {class: width} plan (what ``convert --kb-plan-file`` applies)."""
    return lambda name: int(plan.get(class_of(name), default))


def measure(w: Dict[str, torch.Tensor], names: List[str], hessians: Optional[Dict[str, torch.Tensor]] = None, seed: int = 0
            ) -> Tuple[Dict[str, Dict[int, float]], Dict[str, int]]:
    """({class: {width: error}}, {class: weight count}) for the quantizable linears ``names``."""
    from ..quant import trellis
    err: Dict[str, Dict[int, float]] = {}
    size: Dict[str, int] = {}
    for i, name in enumerate(names):
        t = w[name].float()
        cls = class_of(name)
        size[cls] = size.get(cls, 0) + t.numel()
        H = hessians.get(name).double() if hessians and name in hessians else None
        den = float(torch.einsum("nk,kj,nj->", t.double(), H, t.double())) if H is not None else float((t.double() ** 2).sum())
        for kb in WIDTHS:
            q, _ = trellis.quantize(t, kb, seed=seed * 100003 + i)
            d = (trellis.reconstruct(q) - t).double()
            num = float(torch.einsum("nk,kj,nj->", d, H, d)) if H is not None else float((d ** 2).sum())
            err.setdefault(cls, {}).setdefault(kb, 0.0)
            err[cls][kb] += num / max(den, 1e-30)
    return err, size


def allocate(err: Dict[str, Dict[int, float]], size: Dict[str, int], budget_bytes: int) -> Dict[str, int]:
    plan = {c: WIDTHS[0] for c in err}
    used = sum(size[c] * plan[c] // 8 for c in plan)
    if used > budget_bytes:
        raise ValueError(f"even {WIDTHS[0]} bits everywhere need {used} bytes, the budget is {budget_bytes}")
    while True:
        best, best_gain = None, 0.0
        for c, kb in plan.items():
            if kb == WIDTHS[-1]:
                continue
            extra = size[c] // 8                              # one more bit per weight
            if used + extra > budget_bytes:
                continue
            gain = (err[c][kb] - err[c][kb + 1]) / extra
            if best is None or gain > best_gain:
                best, best_gain = c, gain
        if best is None:
            return plan
        plan[best] += 1
        used += size[best] // 8


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-alloc-bits")
    ap.add_argument("--input", required=True)
    ap.add_argument("--budget-mib", type=float, required=True, help="bytes the trellis code words of all linears may take, in MiB")
    ap.add_argument("--hessians", default=None, help="safetensors file of `calibrate hessians`: errors are weighed by the inputs' second moments")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    from ..cli.convert import load_source
    from ..quant.weights import is_quantized_linear
    cfg, w = load_source(a.input, a.layers, False, a.seed)
    names = [n for n, t in w.items() if is_quantized_linear(n) and t.dim() == 2 and t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0]
    hess = None
    if a.hessians:
        from safetensors.torch import load_file
        hess = {k: v for k, v in load_file(a.hessians).items() if v.dim() == 2}
    err, size = measure(w, names, hess, a.seed)
    plan = allocate(err, size, int(a.budget_mib * 2 ** 20))
    used = sum(size[c] * plan[c] // 8 for c in plan)
    bpw = 8.0 * used / max(1, sum(size.values()))
    json.dump({"format": "r4dxb-kb-plan-1", "classes": plan, "bytes": used, "bits_per_weight": bpw}, open(a.out, "w"), indent=1)
    hist = {kb: sum(1 for v in plan.values() if v == kb) for kb in WIDTHS}
    print(json.dumps({"classes": len(plan), "bytes": used, "bits_per_weight": round(bpw, 3), "widths": hist, "out": a.out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
