"""Calibration passes over the fp32 CPU oracle and the error-compensating w4a16 quantizer that uses them.

* ``kv_descales``: static fp8 descale per (attention layer, KV head) = amax / 448 of the keys (after norm and rope)
  and values seen on calibration prompts (reference: src/convert kv_calib.hpp, docs/container-format.md:668-686).
* ``capture_hessians``: H = sum x x^T over the inputs of every quantizable linear.
* ``gptq_w4a16``: column-by-column rounding onto the w4a16 grid with the rounding error of each column pushed onto
  the not-yet-rounded columns through the inverse Hessian's Cholesky factor, so that the OUTPUT error x (W - Q)^T is
  minimised rather than the weight error (the reference's converter calls its variant LDLQ:
  src/convert/main.cpp:1-120; same group layout and scale / zero rules as ``native/src/host/w4a16.cpp``).

    python -m r4dx_b200.quant.calibrate kv --input random:tiny --tokens 256 --out kv.json
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from .w4a16 import W4Weight


def _run_prompts(cfg: ModelConfig, weights: Dict[str, torch.Tensor], prompts: Sequence[torch.Tensor], on_linear=None, on_kv=None,
                 ngram_table=None):
    from ..models.q4x_oracle import make_oracle
    m = make_oracle(cfg, weights, ngram_table=ngram_table)
    m.on_linear, m.on_kv = on_linear, on_kv
    for ids in prompts:
        m.forward(ids)


def kv_descales(cfg: ModelConfig, weights: Dict[str, torch.Tensor], prompts: Sequence[torch.Tensor], margin: float = 1.0,
                floor: float = 1e-4, ngram_table=None) -> Dict[int, Tuple[List[float], List[float]]]:
    """{layer: (k_descale per KV head, v_descale per KV head)} with descale = margin * amax / 448."""
    amax: Dict[int, List[torch.Tensor]] = {}

    def on_kv(layer, k, v):
        ka, va = k.abs().amax(dim=(0, 2)), v.abs().amax(dim=(0, 2))
        if layer in amax:
            amax[layer][0] = torch.maximum(amax[layer][0], ka)
            amax[layer][1] = torch.maximum(amax[layer][1], va)
        else:
            amax[layer] = [ka, va]

    _run_prompts(cfg, weights, prompts, on_kv=on_kv, ngram_table=ngram_table)
    return {int(l): ([max(floor, float(x) * margin / 448.0) for x in a[0]], [max(floor, float(x) * margin / 448.0) for x in a[1]])
            for l, a in amax.items() if isinstance(l, int)}


def capture_hessians(cfg: ModelConfig, weights: Dict[str, torch.Tensor], prompts: Sequence[torch.Tensor], ngram_table=None,
                     counts: Optional[Dict[str, int]] = None) -> Dict[str, torch.Tensor]:
    """name -> E[x x^T] over the rows each quantizable linear saw (an expert sees its routed rows only).  ``counts`` (optional
    dict) receives the row count per linear.  A linear that saw fewer rows than it has input channels cannot have a
    full-rank second moment: it gets the damped diagonal of what it saw instead, so the error compensation degrades to a
    per-channel weighting (reference: docs/qwen4exp-plan.md Q12/Q16 describes the same fallback and logs the counts)."""
    H: Dict[str, torch.Tensor] = {}
    n: Dict[str, int] = {}

    def on_linear(name, x):
        x = x.reshape(-1, x.shape[-1]).double()
        H[name] = H.get(name, 0) + x.T @ x
        n[name] = n.get(name, 0) + x.shape[0]

    _run_prompts(cfg, weights, prompts, on_linear=on_linear, ngram_table=ngram_table)
    out = {}
    for k, v in H.items():
        h = v / max(1, n[k])
        if n[k] < h.shape[0]:
            d = torch.diagonal(h)
            h = torch.diag(d + 0.01 * d.mean().clamp_min(1e-12))
        out[k] = h.float()
    if counts is not None:
        counts.update(n)
    return out


def _group_params(w: torch.Tensor):
    """Scale and zero of one group slice [N, g] by the packer's rule (fp16 scale, integer zero in 0..15)."""
    lo = torch.minimum(w.amin(1), torch.zeros(()))
    hi = torch.maximum(w.amax(1), torch.zeros(()))
    scale = (hi - lo) / 15.0
    scale = torch.where(scale > 0, scale, torch.ones_like(scale)).to(torch.float16).float()
    scale = torch.where(scale > 0, scale, torch.full_like(scale, 2.0 ** -24))
    zero = torch.round(-lo / scale).clamp(0, 15)
    return scale, zero


def gptq_w4a16(W: torch.Tensor, H: torch.Tensor, group: int = 64, damp: float = 0.01) -> W4Weight:
    """W [N, K] fp32, H [K, K] (input second moment).  Returns packed weights in the engine's w4a16 layout."""
    W = W.detach().double().clone()
    N, K = W.shape
    H = H.double().clone()
    dead = torch.diag(H) == 0
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    H += damp * torch.mean(torch.diag(H)) * torch.eye(K, dtype=torch.float64)
    # upper Cholesky factor of H^-1: row k holds how column k's rounding error spreads over the later columns
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    q = torch.zeros(N, K, dtype=torch.int64)
    scales = torch.zeros(N, K // group)
    zeros = torch.zeros(N, K // group)
    for g0 in range(0, K, group):
        scale, zero = _group_params(W[:, g0:g0 + group].float())
        scales[:, g0 // group], zeros[:, g0 // group] = scale, zero
        sd, zd = scale.double(), zero.double()
        for k in range(g0, g0 + group):
            w = W[:, k]
            qk = (torch.round(w / sd) + zd).clamp(0, 15)
            q[:, k] = qk.long()
            err = (w - sd * (qk - zd)) / Hinv[k, k]
            if k + 1 < K:
                W[:, k + 1:] -= err[:, None] * Hinv[k, k + 1:][None, :]
    return _pack_w4(q, scales, zeros, group)


def _pack_w4(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group: int) -> W4Weight:
    """Nibble i of word j is q for k = 8 j + i; wsz = fp16 scale | fp16 -(1024 + zero) << 16."""
    N, K = q.shape
    sh = (torch.arange(K) % 8) * 4
    wq = (q << sh[None, :]).view(N, K // 8, 8).sum(-1)
    wq = torch.where(wq >= 2 ** 31, wq - 2 ** 32, wq).to(torch.int32)
    s16 = scales.to(torch.float16).view(torch.int16).to(torch.int64) & 0xFFFF
    z16 = (-(1024.0 + zeros)).to(torch.float16).view(torch.int16).to(torch.int64) & 0xFFFF
    wsz = s16 | (z16 << 16)
    wsz = torch.where(wsz >= 2 ** 31, wsz - 2 ** 32, wsz).to(torch.int32)
    return W4Weight(wq.contiguous(), wsz.contiguous(), N, K, group)


def search_w4a16(W: torch.Tensor, importance: Optional[torch.Tensor] = None, group: int = 64, steps: int = 24,
                 min_shrink: float = 0.55) -> W4Weight:
    """Scale search for the w4a16 layout: per (row, group) the [lo, hi] range is shrunk by each of ``steps`` factors in
    [min_shrink, 1] (values outside clip) and the factor with the lowest importance-weighted squared error is kept.
    ``importance`` [K] is the per-input-channel second moment E[x_k^2] (the diagonal of the layer's Hessian, the
    "imatrix"); None weighs all channels equally.  (reference: the converter's ``--quant search --imatrix`` mode,
    src/convert/main.cpp:1-30.)"""
    W = W.detach().float()
    N, K = W.shape
    imp = torch.ones(K) if importance is None else importance.float().clamp_min(0) + 1e-12 * float(importance.float().mean() + 1e-30)
    G = K // group
    w = W.view(N, G, group)
    iw = imp.view(1, G, group)
    lo0 = torch.minimum(w.amin(-1), torch.zeros(()))
    hi0 = torch.maximum(w.amax(-1), torch.zeros(()))
    best_err = torch.full((N, G), float("inf"))
    best_scale = torch.ones(N, G)
    best_zero = torch.zeros(N, G)
    best_q = torch.zeros(N, G, group, dtype=torch.int64)
    for f in torch.linspace(1.0, min_shrink, steps).tolist():
        lo, hi = lo0 * f, hi0 * f
        scale = (hi - lo) / 15.0
        scale = torch.where(scale > 0, scale, torch.ones_like(scale)).to(torch.float16).float()
        scale = torch.where(scale > 0, scale, torch.full_like(scale, 2.0 ** -24))
        zero = torch.round(-lo / scale).clamp(0, 15)
        q = (torch.round(w / scale[..., None]) + zero[..., None]).clamp(0, 15)
        err = (((q - zero[..., None]) * scale[..., None] - w) ** 2 * iw).sum(-1)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best_scale = torch.where(better, scale, best_scale)
        best_zero = torch.where(better, zero, best_zero)
        best_q = torch.where(better[..., None], q.long(), best_q)
    return _pack_w4(best_q.view(N, K), best_scale, best_zero, group)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-calibrate")
    ap.add_argument("what", choices=["kv", "hessians", "imatrix"],
                    help="kv: fp8 KV descales (json); hessians: one [K, K] second-moment matrix per quantizable linear "
                         "(safetensors, for `convert --hessians`); imatrix: their diagonals only (per-input-channel importance)")
    ap.add_argument("--input", required=True, help="'random:<tiny|small>' or a container / checkpoint readable by the converter")
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.add_argument("--ngram-sidecar", default=None, help="qwen4_exp: the n-gram table file the n-gram layer reads its rows from")
    a = ap.parse_args(argv)
    from ..cli.convert import load_source
    cfg, w = load_source(a.input, 0, False, a.seed)
    table = None
    if cfg.is_qwen4_exp and cfg.ple_layers:
        if not a.ngram_sidecar:
            raise SystemExit("qwen4_exp: --ngram-sidecar FILE is required (activations after the n-gram layer depend on its rows)")
        from ..runtime import ngram as NG
        table = NG.NgramTable.open(a.ngram_sidecar, mode="file")
    g = torch.Generator().manual_seed(a.seed)
    prompts = [torch.randint(0, cfg.vocab_size, (a.tokens,), generator=g) for _ in range(a.prompts)]
    if a.what in ("hessians", "imatrix"):
        from safetensors.torch import save_file
        counts: Dict[str, int] = {}
        H = capture_hessians(cfg, w, prompts, ngram_table=table, counts=counts)
        thin = sorted(k for k, v in H.items() if counts.get(k, 0) < v.shape[0])
        if a.what == "imatrix":
            H = {k: torch.diagonal(v).contiguous() for k, v in H.items()}
        save_file({k: v.contiguous() for k, v in H.items()}, a.out)
        print(f"wrote {a.what} of {len(H)} linears to {a.out}")
        if thin:
            print(f"{len(thin)} linears saw fewer rows than input channels and got a damped diagonal (first: {thin[0]}, "
                  f"{counts[thin[0]]} rows)")
        return 0
    d = kv_descales(cfg, w, prompts, ngram_table=table)
    json.dump({str(l): {"k": k, "v": v} for l, (k, v) in d.items()}, open(a.out, "w"), indent=1)
    print(f"wrote fp8 KV descales of {len(d)} attention layers to {a.out}")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
