"""KL report: how far a quantized weight set moves the model's next-token distribution from the unquantized one.

    python -m r4dx_b200.utils.kl_report --input random:tiny [--layout trellis|w4a16] [--kb-plan mix4.5] [--hessians h.safetensors]

Runs the fp32 CPU oracle twice over the same prompts - once on the source weights, once on the dequantized quantized set -
and reports, per position, KL(source || quantized) of the next-token distributions (mean / p50 / p99 / max), the top-1
agreement and the mean absolute logit error.  ``--input`` takes what the converter takes (``random:<tiny|small>``, a
checkpoint directory, a GGUF file).  (reference: tools/reference/kl_report.py, kl_audit.py.)"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def kl_stats(ref_logits: torch.Tensor, got_logits: torch.Tensor) -> dict:
    """Rows of logits [T, V] -> summary of KL(ref || got) per row (nats), top-1 agreement, mean |logit error|."""
    lp = torch.log_softmax(ref_logits.double(), -1)
    lq = torch.log_softmax(got_logits.double(), -1)
    kl = (lp.exp() * (lp - lq)).sum(-1).clamp_min(0)
    s = torch.sort(kl).values
    pick = lambda f: float(s[min(len(s) - 1, int(f * len(s)))])
    return {"positions": int(kl.numel()), "kl_mean": float(kl.mean()), "kl_p50": pick(0.5), "kl_p99": pick(0.99),
            "kl_max": float(kl.max()), "top1_agreement": float((ref_logits.argmax(-1) == got_logits.argmax(-1)).double().mean()),
            "mean_abs_logit_err": float((ref_logits - got_logits).abs().mean())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-kl-report")
    ap.add_argument("--input", required=True)
    ap.add_argument("--layout", default="trellis", choices=["trellis", "w4a16", "bf16"])
    ap.add_argument("--kb-plan", default="mix4.5", choices=["mix4.5", "mix3.3", "kb3", "kb4", "kb5"])
    ap.add_argument("--hessians", default=None)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ngram-sidecar", default=None, help="qwen4_exp: the n-gram table file")
    a = ap.parse_args(argv)
    from ..cli.convert import _kb_rule, load_source
    from ..models.q4x_oracle import make_oracle
    from ..quant.weights import dequantize_weight_set, quantize_weight_set
    cfg, w = load_source(a.input, a.layers, False, a.seed)
    table = None
    if cfg.is_qwen4_exp and cfg.ple_layers:
        if not a.ngram_sidecar:
            raise SystemExit("qwen4_exp: --ngram-sidecar FILE is required")
        from ..runtime import ngram as NG
        table = NG.NgramTable.open(a.ngram_sidecar, mode="file")
    hess = None
    if a.hessians:
        from safetensors.torch import load_file
        hess = {k: v for k, v in load_file(a.hessians).items() if v.dim() == 2}
    q = quantize_weight_set(cfg, w, layout=a.layout, kb_rule=_kb_rule(a.kb_plan), seed=a.seed, hessians=hess)
    src, got = make_oracle(cfg, w, ngram_table=table), make_oracle(cfg, dequantize_weight_set(q), ngram_table=table)
    g = torch.Generator().manual_seed(a.seed + 1)
    ref_rows, got_rows = [], []
    for _ in range(a.prompts):
        ids = torch.randint(0, cfg.vocab_size, (a.tokens,), generator=g)
        ref_rows.append(src.forward(ids)[0])
        got_rows.append(got.forward(ids)[0])
    out = kl_stats(torch.cat(ref_rows), torch.cat(got_rows))
    out.update({"layout": a.layout, "kb_plan": a.kb_plan, "error_compensated": bool(hess)})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
