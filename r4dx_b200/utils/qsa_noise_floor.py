"""How much the tie rule of the block selection moves the logits: KL between the "most recent block wins" rule (what the
engine and its oracle use) and the opposite rule (the oldest block wins) on the same model and prompts.

Ties at the selection cut are frequent (a block whose head scores are all <= 0 scores exactly 0), and a framework that
breaks them in an implementation-defined order differs from any fixed rule by this much; accuracy numbers against such a
framework are read against this floor (reference: docs/qwen4exp-plan.md Q23, tools/reference/qwen4exp/noise_floor.py).

    python -m r4dx_b200.utils.qsa_noise_floor --input random:q4x --ngram-sidecar tiny.r4dx-ngram --tokens 96
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def select_blocks_oldest(scores: torch.Tensor, topk: int) -> torch.Tensor:
    nb = scores.numel()
    order = sorted(range(nb), key=lambda b: (-float(scores[b]), b))[:topk]
    return torch.tensor(sorted(order), dtype=torch.long)


def noise_floor(cfg, weights, table, prompts) -> dict:
    from ..models import q4x_oracle as Q
    from .kl_report import kl_stats
    recent = Q.make_oracle(cfg, weights, ngram_table=table)
    ref_rows, alt_rows, tied, sparse = [], [], 0, 0
    for ids in prompts:
        a, st_a = recent.forward(ids)
        keep = Q.select_blocks
        Q.select_blocks = select_blocks_oldest          # the oracle looks the rule up at call time
        try:
            b, st_b = Q.make_oracle(cfg, weights, ngram_table=table).forward(ids)
        finally:
            Q.select_blocks = keep
        ref_rows.append(a)
        alt_rows.append(b)
        for li, sel in st_a.selected.items():
            for ra, rb in zip(sel, st_b.selected[li]):
                if ra is not None:
                    sparse += 1
                    tied += int(ra != rb)
    out = kl_stats(torch.cat(ref_rows), torch.cat(alt_rows))
    out.update({"sparse_rows": sparse, "rows_where_the_rules_pick_different_blocks": tied})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-qsa-noise-floor")
    ap.add_argument("--input", required=True)
    ap.add_argument("--ngram-sidecar", required=True)
    ap.add_argument("--tokens", type=int, default=96)
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    from ..cli.convert import load_source
    from ..runtime import ngram as NG
    cfg, w = load_source(a.input, a.layers, False, a.seed)
    if not (cfg.is_qwen4_exp and cfg.indexer_heads):
        raise SystemExit("the model has no block-selecting attention layers")
    table = NG.NgramTable.open(a.ngram_sidecar, mode="file")
    g = torch.Generator().manual_seed(a.seed + 1)
    prompts = [torch.randint(0, cfg.vocab_size, (a.tokens,), generator=g) for _ in range(a.prompts)]
    print(json.dumps(noise_floor(cfg, w, table, prompts)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
