"""Child of tests/test_tp_gpu.py: the loader's --pp 2 and --pp 2 --tp 2 --hybrid products on two ranks.

Rank 0 leads through the TpTextModel facade (prefill of a prompt longer than --pp-min-rows, greedy decode, one sampled
step's logits row) and compares against the whole model on its own GPU; rank 1 follows."""
import os
import sys
from types import SimpleNamespace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]
    rank = int(os.environ["RANK"])
    from r4dx_b200.cli.loader import load_text_model
    args = SimpleNamespace(model="synthetic:small", layers=4, tp=2 if mode == "hybrid" else 1, pp=2, hybrid=mode == "hybrid", ep=1,
                           pp_split=0, pp_min_rows=64, tp_mode="fused", tp_ar_timeout_ms=500, tp_fault="", max_ctx=512,
                           mtp=0, ngram=0, dflash=None, tokenizer_dir=None, prefill_chunk=64)
    tm, _, _ = load_text_model(args)
    if rank != 0:
        tm.follow()
        os._exit(0)
    from r4dx_b200.config import small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.quant.weights import synthetic_weight_set
    gcfg = small_hybrid_config()
    gcfg.num_hidden_layers = 4
    gcfg.layer_types = gcfg.layer_types[:4]
    ref = HybridModel(gcfg, synthetic_weight_set(gcfg, device="cuda:0", seed=0), max_ctx=512, device="cuda:0")
    ids = torch.randint(0, gcfg.vocab_size, (150,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    for attempt in range(2):                       # the second prompt exercises reset + a fresh pipeline pass
        tm.reset()
        ref.reset()
        tok = tm.prefill(ids.tolist())
        rtok = ref.prefill(ids, chunk=64)
        assert tok == rtok, (tok, rtok)
        row = tm.last_logits().float().cpu()
        rrow = ref.buf.logits[0].float().cpu()
        assert row.shape == rrow.shape and (row - rrow).abs().max().item() < 0.03 * rrow.abs().max().item()
        out, rout = [tok], [rtok]
        for _ in range(8):
            out.append(tm.decode_step_greedy(out[-1]))
            rout.append(ref.decode_step_greedy(rout[-1]))
        same = sum(int(a == b) for a, b in zip(out, rout))
        print(mode, "tokens", out, "ref", rout, flush=True)
        assert same >= (9 if mode == "split" else 7), (out, rout)
        lg = tm.decode_step(out[-1]).float().cpu()
        assert lg.numel() == gcfg.vocab_size
    if mode == "hybrid":
        assert tm.local.pipelined_prompts == 2
    tm.shutdown()
    print("PP_PRODUCT_OK", mode, flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
