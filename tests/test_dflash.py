"""Block-diffusion drafter: host selector walk (CPU), device round vs the fp32 restatement, lossless speculation."""
import pytest
import torch

from r4dx_b200.models import dflash as DF


def _py_select(c, cand, unary, gate, succ, pred, anchor):
    out, prev = [], anchor
    for t in range(1, cand.shape[0]):
        score = unary[t].double() + ((succ[cand[t].long()].double() * pred[prev].double()[None]) * gate[t].double()[None]).sum(-1)
        b = int(score.argmax())
        p = torch.softmax(score, 0)[b].item()
        if p < c.p_min:
            break
        out.append(int(cand[t, b]))
        prev = out[-1]
    return out if len(out) >= c.n_min else []


def test_selector_walk_matches_python_restatement():
    c = DF.tiny_dflash_config()
    g = torch.Generator().manual_seed(0)
    V = 500
    succ, pred = torch.randn(V, c.rank, generator=g), torch.randn(V, c.rank, generator=g)
    for trial in range(5):
        cand = torch.stack([torch.randperm(V, generator=g)[:c.cands] for _ in range(c.block)]).to(torch.int32)
        unary = torch.randn(c.block, c.cands, generator=g) * 2
        gate = torch.randn(c.block, c.rank, generator=g) * 0.2
        c.p_min = [0.0, 0.0, 0.2, 0.5, 0.0][trial]
        c.n_min = [0, 3, 0, 0, 8][trial]
        assert DF.select_chain(c, cand, unary, gate, succ, pred, 7) == _py_select(c, cand, unary, gate, succ, pred, 7)


@pytest.mark.gpu
def test_device_round_matches_restatement_and_speculation_is_lossless(same_kernels_for_every_row_count):
    from r4dx_b200.config import tiny_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.models.oracle import init_weights
    from r4dx_b200.quant.weights import dequantize_weight_set, quantize_weight_set
    cfg = tiny_hybrid_config()
    q = quantize_weight_set(cfg, init_weights(cfg, 0))
    dq = dequantize_weight_set(q)
    qd = {k: (v.to("cuda") if hasattr(v, "to") else v) for k, v in q.items()}
    c = DF.tiny_dflash_config(cfg.hidden_size, (1, 3))
    dw, dwf = DF.quantize_dflash_weights(c, DF.init_dflash_weights(c, cfg.vocab_size, 1))
    main = HybridModel(cfg, qd, max_ctx=256)
    dr = DF.DflashDrafter(main, c, dw)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(2)).to(torch.int32)

    feats = []

    def hook(start, T, _h):
        feats.append(main.captured[:, :T].permute(1, 0, 2).reshape(T, -1).float().cpu().clone())
        dr.inject(main.captured, start, T)

    tok = main.prefill(prompt, hook=hook)
    oracle = DF.DflashOracle(c, dwf, dq["text.embed_tokens"], dq["lm_head"])
    oracle.inject(torch.cat(feats), 0)
    ref_logits, _ = oracle.draft_logits(tok, 70)
    got, _ = dr.draft_rows(tok)
    scale = ref_logits.abs().max().item()
    assert (got.float().cpu() - ref_logits).abs().max().item() < 0.06 * scale
    # lossless: whatever the drafter proposes, the emitted stream is the target's greedy stream
    plain = HybridModel(cfg, qd, max_ctx=256).generate_greedy(prompt, 24, use_graph=False)
    spec = dr.generate(prompt, 24)
    assert spec == plain
    assert dr.rounds > 0
