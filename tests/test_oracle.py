"""CPU oracle self-consistency (tiny hybrid geometry)."""
import torch

from r4dx_b200.config import tiny_hybrid_config, tiny_moe_config
from r4dx_b200.models.oracle import OracleModel, OracleState, init_weights
from r4dx_b200.ops import reference as R


def test_gdn_chunked_matches_recurrent():
    g = torch.Generator().manual_seed(3)
    T, Hk, H, K, V = 150, 2, 4, 64, 64
    q = R.l2norm(torch.randn(T, Hk, K, generator=g))
    k = R.l2norm(torch.randn(T, Hk, K, generator=g))
    v = torch.randn(T, H, V, generator=g)
    gate = -torch.rand(T, H, generator=g) * 0.5
    beta = torch.rand(T, H, generator=g)
    s0 = torch.randn(H, V, K, generator=g) * 0.1
    o1, s1 = R.gdn_recurrent(q, k, v, gate, beta, s0)
    o2, s2 = R.gdn_chunked(q, k, v, gate, beta, s0, chunk=64)
    assert torch.allclose(o1, o2, atol=2e-4, rtol=1e-4)
    assert torch.allclose(s1, s2, atol=2e-4, rtol=1e-4)


def test_prefill_equals_stepwise():
    cfg = tiny_hybrid_config()
    w = init_weights(cfg, 0)
    m = OracleModel(cfg, w)
    ids = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1))
    full, _ = m.forward(ids)
    st = OracleState()
    rows = []
    for s in (0, 7, 8, 20):
        e = {0: 7, 7: 8, 8: 20, 20: 24}[s]
        lg, st = m.forward(ids[s:e], st)
        rows.append(lg)
    step = torch.cat(rows)
    assert torch.allclose(full, step, atol=1e-4, rtol=1e-4)


def test_chunked_model_equals_recurrent_model():
    cfg = tiny_hybrid_config()
    w = init_weights(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(1))
    a, _ = OracleModel(cfg, w).forward(ids)
    b, _ = OracleModel(cfg, w, chunked_gdn=True).forward(ids)
    assert torch.allclose(a, b, atol=2e-4, rtol=1e-3)


def test_greedy_16_tokens_deterministic():
    cfg = tiny_hybrid_config()
    w = init_weights(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(1))
    t1 = OracleModel(cfg, w).greedy(ids, 16)
    t2 = OracleModel(cfg, w).greedy(ids, 16)
    assert t1 == t2 and len(t1) == 16


def test_moe_oracle_runs():
    cfg = tiny_moe_config()
    w = init_weights(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (6,), generator=torch.Generator().manual_seed(1))
    lg, st = OracleModel(cfg, w).forward(ids)
    assert lg.shape == (6, cfg.vocab_size) and torch.isfinite(lg).all()


def test_shard_views():
    from r4dx_b200.config import qwen_hybrid_27b_config
    cfg = qwen_hybrid_27b_config()
    for world in (1, 2, 4, 8):
        for r in range(world):
            s = cfg.shard(world, r)
            assert s.num_attention_heads * world == 24
            assert s.intermediate_size % 128 == 0
    s8 = cfg.shard(8, 5)
    assert s8.num_key_value_heads == 1 and s8.kv_replicas == 2 and s8.kv_head_of_rank() == 2


def test_llama_style_config_prefill_equals_stepwise():
    """The dense family (no q/k norm, no gate, full rope) through the same oracle: chunk invariance."""
    import torch
    from r4dx_b200.config import tiny_llama_config
    from r4dx_b200.models.oracle import OracleModel, OracleState, init_weights
    cfg = tiny_llama_config()
    cfg.validate()
    w = init_weights(cfg, 3)
    assert "text.layers.0.attn.q_norm" not in w and w["text.layers.0.attn.qg"].shape[0] == cfg.q_dim
    m = OracleModel(cfg, w)
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(0))
    full, _ = m.forward(ids)
    st = OracleState()
    rows = []
    for t in range(12):
        lg, st = m.forward(ids[t:t + 1], st)
        rows.append(lg)
    assert torch.allclose(full, torch.cat(rows), atol=1e-4, rtol=1e-4)


def test_gemma_style_config_chunk_invariance_and_window():
    """Sandwich norms, GeGLU, sliding-window layers with their own rope base: prefill == stepwise, and tokens beyond
    the window do not influence a windowed layer's output."""
    import torch
    from r4dx_b200.config import tiny_gemma_config
    from r4dx_b200.models.oracle import OracleModel, OracleState, init_weights
    from r4dx_b200.ops import reference as R
    cfg = tiny_gemma_config()
    cfg.validate()
    assert [cfg.layer_window(i) for i in range(4)] == [24, 0, 24, 0]
    assert cfg.layer_theta(0) == cfg.rope_local_theta and cfg.layer_theta(1) == cfg.rope_theta
    w = init_weights(cfg, 4)
    assert "text.layers.0.post_attn_out_norm" in w and "text.layers.0.attn.q_norm" in w
    m = OracleModel(cfg, w)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(0))
    full, _ = m.forward(ids)
    st = OracleState()
    rows = []
    for s in range(0, 40, 7):
        lg, st = m.forward(ids[s:s + 7], st)
        rows.append(lg)
    assert torch.allclose(full, torch.cat(rows), atol=2e-4, rtol=1e-4)
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(3, 4, 16, generator=g), torch.randn(30, 2, 16, generator=g), torch.randn(30, 2, 16, generator=g)
    a = R.causal_gqa_attention(q, k, v, 27, window=8)
    k2, v2 = k.clone(), v.clone()
    k2[:19] += 5.0
    v2[:19] -= 3.0                                        # keys 0..18 are outside every row's window (rows at 27..29)
    assert torch.allclose(a, R.causal_gqa_attention(q, k2, v2, 27, window=8), atol=1e-6)
    assert not torch.allclose(a, R.causal_gqa_attention(q, k2, v2, 27), atol=1e-3)


def test_short_conv_moe_family_is_invariant_to_how_the_prompt_is_split():
    """Short-conv + attention MoE family on the oracle: feeding a prompt whole or in pieces gives the same logits (the conv
    state carries the last taps - 1 rows of B * x), the dense first layer and the sigmoid-routed layers both run."""
    from r4dx_b200.config import tiny_lfm2_config
    from r4dx_b200.models.oracle import OracleModel, init_weights, linear_names
    cfg = tiny_lfm2_config()
    assert cfg.layer_types == ["conv", "conv", "full_attention", "conv", "full_attention"]
    assert not cfg.layer_is_moe(0) and cfg.layer_is_moe(1)
    w = init_weights(cfg, 3)
    assert "text.layers.0.mlp.gate_up" in w and "text.layers.1.moe.experts.7.down" in w and "text.layers.1.moe.expert_bias" in w
    assert "text.layers.1.moe.shared.gate_up" not in w
    assert set(linear_names(cfg)) <= set(w)
    m = OracleModel(cfg, w)
    ids = torch.randint(0, cfg.vocab_size, (11,), generator=torch.Generator().manual_seed(1))
    whole, _ = m.forward(ids)
    a, st = m.forward(ids[:4])
    b, st = m.forward(ids[4:5], st)
    c, st = m.forward(ids[5:], st)
    assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-5, rtol=1e-4)


def test_sigmoid_router_bias_moves_the_selection_but_not_the_weights():
    from r4dx_b200.ops import reference as R
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    ids, w = R.moe_route_sigmoid(logits, None, 2, True, 1.0)
    assert ids.tolist() == [[0, 1]]
    s = torch.sigmoid(logits[0])
    assert torch.allclose(w[0], (s[:2] / (s[:2].sum() + 1e-6)).to(torch.bfloat16).float())
    ids, w = R.moe_route_sigmoid(logits, torch.tensor([0.0, 0.0, 0.0, 5.0]), 2, True, 2.0)
    assert ids.tolist() == [[3, 0]]
    sel = torch.stack([s[3], s[0]])
    assert torch.allclose(w[0], (sel / (sel.sum() + 1e-6) * 2.0).to(torch.bfloat16).float())


def test_image_blocks_are_bidirectional_on_sliding_layers_only():
    """Gemma-style image rows: inside a block the sliding-window layers see the whole block, so an early row of the block
    depends on a later one; outside blocks, and on a model without windows, the mask stays causal.  Chunking that keeps a
    block whole gives the same logits as one call."""
    from r4dx_b200.config import tiny_gemma_config, tiny_llama_config
    from r4dx_b200.models import gemma_vision as GV
    from r4dx_b200.models.oracle import OracleModel, init_weights
    from r4dx_b200.ops import reference as R
    # op level: the dense reference mask and the key-limit form agree
    g = torch.Generator().manual_seed(0)
    T, window, blocks = 20, 5, [(4, 9), (12, 15)]
    q, k, v = torch.randn(T, 4, 16, generator=g), torch.randn(T, 2, 16, generator=g), torch.randn(T, 2, 16, generator=g)
    got = R.causal_gqa_attention(q, k, v, 0, window, GV.key_limit_ext(0, T, blocks))
    mask = GV.dense_mask(T, window, True, blocks)
    s = torch.einsum("thgd,shd->hgts", q.view(T, 2, 2, 16), k) / 4.0
    ref = torch.einsum("hgts,shd->thgd", torch.softmax(s.masked_fill(~mask[None, None], float("-inf")), -1), v).reshape(T, 4, 16)
    assert torch.allclose(got, ref, atol=1e-5)
    # model level
    cfg = tiny_gemma_config()
    w = init_weights(cfg, 3)
    m = OracleModel(cfg, w)
    ids = torch.randint(0, cfg.vocab_size, (18,), generator=g)
    rows = torch.randn(5, cfg.hidden_size, generator=g) * 0.5
    ov = (torch.arange(6, 11), rows)
    blocks = [(6, 11)]
    causal, _ = m.forward(ids, embed_overrides=ov)
    bidir, _ = m.forward(ids, embed_overrides=ov, image_blocks=blocks)
    assert torch.allclose(causal[:6], bidir[:6], atol=1e-5)                  # rows before the block are untouched
    assert not torch.allclose(causal[6], bidir[6], atol=1e-4)                # the block's first row now sees the rest of it
    rows2 = rows.clone()
    rows2[4] += 1.0                                                          # change the block's LAST row
    moved, _ = m.forward(ids, embed_overrides=(ov[0], rows2), image_blocks=blocks)
    assert not torch.allclose(moved[6], bidir[6], atol=1e-4)                 # ... and its first row's logits move
    moved_c, _ = m.forward(ids, embed_overrides=(ov[0], rows2))
    assert torch.allclose(moved_c[6], causal[6], atol=1e-5)                  # causal: they do not
    # block-safe chunking reproduces the single call
    chunks = GV.plan_prefill_chunks(18, blocks, 8, max_block=8)
    st, out = None, []
    for s0, n in chunks:
        sel = (ov[0] >= s0) & (ov[0] < s0 + n)
        lg, st = m.forward(ids[s0:s0 + n], st, embed_overrides=(ov[0][sel] - s0, rows[sel]), image_blocks=blocks)
        out.append(lg)
    assert torch.allclose(torch.cat(out), bidir, atol=1e-4, rtol=1e-4)
    # a family without sliding windows ignores the blocks
    lc = tiny_llama_config()
    lm = OracleModel(lc, init_weights(lc, 1))
    a, _ = lm.forward(ids % lc.vocab_size)
    b, _ = lm.forward(ids % lc.vocab_size, image_blocks=blocks)
    assert torch.equal(a, b)
