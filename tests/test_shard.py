"""Tensor-parallel shard slicing of quantized weights (CPU)."""
import torch

from r4dx_b200.config import qwen_hybrid_27b_config, small_hybrid_config
from r4dx_b200.parallel.shard import shard_plan, slice_trellis_cols, slice_trellis_rows
from r4dx_b200.quant import trellis, w4a16
from r4dx_b200.parallel.shard import slice_cols, slice_rows


def test_trellis_row_parallel_partials_add_up():
    tw = trellis.random_weight(256, 512, 5, seed=2, sigma=0.05)
    x = torch.randn(2, 512, generator=torch.Generator().manual_seed(0))
    full = trellis.linear_reference(tw, x)
    acc = sum(trellis.linear_reference(slice_trellis_cols(tw, 4, r), x[:, r * 128:(r + 1) * 128]) for r in range(4))
    assert torch.allclose(acc, full, atol=1e-4)


def test_trellis_column_parallel_is_a_row_subset():
    tw = trellis.random_weight(384, 256, 3, seed=1, sigma=0.05)
    x = torch.randn(2, 256, generator=torch.Generator().manual_seed(0))
    full = trellis.linear_reference(tw, x)
    part = slice_trellis_rows(tw, [(0, 128), (256, 384)])
    got = trellis.linear_reference(part, x)
    assert torch.equal(got, torch.cat([full[:, :128], full[:, 256:]], 1))


def test_w4_slices():
    W = torch.randn(64, 256, generator=torch.Generator().manual_seed(3)) * 0.02
    q = w4a16.quantize(W, 64)
    Wd = w4a16.dequantize(q)
    assert torch.equal(w4a16.dequantize(slice_rows(q, [(16, 32)])), Wd[16:32])
    assert torch.equal(w4a16.dequantize(slice_cols(q, 2, 1)), Wd[:, 128:])


def test_plan_covers_27b_at_every_world():
    cfg = qwen_hybrid_27b_config()
    for world in (2, 4, 8):
        seen_q = []
        for r in range(world):
            plan = shard_plan(cfg, world, r)
            (a, b), = plan["attn.qg"][1]
            seen_q.append((a, b))
            for rng in plan["gdn.in_proj_qkv"][1] + plan["mlp.gate_up"][1]:
                assert rng[0] % 128 == 0 and rng[1] % 128 == 0
            (ka, kb), = plan["attn.k"][1]
            assert (kb - ka) == 256 * max(1, cfg.num_key_value_heads // world)
        assert seen_q[0][0] == 0 and seen_q[-1][1] == 2 * cfg.q_dim
        assert all(seen_q[i][1] == seen_q[i + 1][0] for i in range(world - 1))
    # at world 8 ranks 2r and 2r+1 share KV head r
    p5 = shard_plan(cfg, 8, 5)
    assert p5["attn.k"][1] == [(2 * 256, 3 * 256)]


def test_short_conv_moe_family_shards_add_up():
    """Conv mixers split by channel block (B | C | x thirds each), experts by inner width: per-rank partial outputs of the
    row-parallel halves sum to the unsharded block (fp32 weights, CPU reference ops)."""
    import torch
    from r4dx_b200.config import lfm2_moe_config
    from r4dx_b200.models.oracle import OracleModel, init_weights
    from r4dx_b200.ops import reference as R
    from r4dx_b200.parallel.shard import shard_weight_set
    cfg = lfm2_moe_config(hidden=256, layers=3, heads=4, kv_heads=2, head_dim=64, intermediate=512, experts=4, top_k=2,
                          moe_intermediate=256, dense_layers=1, vocab=4096, attention_layers=(1,))
    w = init_weights(cfg, 7)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 256, generator=g)
    full = OracleModel(cfg, w)
    st = type("S", (), {"conv": {}})()
    ref_conv = full.short_conv("text.layers.0.", 0, x, st)
    ref_exp = full.mlp("text.layers.2.", x, "moe.experts.3")
    ref_dense = full.mlp("text.layers.0.", x)
    world = 2
    acc_conv, acc_exp, acc_dense = 0, 0, 0
    for r in range(world):
        c = cfg.shard(world, r)
        assert c.conv_channels == 128 and c.moe_intermediate_size == 128 and c.intermediate_size == 256
        ws = shard_weight_set(cfg, w, world, r)
        assert ws["text.layers.0.conv.in_proj"].shape == (3 * 128, 256) and ws["text.layers.0.conv.weight"].shape == (128, 3)
        assert ws["text.layers.2.moe.experts.3.gate_up"].shape == (256, 256) and ws["text.layers.2.moe.experts.3.down"].shape == (256, 128)
        assert ws["text.layers.2.moe.router"].shape == (4, 256)          # replicated
        m = OracleModel(c, ws)
        st_r = type("S", (), {"conv": {}})()
        acc_conv = acc_conv + m.short_conv("text.layers.0.", 0, x, st_r)
        acc_exp = acc_exp + m.mlp("text.layers.2.", x, "moe.experts.3")
        acc_dense = acc_dense + m.mlp("text.layers.0.", x)
    assert torch.allclose(acc_conv, ref_conv, atol=1e-5, rtol=1e-4)
    assert torch.allclose(acc_exp, ref_exp, atol=1e-6, rtol=1e-4)
    assert torch.allclose(acc_dense, ref_dense, atol=1e-6, rtol=1e-4)
    import pytest
    with pytest.raises(ValueError):
        cfg.shard(4, 0)               # 64 channels / 64-wide expert slices per rank: not whole 128 blocks
