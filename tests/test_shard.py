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
