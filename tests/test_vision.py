"""Vision tower: host preprocessing on CPU, device encoder against the fp32 restatement."""
import pytest
import torch

from r4dx_b200.models import vision as V


def test_smart_resize_bounds_and_multiples():
    h, w = V.smart_resize(1000, 700, 32, 64 * 64, 512 * 512)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 512 * 512 and abs(h / w - 1000 / 700) < 0.1
    h, w = V.smart_resize(20, 30, 32, 64 * 64, 512 * 512)
    assert h * w >= 64 * 64 and h % 32 == 0 and w % 32 == 0
    with pytest.raises(ValueError):
        V.smart_resize(10, 5000, 32, 1, 10 ** 9)


def test_patch_order_positions_taps_and_segments():
    cfg = V.tiny_vision_config()
    g = torch.Generator().manual_seed(0)
    img = torch.randint(0, 256, (40, 56, 3), generator=g, dtype=torch.uint8)
    patches, grid = V.preprocess_image(img, cfg)
    t, gh, gw = grid
    assert patches.shape == (gh * gw, cfg.patch_dim) and gh % 2 == 0 and gw % 2 == 0
    ids = V.position_ids(grid, 2)
    # merge-major: the first four tokens are the 2x2 block at the top-left corner
    assert ids[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    assert ids[4].tolist() == [0, 2]
    # a patch's content is the normalised pixel block at its (row, column)
    r, c = ids[5].tolist()
    ps = cfg.patch_size
    blk = patches[5].view(3, cfg.temporal_patch_size, ps, ps)
    assert torch.equal(blk[:, 0], blk[:, 1])               # still image: both temporal slots
    idx, wts = V.pos_embed_taps(grid, 8, 2)
    assert idx.shape == (gh * gw, 4) and torch.allclose(wts.sum(-1), torch.ones(gh * gw))
    assert idx.max() < 64 and idx.min() >= 0
    cu = V.segment_offsets([grid, (2, 2, 4)])
    assert cu.tolist() == [0, gh * gw, gh * gw + 8, gh * gw + 16]


def test_reference_attention_is_confined_to_segments():
    cfg = V.tiny_vision_config()
    w = V.init_vision_weights(cfg, 1)
    g = torch.Generator().manual_seed(2)
    grids = [(1, 4, 4), (1, 2, 4)]
    T = 16 + 8
    patches = torch.randn(T, cfg.patch_dim, generator=g)
    ids = torch.cat([V.position_ids(x, 2) for x in grids])
    taps = [V.pos_embed_taps(x, 8, 2) for x in grids]
    idx, wts = torch.cat([a for a, _ in taps]), torch.cat([b for _, b in taps])
    cu = V.segment_offsets(grids)
    full = V.vision_forward_reference(cfg, w, patches, ids, idx, wts, cu)
    first = V.vision_forward_reference(cfg, w, patches[:16], ids[:16], idx[:16], wts[:16], cu[:2])
    assert torch.allclose(full[:4], first, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("D,H,segs", [(72, 2, [70, 130]), (64, 3, [200]), (32, 1, [5, 64, 3])])
def test_vit_rope_and_attention_kernels(D, H, segs):
    from r4dx_b200 import native
    L = native.cuda()
    g = torch.Generator().manual_seed(D)
    T = sum(segs)
    qkv = torch.randn(T, 3, H, D, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 40, (T, 2), generator=g, dtype=torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(segs).cumsum(0)), dtype=torch.int32)
    q = V._rope_ref(qkv[:, 0].float(), pos, 10000.0).to(torch.bfloat16).float()
    k = V._rope_ref(qkv[:, 1].float(), pos, 10000.0).to(torch.bfloat16).float()
    v = qkv[:, 2].float()
    ref = torch.zeros(T, H, D)
    for s in range(len(segs)):
        a, b = int(cu[s]), int(cu[s + 1])
        att = torch.einsum("qhd,khd->hqk", q[a:b], k[a:b]) / D ** 0.5
        ref[a:b] = torch.einsum("hqk,khd->qhd", att.softmax(-1), v[a:b])
    d = qkv.cuda().contiguous()
    st = torch.cuda.current_stream().cuda_stream
    assert L.r4dxb_vit_rope(d.data_ptr(), pos.cuda().data_ptr(), T, H, D, 10000.0, st) == 0
    assert torch.allclose(d[:, 0].float().cpu(), q, atol=2e-2, rtol=2e-2)
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    cud = cu.cuda()
    assert L.r4dxb_vit_attention(d.data_ptr(), out.data_ptr(), cud.data_ptr(), len(segs), T, H, D, st) == 0
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_vision_tower_matches_reference():
    cfg = V.tiny_vision_config()
    w = V.init_vision_weights(cfg, 3)
    g = torch.Generator().manual_seed(4)
    imgs = [torch.randint(0, 256, (48, 64, 3), generator=g, dtype=torch.uint8),
            torch.randint(0, 256, (30, 30, 3), generator=g, dtype=torch.uint8)]
    tower = V.VisionTower(cfg, w)
    got = tower.encode_images(imgs).float().cpu()
    ps, grids = zip(*[V.preprocess_image(i, cfg) for i in imgs])
    ids = torch.cat([V.position_ids(x, 2) for x in grids])
    taps = [V.pos_embed_taps(x, 8, 2) for x in grids]
    ref = V.vision_forward_reference(cfg, w, torch.cat(ps), ids, torch.cat([a for a, _ in taps]),
                                     torch.cat([b for _, b in taps]), V.segment_offsets(grids))
    assert got.shape == ref.shape == (sum(gh * gw for _, gh, gw in grids) // 4, cfg.out_hidden_size)
    assert torch.allclose(got, ref, atol=0.06 * ref.abs().max().item(), rtol=0.05)
