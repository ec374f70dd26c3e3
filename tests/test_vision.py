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


def test_gemma_style_vision_host_half():
    """Preprocessor geometry and raster order, placeholder expansion, image blocks, chunk planning that never cuts a block,
    the per-row key limits against the dense reference mask, and the embedder chain's shapes and rounding."""
    import pytest
    import torch
    from r4dx_b200.models import gemma_vision as GV
    # target size: multiples of 48 inside the budget, aspect kept, small images grown
    for H, W in ((480, 640), (100, 50), (2000, 3000), (48, 48)):
        h, w = GV.target_size(H, W, 280)
        assert h % 48 == 0 and w % 48 == 0 and (h // 48) * (w // 48) <= 280
        assert (h + 48) * (w + 48) > 280 * 48 * 48 * 0.6 and abs(h / w - H / W) < 0.35 * H / W
    with pytest.raises(ValueError):
        GV.target_size(10, 100000, 70)
    with pytest.raises(ValueError):
        GV.target_size(100, 100, 100)
    # an image already at its target size is only rescaled: raster order is checkable exactly
    h, w = GV.target_size(96, 144, 70)
    img = torch.randint(0, 256, (h, w, 3), generator=torch.Generator().manual_seed(0), dtype=torch.uint8)
    px, pos, (gh, gw) = GV.preprocess(img, 70)
    assert px.shape == (gh * gw, 6912) and pos.shape == (gh * gw, 2) and (gh, gw) == (h // 48, w // 48)
    r, c = 1 % gh, 2 % gw
    patch = px[r * gw + c].view(48, 48, 3)
    assert torch.allclose(patch, img[r * 48:(r + 1) * 48, c * 48:(c + 1) * 48].float() * (1.0 / 255.0))
    assert pos[r * gw + c].tolist() == [c, r]
    # placeholders and blocks
    toks, spans = GV.expand_placeholders([5, 9, 6, 9, 7], [3, 2], image_id=9, boi_id=1, eoi_id=2)
    assert toks == [5, 1, 9, 9, 9, 2, 6, 1, 9, 9, 2, 7] and spans == [(2, 3), (8, 2)]
    blocks = GV.find_blocks(toks, 9, base=100)
    assert blocks == [(102, 105), (108, 110)]
    with pytest.raises(ValueError):
        GV.expand_placeholders([9], [1, 1], 9, 1, 2)
    # chunk planning: no block is ever cut, every row is covered once
    blocks = [(3, 9), (10, 14), (20, 27)]
    for max_rows in (7, 8, 12, 100):
        chunks = GV.plan_prefill_chunks(30, blocks, max_rows, max_block=8)
        assert sum(n for _, n in chunks) == 30 and chunks[0][0] == 0
        assert all(chunks[i][0] + chunks[i][1] == chunks[i + 1][0] for i in range(len(chunks) - 1))
        for s, n in chunks:
            assert all(not (a < s + n < b) and not (a < s < b) for a, b in blocks), (max_rows, chunks)
    with pytest.raises(ValueError):
        GV.plan_prefill_chunks(30, [(0, 20)], 8, max_block=8)
    # key limits reproduce the dense mask of a sliding layer
    T, window = 30, 6
    ext = GV.key_limit_ext(0, T, blocks)
    mask = GV.dense_mask(T, window, True, blocks)
    for q in range(T):
        hi = max(q, int(ext[q]))
        want = torch.zeros(T, dtype=torch.bool)
        want[max(0, q - window + 1):hi + 1] = True
        assert torch.equal(mask[q], want), q
    assert torch.equal(GV.dense_mask(T, 0, False, blocks), torch.tril(torch.ones(T, T, dtype=torch.bool)))
    # embedder chain
    g = torch.Generator().manual_seed(1)
    n = lambda *s: torch.randn(*s, generator=g) * 0.05
    mm, out = 64, 32
    w = GV.GemmaEmbedderWeights(1 + n(6912), n(6912), n(mm, 6912), n(mm), 1 + n(mm), n(mm), n(16, 2, mm), 1 + n(mm), n(mm), n(out, mm))
    rows = GV.embed_reference(px, pos, w)
    assert rows.shape == (gh * gw, out) and torch.equal(rows, rows.to(torch.bfloat16).float())
    assert torch.equal(GV.embed_reference(px[2:3], pos[2:3], w), rows[2:3])       # rows are independent
    moved = GV.embed_reference(px, torch.flip(pos, [1]), w)
    assert not torch.equal(moved, rows)                                           # the position terms matter


@pytest.mark.gpu
def test_gemma_embedder_on_the_device_matches_the_host_chain():
    from r4dx_b200.models import gemma_vision as GV
    g = torch.Generator().manual_seed(4)
    n = lambda *s: torch.randn(*s, generator=g) * 0.05
    mm, out, pd, rows = 128, 256, 6912, 37
    w = GV.GemmaEmbedderWeights(1 + n(pd), n(pd), n(mm, pd), n(mm), 1 + n(mm), n(mm), n(16, 2, mm), 1 + n(mm), n(mm), n(out, mm))
    px = torch.rand(rows, pd, generator=g)
    pos = torch.randint(0, 16, (rows, 2), generator=g)
    ref = GV.embed_reference(px, pos, w)
    got = GV.GemmaEmbedder(w).embed(px, pos).float().cpu()
    assert got.shape == ref.shape
    assert (got - ref).abs().max().item() < 0.03 * ref.abs().max().item()


@pytest.mark.gpu
@pytest.mark.parametrize("D,window", [(64, 24), (256, 40), (128, 0)])
def test_prefill_attention_with_per_row_key_limits(D, window):
    """Rows of a block see keys up to the block's end: the windowed prefill kernel against the reference attention."""
    from r4dx_b200.models import gemma_vision as GV
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.ops import reference as R
    g = torch.Generator().manual_seed(D)
    T, Hq, Hkv, pos0 = 90, 4, 2, 0
    blocks = [(7, 23), (40, 71)]
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    k = (torch.randn(T, Hkv, D, generator=g) * 0.5)
    v = (torch.randn(T, Hkv, D, generator=g) * 0.5)
    lim = GV.key_limit_ext(pos0, T, blocks)
    nblk = (T + 15) // 16
    dev = "cuda"
    cache = torch.zeros(nblk, Hkv, 2, 16, D, dtype=torch.uint8, device=dev)
    k8 = (k * 16).to(torch.float8_e4m3fn)
    v8 = (v * 16).to(torch.float8_e4m3fn)
    for t in range(T):
        cache[t // 16, :, 0, t % 16] = k8[t].view(torch.uint8).to(dev)
        cache[t // 16, :, 1, t % 16] = v8[t].view(torch.uint8).to(dev)
    table = torch.arange(nblk, dtype=torch.int32, device=dev)
    ds = torch.full((Hkv,), 1 / 16.0, device=dev)
    out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=dev)
    qg = torch.zeros(T, Hq, 2 * D, dtype=torch.bfloat16, device=dev)
    K.attn_prefill(q.to(dev), qg, cache, table, ds, ds, out, T, Hq, Hkv, D, pos0, gated=False, window=window, key_limit=lim.to(dev))
    kd, vd = k8.float() / 16, v8.float() / 16
    ref = R.causal_gqa_attention(q.float(), kd, vd, pos0, window=window, key_limit=lim).reshape(T, Hq * D)
    assert (out.float().cpu() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 1e-3
    # without the limits the block rows come out differently
    K.attn_prefill(q.to(dev), qg, cache, table, ds, ds, out, T, Hq, Hkv, D, pos0, gated=False, window=window)
    assert (out.float().cpu() - ref).abs().max().item() > 0.05 * ref.abs().max().item()
