"""CUDA kernels vs the plain PyTorch fp32 reference of the same op (needs a B200)."""
import math

import pytest
import torch

from r4dx_b200.ops import reference as R

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def K():
    from r4dx_b200.ops import kernels
    from r4dx_b200 import native
    native.cuda()
    return kernels


def _bf(t):
    return t.to(BF).cuda()


def test_native_library_is_loaded(K):
    from r4dx_b200 import native
    assert native.cuda_loaded()


def test_embed_rmsnorm_silu(K):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(100, 256, generator=g)
    ids = torch.tensor([3, 99, 0, 250, -4], dtype=torch.int32)
    out = K.embed_gather(ids.cuda(), _bf(table))
    exp = table.to(BF)[ids.clamp(0, 99).long()]
    assert torch.equal(out.cpu(), exp)

    x = torch.randn(5, 5120, generator=g)
    w = torch.randn(5120, generator=g) * 0.1
    y = K.rmsnorm(_bf(x), _bf(w))
    ref = R.rmsnorm_1pw(x.to(BF), w.to(BF))
    assert torch.allclose(y.float().cpu(), ref, atol=2e-2, rtol=1e-2)
    y2 = K.rmsnorm(_bf(x), _bf(w), zero_centered=False)
    assert torch.allclose(y2.float().cpu(), R.rmsnorm_plain(x.to(BF), w.to(BF)), atol=2e-2, rtol=1e-2)

    res = _bf(x.clone())
    delta = _bf(torch.randn(5, 5120, generator=g))
    res0 = res.clone()
    y3 = K.add_rmsnorm(res, delta, _bf(w))
    summed = (res0.float() + delta.float()).to(BF)
    assert torch.equal(res, summed)
    assert torch.allclose(y3.float().cpu(), R.rmsnorm_1pw(summed.cpu(), w.to(BF)), atol=2e-2, rtol=1e-2)

    gu = torch.randn(3, 2 * 1024, generator=g)
    act = K.silu_mul(_bf(gu))
    assert torch.allclose(act.float().cpu(), R.silu_mul(gu.to(BF)), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("kb", [3, 4, 5])
@pytest.mark.parametrize("T,ksplit", [(1, 1), (1, 4), (3, 2), (8, 8)])
def test_trellis_gemv(K, kb, T, ksplit):
    from r4dx_b200.quant import trellis
    N, Kd = 256, 1024
    tw = trellis.random_weight(N, Kd, kb, seed=kb * 10 + T, sigma=0.02)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, Kd, generator=g).to(BF)
    res = torch.randn(T, N, generator=g).to(BF)
    ref = trellis.linear_reference(tw, x.float())
    y = K.trellis_gemv(tw.to("cuda"), x.cuda(), ksplit=ksplit)
    scale = ref.abs().max().item()
    assert (y.float().cpu() - ref).abs().max().item() < 0.02 * scale + 1e-3
    y2 = K.trellis_gemv(tw.to("cuda"), x.cuda(), residual=res.cuda(), ksplit=ksplit)
    assert (y2.float().cpu() - (ref + res.float())).abs().max().item() < 0.02 * (scale + 3) + 1e-3


@pytest.mark.parametrize("kb", [3, 4, 5])
@pytest.mark.parametrize("T,ksplit,Kd", [(1, 2, 5120), (4, 8, 17408), (8, 1, 1024), (2, 4, 6144)])
def test_trellis_gemv_tensor_memory_path_against_reference_and_cuda_core_path(K, kb, T, ksplit, Kd):
    """The int8 tcgen05 path (hash words in tensor memory) and the CUDA-core path compute the same linear map."""
    from r4dx_b200.quant import trellis
    N = 256
    tw = trellis.random_weight(N, Kd, kb, seed=kb + T, sigma=0.02)
    x = torch.randn(T, Kd, generator=torch.Generator().manual_seed(T + Kd)).to(BF)
    ref = trellis.linear_reference(tw, x.float())
    twd, xd = tw.to("cuda"), x.cuda()
    scale = ref.abs().max().item()
    impl0 = K.GEMV_IMPL
    try:
        K.set_gemv_impl("mma")
        y_mma = K.trellis_gemv(twd, xd, ksplit=ksplit).float().cpu()
        K.check_gemm_status("cuda")
        K.set_gemv_impl("simt")
        y_simt = K.trellis_gemv(twd, xd, ksplit=ksplit).float().cpu()
    finally:
        K.set_gemv_impl(impl0)
    assert (y_mma - ref).abs().max().item() < 0.01 * scale + 1e-3        # exact integer sums: tighter than the fp16 path
    assert (y_simt - ref).abs().max().item() < 0.02 * scale + 1e-3
    assert (y_mma - y_simt).abs().max().item() < 0.02 * scale + 1e-3


def test_trellis_gemv_one_hot_returns_decoded_rows(K):
    """x = e_k after undoing the input transform picks out column k of H Q H exactly (up to bf16)."""
    from r4dx_b200.quant import trellis
    tw = trellis.random_weight(128, 128, 4, seed=3, sigma=1.0)
    Wr = trellis.reconstruct(tw)
    x = torch.zeros(2, 128)
    x[0, 5] = 1.0
    x[1, 77] = 2.0
    y = K.trellis_gemv(tw.to("cuda"), _bf(x), ksplit=1).float().cpu()
    assert torch.allclose(y[0], Wr[:, 5], atol=0.03, rtol=0.02)
    assert torch.allclose(y[1], 2 * Wr[:, 77], atol=0.06, rtol=0.02)


@pytest.mark.parametrize("T,ksplit", [(1, 1), (3, 2), (8, 4)])
def test_sibling_launch_equals_separate_launches(K, T, ksplit):
    """Three weights of one K and bit width in one launch give bit-identical rows to three launches."""
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(T)
    ws = [trellis.random_weight(n, 640, 4, seed=n, sigma=0.05).to("cuda") for n in (384, 128, 256)]
    x = torch.randn(T, 640, generator=g).to(BF).cuda()
    nw = (torch.randn(640, generator=g) * 0.1).to(BF).cuda()
    grp = K.SiblingGroup(ws)
    grp.ksplit = ksplit
    outs = [torch.zeros(T, w.N, dtype=BF, device="cuda") for w in ws]
    grp(x, outs, prologue=K.PRO_RMSNORM, norm_w=nw, eps=1e-6)
    for w, o in zip(ws, outs):
        ref = K.trellis_gemv(w, x, ksplit=ksplit, prologue=K.PRO_RMSNORM, norm_w=nw, eps=1e-6)
        assert torch.equal(o, ref)


@pytest.mark.parametrize("ksplit", [2, 4, 8])
def test_trellis_gemv_uneven_k_split(K, ksplit):
    """17 K blocks over 2 / 4 / 8 CTAs of a cluster (uneven slices) against the unsplit launch and the reference."""
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(ksplit)
    w = trellis.random_weight(256, 17 * 128, 5, seed=9, sigma=0.05)
    x = torch.randn(4, 17 * 128, generator=g).to(BF)
    ref = trellis.linear_reference(w, x.float())
    y1 = K.trellis_gemv(w.to("cuda"), x.cuda(), ksplit=1).float().cpu()
    ys = K.trellis_gemv(w.to("cuda"), x.cuda(), ksplit=ksplit).float().cpu()
    scale = ref.abs().max().item()
    assert (ys - ref).abs().max().item() < 0.02 * scale
    assert (ys - y1).abs().max().item() < 0.01 * scale


@pytest.mark.parametrize("T", [1, 2, 5, 8])
def test_w4a16_gemv_and_argmax(K, T):
    from r4dx_b200.quant import w4a16
    g = torch.Generator().manual_seed(T)
    W = torch.randn(1000, 512, generator=g) * 0.02
    q = w4a16.quantize(W, 64)
    Wd = w4a16.dequantize(q)
    x = torch.randn(T, 512, generator=g).to(BF)
    y = K.w4a16_gemv(q.to("cuda"), x.cuda())
    ref = x.float() @ Wd.T
    assert torch.allclose(y.cpu(), ref, atol=5e-3, rtol=1e-2)
    ids, vals = K.argmax_rows(y, id_offset=7)
    assert torch.equal(ids.cpu().long(), y.cpu().argmax(-1) + 7)


@pytest.mark.parametrize("T,N,Kd,group", [(16, 256, 512, 64), (40, 1024, 1024, 32), (300, 512, 2048, 128), (1100, 384, 640, 64)])
def test_linear_tc_w4a16_matches_fp32_reference(K, T, N, Kd, group):
    """The tensor-core w4a16 product against x @ dequant(W)^T in fp32, with bias, residual and an fp32 output."""
    from r4dx_b200.quant import w4a16
    g = torch.Generator().manual_seed(T + N)
    W = torch.randn(N, Kd, generator=g) * 0.03
    q = w4a16.quantize(W, group)
    Wd = w4a16.dequantize(q)
    x = torch.randn(T, Kd, generator=g).to(BF)
    ref = x.half().float() @ Wd.T
    y = K.linear_tc(q.to("cuda"), x.cuda(), out_f32=True)
    K.check_gemm_status(y.device)
    assert torch.allclose(y.cpu(), ref, atol=2e-2, rtol=1e-2)
    bias = torch.randn(N, generator=g).to(BF)
    res = torch.randn(T, N, generator=g).to(BF)
    y2 = K.linear_tc(q.to("cuda"), x.cuda(), bias=bias.cuda(), residual=res.cuda())
    K.check_gemm_status(y2.device)
    assert y2.dtype == BF
    assert torch.allclose(y2.float().cpu(), ref + bias.float() + res.float(), atol=6e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,Kd", [(24, 256, 384), (520, 1152, 1152), (2050, 128, 4352), (70, 4304, 1152), (33, 1152, 4304), (9, 20, 72)])
def test_linear_tc_dense_matches_fp32_reference(K, dtype, T, N, Kd):
    g = torch.Generator().manual_seed(N + Kd)
    W = (torch.randn(N, Kd, generator=g) * 0.05).to(dtype)
    x = torch.randn(T, Kd, generator=g).to(dtype)
    bias = torch.randn(N, generator=g).to(BF)
    ref = x.float() @ W.float().T + bias.float()
    y = K.linear_tc(W.cuda(), x.cuda(), bias=bias.cuda(), out_f32=True)
    K.check_gemm_status(y.device)
    assert torch.allclose(y.cpu(), ref, atol=3e-2, rtol=1e-2)
    yb = K.linear_tc(W.cuda(), x.cuda(), bias=bias.cuda())
    assert torch.allclose(yb.float().cpu(), ref, atol=8e-2, rtol=2e-2)
    for act, fn in ((1, lambda v: torch.nn.functional.gelu(v, approximate="tanh")), (2, torch.nn.functional.gelu)):
        ya = K.linear_tc(W.cuda(), x.cuda(), bias=bias.cuda(), act=act, out_f32=True)
        assert torch.allclose(ya.cpu(), fn(ref), atol=3e-2, rtol=1e-2)


def test_argmax_ties_take_lowest_id(K):
    lg = torch.zeros(2, 5000, device="cuda")
    lg[0, 4000] = 1.0
    lg[0, 123] = 1.0
    lg[1, 4999] = 2.0
    ids, vals = K.argmax_rows(lg)
    assert ids.tolist() == [123, 4999] and vals.tolist() == [1.0, 2.0]
    ids, _ = K.argmax_rows(lg.to(BF))
    assert ids.tolist() == [123, 4999]


def test_bf16_gemv(K):
    g = torch.Generator().manual_seed(0)
    W = torch.randn(96, 1024, generator=g).to(BF)
    x = torch.randn(4, 1024, generator=g).to(BF)
    y = K.bf16_gemv(W.cuda(), x.cuda())
    assert torch.allclose(y.cpu(), x.float() @ W.float().T, atol=1e-2, rtol=1e-3)


@pytest.mark.parametrize("T", [1, 3, 8])
def test_gdn_decode_with_in_kernel_ab_projection(K, T):
    """The a / b projections computed inside the GDN kernel give the rows of the stand-alone norm + product kernel."""
    g = torch.Generator().manual_seed(T)
    D, Hv, Hk, Kd = 128, 6, 2, 1024
    conv_dim = 2 * Hk * D + Hv * D
    dev = "cuda"
    mixed = (torch.randn(T, conv_dim, generator=g) * 0.5).to(BF).to(dev)
    z = torch.randn(T, Hv * D, generator=g).to(BF).to(dev)
    x = torch.randn(T, Kd, generator=g).to(BF).to(dev)
    nw = (torch.randn(Kd, generator=g) * 0.1).to(BF).to(dev)
    ab_w = (torch.randn(2 * Hv, Kd, generator=g) * 0.05).to(BF).to(dev)
    conv_w = (torch.randn(conv_dim, 4, generator=g) * 0.5).to(BF).to(dev)
    A_log = (torch.randn(Hv, generator=g) * 0.3).to(dev)
    dt_bias = (torch.randn(Hv, generator=g) * 0.3).to(dev)
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF).to(dev)
    positions = torch.arange(0, T, dtype=torch.int32, device=dev)
    outs, logs = [], []
    for fused in (False, True):
        ring = torch.zeros(16, conv_dim, dtype=BF, device=dev)
        state = torch.zeros(Hv, D, D, device=dev)
        log_u, log_k = torch.zeros(8, Hv, D, device=dev), torch.zeros(8, Hv, D, device=dev)
        log_eg = torch.zeros(8, Hv, device=dev)
        n_replay = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.zeros(8, Hv * D, dtype=BF, device=dev)
        ab = torch.zeros(T, 2 * Hv, device=dev)
        if not fused:
            K.bf16_gemv_norm(ab_w, x, nw, 1e-6, ab)
        K.gdn_decode(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, log_u, log_k, log_eg, positions, n_replay,
                     out, T, Hv, Hk, D, ab_w=ab_w if fused else None, x=x, in_norm_w=nw, in_eps=1e-6)
        outs.append(out[:T].float().cpu())
        logs.append(log_eg[:T].cpu())
    assert torch.allclose(logs[0], logs[1], atol=1e-5, rtol=1e-4)
    assert torch.allclose(outs[0], outs[1], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("D,Hv,Hk", [(128, 6, 2), (64, 4, 2)])
def test_gdn_decode_matches_recurrence_with_rollback(K, D, Hv, Hk):
    """Rows are fed in windows; only an accepted prefix of each window is committed."""
    g = torch.Generator().manual_seed(D)
    key_dim, conv_dim = Hk * D, 2 * Hk * D + Hv * D
    n_tok = 40
    mixed = (torch.randn(n_tok, conv_dim, generator=g) * 0.5).to(BF)
    z = torch.randn(n_tok, Hv * D, generator=g).to(BF)
    ab = torch.randn(n_tok, 2 * Hv, generator=g)
    conv_w = (torch.randn(conv_dim, 4, generator=g) * 0.5).to(BF)
    A_log = torch.randn(Hv, generator=g) * 0.3
    dt_bias = torch.randn(Hv, generator=g) * 0.3
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    # reference over the full accepted sequence
    y, _ = R.causal_conv1d_silu(mixed.float(), conv_w.float(), None)
    q = R.l2norm(y[:, :key_dim].view(n_tok, Hk, D))
    k = R.l2norm(y[:, key_dim:2 * key_dim].view(n_tok, Hk, D))
    v = y[:, 2 * key_dim:].view(n_tok, Hv, D)
    gg, beta = R.gdn_gates(ab[:, :Hv], ab[:, Hv:], A_log, dt_bias)
    o, S_ref = R.gdn_recurrent(q, k, v, gg, beta, None)
    ref = R.gated_rmsnorm(o, z.float().view(n_tok, Hv, D), norm_w.float()).view(n_tok, Hv * D)

    dev = "cuda"
    ring = torch.zeros(16, conv_dim, dtype=BF, device=dev)
    state = torch.zeros(Hv, D, D, device=dev)
    log_u = torch.zeros(8, Hv, D, device=dev)
    log_k = torch.zeros(8, Hv, D, device=dev)
    log_eg = torch.zeros(8, Hv, device=dev)
    n_replay = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(8, Hv * D, dtype=BF, device=dev)
    got = torch.zeros(n_tok, Hv * D)
    pos = 0
    gj = torch.Generator().manual_seed(1)
    pending = 0
    while pos < n_tok:
        T = min(int(torch.randint(1, 9, (1,), generator=gj)), n_tok - pos)
        acc = int(torch.randint(1, T + 1, (1,), generator=gj))
        # rejected rows carry junk that must leave no trace
        rows_m = mixed[pos:pos + T].clone()
        rows_z = z[pos:pos + T].clone()
        rows_ab = ab[pos:pos + T].clone()
        if acc < T:
            rows_m[acc:] = 3.0
            rows_ab[acc:] = -1.0
        positions = torch.arange(pos, pos + T, dtype=torch.int32, device=dev)
        n_replay.fill_(pending)
        K.gdn_decode(rows_m.cuda(), rows_z.cuda(), rows_ab.cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(),
                     norm_w.cuda(), ring, state, log_u, log_k, log_eg, positions, n_replay, out, T, Hv, Hk, D)
        got[pos:pos + acc] = out[:acc].float().cpu()
        pending = acc
        pos += acc
    assert torch.allclose(got, ref, atol=3e-2, rtol=3e-2)
    # commit the tail and compare the state
    n_replay.fill_(pending)
    K.gdn_decode(mixed[:1].cuda(), z[:1].cuda(), ab[:1].cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(),
                 norm_w.cuda(), ring, state, log_u, log_k, log_eg, torch.zeros(1, dtype=torch.int32, device=dev),
                 n_replay, out, 0, Hv, Hk, D)
    assert torch.allclose(state.cpu(), S_ref, atol=2e-3, rtol=2e-2)


@pytest.mark.parametrize("Hv,Hk,T", [(2, 1, 128), (6, 2, 333), (3, 3, 1000)])
def test_gdn_chunked_prefill_matches_recurrence(K, Hv, Hk, T):
    """The chunked tensor-core form against the fp32 token-by-token reference, and against the scan kernel's state."""
    D = 128
    g = torch.Generator().manual_seed(T)
    key_dim, conv_dim = Hk * D, 2 * Hk * D + Hv * D
    mixed = (torch.randn(T, conv_dim, generator=g) * 0.5).to(BF)
    z = torch.randn(T, Hv * D, generator=g).to(BF)
    ab = torch.randn(T, 2 * Hv, generator=g)
    ab[:, :Hv] += 1.0
    conv_w = (torch.randn(conv_dim, 4, generator=g) * 0.5).to(BF)
    A_log = torch.randn(Hv, generator=g) * 0.3
    dt_bias = torch.randn(Hv, generator=g) * 0.3
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    y, _ = R.causal_conv1d_silu(mixed.float(), conv_w.float(), None)
    q = R.l2norm(y[:, :key_dim].view(T, Hk, D))
    k = R.l2norm(y[:, key_dim:2 * key_dim].view(T, Hk, D))
    v = y[:, 2 * key_dim:].view(T, Hv, D)
    gg, beta = R.gdn_gates(ab[:, :Hv], ab[:, Hv:], A_log, dt_bias)
    o, S_ref = R.gdn_recurrent(q, k, v, gg, beta, None)
    ref = R.gated_rmsnorm(o, z.float().view(T, Hv, D), norm_w.float()).view(T, Hv * D)
    dev = "cuda"
    outs, states = [], []
    for use_ws in (True, False):
        ring = torch.zeros(16, conv_dim, dtype=BF, device=dev)
        state = torch.zeros(Hv, D, D, device=dev)
        out = torch.zeros(T, Hv * D, dtype=BF, device=dev)
        sc = dict(q=torch.empty(T, Hk, D, device=dev), k=torch.empty(T, Hk, D, device=dev), v=torch.empty(T, Hv, D, device=dev),
                  o=torch.empty(T, Hv, D, device=dev), eg=torch.empty(T, Hv, device=dev), beta=torch.empty(T, Hv, device=dev))
        if use_ws:
            sc["ws"] = torch.full((K.gdn_chunk_ws_floats(T, Hv),), float("nan"), device=dev)
        K.gdn_prefill(mixed.cuda(), z.cuda(), ab.cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(), norm_w.cuda(), ring, state,
                      sc, out, T, Hv, Hk, D, 0)
        outs.append(out.float().cpu())
        states.append(state.cpu())
    assert torch.allclose(outs[0], ref, atol=3e-2, rtol=3e-2)
    assert torch.allclose(outs[0], outs[1], atol=3e-2, rtol=3e-2)
    # S_ref is [H, Dk, Dv] or [H, Dv, Dk] depending on the reference's convention: compare with the scan kernel's state
    rel = (states[0] - states[1]).norm() / states[1].norm()
    assert rel < 5e-3, rel


@pytest.mark.parametrize("D,Hq,Hkv,T,ctx", [(256, 6, 1, 1, 100), (256, 12, 2, 4, 333), (64, 4, 2, 8, 40), (256, 24, 4, 1, 1500)])
def test_attention_precore_and_decode(K, D, Hq, Hkv, T, ctx):
    g = torch.Generator().manual_seed(ctx)
    dev = "cuda"
    rd = D // 4
    theta = 1e7
    nblk = (ctx + T + 15) // 16 + 1
    cache = torch.zeros(nblk, Hkv, 2, 16, D, dtype=torch.uint8, device=dev)
    # shuffled physical blocks exercise the block table
    table = torch.randperm(nblk, generator=g).to(torch.int32).cuda()
    qn = (torch.randn(D, generator=g) * 0.1).to(BF)
    kn = (torch.randn(D, generator=g) * 0.1).to(BF)
    kds = torch.full((Hkv,), 1 / 8.0)
    vds = torch.full((Hkv,), 1 / 16.0)
    total = ctx + T
    qg_all = torch.randn(total, Hq, 2 * D, generator=g).to(BF)
    k_all = torch.randn(total, Hkv, D, generator=g).to(BF)
    v_all = torch.randn(total, Hkv, D, generator=g).to(BF)
    q_out = torch.zeros(8, Hq, D, dtype=BF, device=dev)
    # fill the context through the precore kernel, 8 rows per call
    for s in range(0, ctx, 8):
        e = min(ctx, s + 8)
        pos = torch.arange(s, e, dtype=torch.int32, device=dev)
        K.attn_precore(qg_all[s:e].cuda(), k_all[s:e].cuda(), v_all[s:e].cuda(), qn.cuda(), kn.cuda(), kds.cuda(),
                       vds.cuda(), pos, table, q_out, cache, e - s, Hq, Hkv, D, rd, theta)
    pos = torch.arange(ctx, ctx + T, dtype=torch.int32, device=dev)
    qg_new = qg_all[ctx:].cuda().contiguous()
    K.attn_precore(qg_new, k_all[ctx:].cuda(), v_all[ctx:].cuda(), qn.cuda(), kn.cuda(), kds.cuda(), vds.cuda(), pos,
                   table, q_out, cache, T, Hq, Hkv, D, rd, theta)
    splits = 5
    G = Hq // Hkv * T
    part_acc = torch.zeros(splits * Hkv * G * D, device=dev)
    part_ml = torch.zeros(splits * Hkv * G * 2, device=dev)
    out = torch.zeros(T, Hq * D, dtype=BF, device=dev)
    K.attn_decode(q_out, qg_new, cache, table, pos, kds.cuda(), vds.cuda(), part_acc, part_ml, out, T, Hq, Hkv, D,
                  splits, True)
    # reference
    allpos = torch.arange(total)
    qf = R.rope_partial_neox(R.rmsnorm_1pw(qg_all[..., :D], qn), allpos, rd, theta)
    kf = R.rope_partial_neox(R.rmsnorm_1pw(k_all, kn), allpos, rd, theta)
    kq = R.fp8_e4m3_roundtrip(kf, 1 / 8.0)
    vq = R.fp8_e4m3_roundtrip(v_all.float(), 1 / 16.0)
    assert torch.allclose(q_out[:T].float().cpu(), qf[ctx:].to(BF).float(), atol=3e-2, rtol=2e-2)
    o = R.causal_gqa_attention(qf[ctx:].to(BF), kq, vq, ctx)
    o = o * torch.sigmoid(qg_all[ctx:, :, D:].float())
    K.set_attn_prefill_impl("tc")
    K.check_gemm_status("cuda")
    assert torch.allclose(out.float().cpu().view(T, Hq, D), o, atol=2e-2, rtol=3e-2)


def test_bf16_gemv_many_rows(K):
    g = torch.Generator().manual_seed(5)
    W = torch.randn(96, 1024, generator=g).to(BF)
    x = torch.randn(37, 1024, generator=g).to(BF)
    y = K.bf16_gemv(W.cuda(), x.cuda())
    assert torch.allclose(y.cpu(), x.float() @ W.float().T, atol=1e-2, rtol=1e-3)


def test_gdn_chunked_prefill_with_gates_of_thousands_of_nats_per_chunk(K):
    """Per-step decays from exp(-0.03) to exp(-158) (A = exp(A_log), A_log from -3.5 to 5.06): a 64-token chunk's summed
    log-gates reach ~10^4, far past where a decay split around the chunk's midpoint overflows.  The chunked kernel forms each
    pair decay as exp(G_i - G_j) <= 1, so it must still equal the token-by-token recurrence; both with the sigmoid gate."""
    D, Hv, Hk, T = 128, 8, 2, 300
    g = torch.Generator().manual_seed(77)
    key_dim, conv_dim = Hk * D, 2 * Hk * D + Hv * D
    mixed = (torch.randn(T, conv_dim, generator=g) * 0.5).to(BF)
    z = torch.randn(T, Hv * D, generator=g).to(BF)
    ab = torch.randn(T, 2 * Hv, generator=g)
    conv_w = (torch.randn(conv_dim, 4, generator=g) * 0.5).to(BF)
    A_log = torch.linspace(-3.5, 5.06, Hv)
    dt_bias = torch.linspace(-6.0, 1.0, Hv)
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    y, _ = R.causal_conv1d_silu(mixed.float(), conv_w.float(), None)
    q = R.l2norm(y[:, :key_dim].view(T, Hk, D))
    k = R.l2norm(y[:, key_dim:2 * key_dim].view(T, Hk, D))
    v = y[:, 2 * key_dim:].view(T, Hv, D)
    gg, beta = R.gdn_gates(ab[:, :Hv], ab[:, Hv:], A_log, dt_bias)
    assert float((-gg[:64].sum(0)).max()) > 5000                     # the widest head's first chunk spans hundreds of nats at least
    o, _ = R.gdn_recurrent(q, k, v, gg, beta, None)
    ref = (R.rmsnorm_plain(o, norm_w.float(), 1e-6) * torch.sigmoid(z.float().view(T, Hv, D))).view(T, Hv * D)
    dev = "cuda"
    outs, states = [], []
    for exact in (False, True):
        ring = torch.zeros(16, conv_dim, dtype=BF, device=dev)
        state = torch.zeros(Hv, D, D, device=dev)
        out = torch.zeros(T, Hv * D, dtype=BF, device=dev)
        sc = dict(q=torch.empty(T, Hk, D, device=dev), k=torch.empty(T, Hk, D, device=dev), v=torch.empty(T, Hv, D, device=dev),
                  o=torch.empty(T, Hv, D, device=dev), eg=torch.empty(T, Hv, device=dev), beta=torch.empty(T, Hv, device=dev),
                  ws=torch.full((K.gdn_chunk_ws_floats(T, Hv),), float("nan"), device=dev))
        K.gdn_prefill_gate(mixed.cuda(), z.cuda(), ab.cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(), norm_w.cuda(), ring, state,
                           sc, out, T, Hv, Hk, D, 0, 1e-6, 1, exact_scan=exact)
        outs.append(out.float().cpu())
        states.append(state.cpu())
    assert bool(torch.isfinite(outs[0]).all()) and bool(torch.isfinite(states[0]).all())
    assert torch.allclose(outs[1], ref, atol=3e-2, rtol=3e-2)
    assert torch.allclose(outs[0], ref, atol=3e-2, rtol=3e-2)
    assert (states[0] - states[1]).norm() / states[1].norm() < 5e-3


@pytest.mark.parametrize("D,Hv,Hk,T", [(128, 6, 2, 70), (64, 4, 2, 33)])
def test_gdn_prefill_matches_recurrence_and_hands_over_to_decode(K, D, Hv, Hk, T):
    g = torch.Generator().manual_seed(D + T)
    key_dim, conv_dim = Hk * D, 2 * Hk * D + Hv * D
    n_tok = T + 5
    mixed = (torch.randn(n_tok, conv_dim, generator=g) * 0.5).to(BF)
    z = torch.randn(n_tok, Hv * D, generator=g).to(BF)
    ab = torch.randn(n_tok, 2 * Hv, generator=g)
    conv_w = (torch.randn(conv_dim, 4, generator=g) * 0.5).to(BF)
    A_log = torch.randn(Hv, generator=g) * 0.3
    dt_bias = torch.randn(Hv, generator=g) * 0.3
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    y, _ = R.causal_conv1d_silu(mixed.float(), conv_w.float(), None)
    q = R.l2norm(y[:, :key_dim].view(n_tok, Hk, D))
    k = R.l2norm(y[:, key_dim:2 * key_dim].view(n_tok, Hk, D))
    v = y[:, 2 * key_dim:].view(n_tok, Hv, D)
    gg, beta = R.gdn_gates(ab[:, :Hv], ab[:, Hv:], A_log, dt_bias)
    o, S_ref = R.gdn_recurrent(q, k, v, gg, beta, None)
    ref = R.gated_rmsnorm(o, z.float().view(n_tok, Hv, D), norm_w.float()).view(n_tok, Hv * D)
    dev = "cuda"
    f32 = torch.float32
    ring = torch.zeros(16, conv_dim, dtype=BF, device=dev)
    state = torch.zeros(Hv, D, D, device=dev)
    # two prefill chunks (the second starts mid-ring), then decode rows
    split = T // 2 + 3
    out = torch.zeros(n_tok, Hv * D, dtype=BF, device=dev)
    for s, e in ((0, split), (split, T)):
        n = e - s
        sc = dict(q=torch.empty(n, Hk, D, device=dev), k=torch.empty(n, Hk, D, device=dev), v=torch.empty(n, Hv, D, device=dev),
                  o=torch.empty(n, Hv, D, device=dev), eg=torch.empty(n, Hv, device=dev), beta=torch.empty(n, Hv, device=dev))
        K.gdn_prefill(mixed[s:e].cuda(), z[s:e].cuda(), ab[s:e].cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(),
                      norm_w.cuda(), ring, state, sc, out[s:e], n, Hv, Hk, D, s)
    log_u = torch.zeros(8, Hv, D, device=dev); log_k = torch.zeros(8, Hv, D, device=dev); log_eg = torch.zeros(8, Hv, device=dev)
    n_replay = torch.zeros(1, dtype=torch.int32, device=dev)
    dec = torch.zeros(8, Hv * D, dtype=BF, device=dev)
    K.gdn_decode(mixed[T:].cuda(), z[T:].cuda(), ab[T:].cuda(), conv_w.cuda(), A_log.cuda(), dt_bias.cuda(), norm_w.cuda(),
                 ring, state, log_u, log_k, log_eg, torch.arange(T, n_tok, dtype=torch.int32, device=dev), n_replay, dec,
                 5, Hv, Hk, D)
    out[T:] = dec[:5]
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("impl", ["tc", "mma"])
@pytest.mark.parametrize("D,Hq,Hkv,T,ctx", [(256, 6, 1, 40, 0), (256, 12, 2, 70, 100), (64, 4, 2, 33, 17), (256, 3, 1, 20, 64),
                                            (256, 6, 1, 300, 0), (256, 4, 2, 257, 391), (128, 4, 1, 200, 75)])
def test_attention_prefill(K, D, Hq, Hkv, T, ctx, impl):
    K.set_attn_prefill_impl(impl)
    g = torch.Generator().manual_seed(ctx + T)
    dev = "cuda"
    rd, theta = D // 4, 1e7
    total = ctx + T
    nblk = (total + 15) // 16 + 1
    cache = torch.zeros(nblk, Hkv, 2, 16, D, dtype=torch.uint8, device=dev)
    table = torch.randperm(nblk, generator=g).to(torch.int32).cuda()
    qn = (torch.randn(D, generator=g) * 0.1).to(BF)
    kn = (torch.randn(D, generator=g) * 0.1).to(BF)
    kds = torch.full((Hkv,), 1 / 8.0)
    vds = torch.full((Hkv,), 1 / 16.0)
    qg_all = torch.randn(total, Hq, 2 * D, generator=g).to(BF)
    k_all = torch.randn(total, Hkv, D, generator=g).to(BF)
    v_all = torch.randn(total, Hkv, D, generator=g).to(BF)
    q_out = torch.zeros(total, Hq, D, dtype=BF, device=dev)
    pos = torch.arange(total, dtype=torch.int32, device=dev)
    K.attn_precore(qg_all.cuda(), k_all.cuda(), v_all.cuda(), qn.cuda(), kn.cuda(), kds.cuda(), vds.cuda(), pos, table,
                   q_out, cache, total, Hq, Hkv, D, rd, theta)
    out = torch.zeros(T, Hq * D, dtype=BF, device=dev)
    K.attn_prefill(q_out[ctx:].contiguous(), qg_all[ctx:].cuda().contiguous(), cache, table, kds.cuda(), vds.cuda(), out,
                   T, Hq, Hkv, D, ctx, True)
    allpos = torch.arange(total)
    qf = R.rope_partial_neox(R.rmsnorm_1pw(qg_all[..., :D], qn), allpos, rd, theta)
    kf = R.rope_partial_neox(R.rmsnorm_1pw(k_all, kn), allpos, rd, theta)
    kq = R.fp8_e4m3_roundtrip(kf, 1 / 8.0)
    vq = R.fp8_e4m3_roundtrip(v_all.float(), 1 / 16.0)
    o = R.causal_gqa_attention(qf[ctx:].to(BF), kq, vq, ctx)
    o = o * torch.sigmoid(qg_all[ctx:, :, D:].float())
    assert torch.allclose(out.float().cpu().view(T, Hq, D), o, atol=2e-2, rtol=3e-2)


@pytest.mark.parametrize("T", [1, 3, 8])
def test_trellis_gemv_fused_prologues_equal_the_unfused_chain(K, T):
    """RMSNorm / SwiGLU folded into the GEMV prologue give the same bits as the separate kernels."""
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(T)
    N, Kd = 256, 1024
    tw = trellis.random_weight(N, Kd, 5, seed=T, sigma=0.02).to("cuda")
    x = torch.randn(T, Kd, generator=g).to(BF).cuda()
    nw = (torch.randn(Kd, generator=g) * 0.1).to(BF).cuda()
    h = K.rmsnorm(x, nw)
    ref = K.trellis_gemv(tw, h, ksplit=4)
    got = K.trellis_gemv(tw, x, ksplit=4, prologue=K.PRO_RMSNORM, norm_w=nw)
    assert torch.equal(ref, got)
    gu = torch.randn(T, 2 * Kd, generator=g).to(BF).cuda()
    ref2 = K.trellis_gemv(tw, K.silu_mul(gu), ksplit=2)
    got2 = K.trellis_gemv(tw, gu, ksplit=2, prologue=K.PRO_SILU_MUL)
    assert torch.equal(ref2, got2)
    W = torch.randn(96, Kd, generator=g).to(BF).cuda()
    out = torch.empty(T, 96, device="cuda")
    K.bf16_gemv_norm(W, x, nw, 1e-6, out)
    assert torch.allclose(out, K.bf16_gemv(W, h), atol=1e-3, rtol=1e-3)


def test_trellis_gemv_long_k_uses_the_stage_ring(K):
    """K large enough that the weight stages wrap around the ring several times."""
    from r4dx_b200.quant import trellis
    tw = trellis.random_weight(128, 4096, 4, seed=9, sigma=0.02)
    x = torch.randn(2, 4096, generator=torch.Generator().manual_seed(1)).to(BF)
    ref = trellis.linear_reference(tw, x.float())
    y = K.trellis_gemv(tw.to("cuda"), x.cuda(), ksplit=1)
    assert (y.float().cpu() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3


def test_moe_router_plan_combine(K):
    g = torch.Generator().manual_seed(3)
    T, E, k, H = 9, 64, 6, 256
    logits = torch.randn(T, E, generator=g)
    logits[2, 5] = logits[2, 40] = 9.0                      # a tie at the top: the lower id comes first
    ids = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, k, device="cuda")
    K.moe_router(logits.cuda(), k, True, ids, w)
    rid, rw = R.moe_route(logits, k, True)
    assert torch.equal(ids.cpu().long(), rid)
    assert torch.allclose(w.cpu(), rw, atol=4e-3)
    off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    perm = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    K.moe_plan(ids, T * k, E, 0, E, off, perm)
    flat = ids.cpu().view(-1)
    exp_perm = torch.sort(flat, stable=True).indices
    assert torch.equal(perm.cpu().long(), exp_perm)
    assert off.cpu().tolist() == [0] + torch.cumsum(torch.bincount(flat.long(), minlength=E), 0).tolist()
    y = torch.randn(T * k, H, generator=g).to(BF)
    sh = torch.randn(T, H, generator=g).to(BF)
    sg = torch.randn(T, 1, generator=g)
    res = torch.randn(T, H, generator=g).to(BF)
    out = torch.zeros(T, H, dtype=BF, device="cuda")
    K.moe_combine(y.cuda(), ids, w, sh.cuda(), sg.cuda(), res.cuda(), out, T, H, k)
    ref = (w.cpu()[:, :, None] * y.float().view(T, k, H)).sum(1) + torch.sigmoid(sg) * sh.float() + res.float()
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("npairs,E,e_begin,e_count", [(40960, 512, 0, 512), (5000, 64, 16, 32), (1025, 8, 0, 8), (20000, 128, 64, 64)])
def test_moe_plan_many_pairs(K, npairs, E, e_begin, e_count):
    """Prefill-sized plans take the 32-warp kernel: same offsets and the same stable order as a stable sort."""
    g = torch.Generator().manual_seed(npairs)
    flat = torch.randint(0, E, (npairs,), generator=g, dtype=torch.int32)
    flat[:40] = e_begin                                        # one expert with a run that spans lanes of one step
    off = torch.zeros(e_count + 1, dtype=torch.int32, device="cuda")
    perm = torch.full((npairs,), -1, dtype=torch.int32, device="cuda")
    K.moe_plan(flat.cuda(), npairs, E, e_begin, e_count, off, perm)
    local = (flat >= e_begin) & (flat < e_begin + e_count)
    idx = torch.nonzero(local).view(-1)
    order = idx[torch.sort(flat[idx], stable=True).indices]
    n = int(local.sum())
    assert torch.equal(perm.cpu()[:n].long(), order)
    assert bool((perm.cpu()[n:] == -1).all())
    counts = torch.bincount((flat[idx] - e_begin).long(), minlength=e_count)
    assert off.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()


@pytest.mark.parametrize("T,E,k,sigmoid,e_begin,e_count", [(1, 512, 10, False, 0, 512), (8, 64, 4, True, 16, 32), (3, 1000, 16, False, 0, 1000),
                                                             (5, 16, 4, False, 0, 16)])
def test_route_and_plan_in_one_launch_equal_the_two_kernels(K, T, E, k, sigmoid, e_begin, e_count):
    g = torch.Generator().manual_seed(T * 1000 + E)
    logits = (torch.randn(T, E, generator=g) * 3).cuda()
    logits[0, 3] = logits[0, 7] = logits[0].max() + 1.0          # a tie at the top: the lower id first
    bias = (torch.randn(E, generator=g) * 0.3).cuda() if sigmoid else None
    mk = lambda *s, dt=torch.int32: torch.full(s, -7, dtype=dt, device="cuda")
    ids_a, w_a, off_a, perm_a = mk(T, k), mk(T, k, dt=torch.float32), mk(e_count + 1), mk(T * k)
    ids_b, w_b, off_b, perm_b = mk(T, k), mk(T, k, dt=torch.float32), mk(e_count + 1), mk(T * k)
    if sigmoid:
        K.moe_router_sigmoid(logits, bias, k, True, 1.5, ids_a, w_a)
    else:
        K.moe_router(logits, k, True, ids_a, w_a)
    K.moe_plan(ids_a, T * k, E, e_begin, e_count, off_a, perm_a)
    K.moe_route_plan(logits, bias, k, True, sigmoid, 1.5 if sigmoid else 1.0, ids_b, w_b, e_begin, e_count, off_b, perm_b)
    assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b) and torch.equal(off_a, off_b)
    n = int(off_a[-1])
    assert torch.equal(perm_a[:n], perm_b[:n])
    if not sigmoid:
        assert ids_a[0, 0].item() == 3 and ids_a[0, 1].item() == 7


def test_grouped_expert_gemv(K):
    from r4dx_b200.models.moe import ExpertStack
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(4)
    E, N, Kd, T, k = 6, 256, 256, 11, 2
    ws = [trellis.random_weight(N, Kd, 3, seed=e, sigma=0.05) for e in range(E)]
    st = ExpertStack.from_list([w.to("cuda") for w in ws])
    x = torch.randn(T, Kd, generator=g).to(BF)
    ids = torch.randint(0, E, (T, k), generator=g).to(torch.int32)
    ids[:, 1] = (ids[:, 0] + 1) % E
    ids[:6, 0] = 2                                            # six rows on one expert -> several passes at tmax 2
    off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    perm = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    K.moe_plan(ids.cuda(), T * k, E, 0, E, off, perm)
    y = torch.zeros(T * k, N, dtype=BF, device="cuda")
    K.trellis_gemv_grouped(st.words, st.suh, st.svh, x.cuda(), y, off, perm, k, (T + 1) // 2, 2, 0, E, N, Kd, 3, 2)
    for t in range(T):
        for j in range(k):
            ref = trellis.linear_reference(ws[int(ids[t, j])], x[t:t + 1].float())[0]
            got = y[t * k + j].float().cpu()
            assert (got - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 1e-3
    # the compact grid (CTAs for the experts the pairs name, here a local slice 1..4 of the six) writes the same rows
    e_begin, e_count = 1, 4
    sub = ExpertStack.from_list([w.to("cuda") for w in ws[e_begin:e_begin + e_count]])
    off2 = torch.zeros(e_count + 1, dtype=torch.int32, device="cuda")
    perm2 = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    K.moe_plan(ids.cuda(), T * k, E, e_begin, e_count, off2, perm2)
    y_full = torch.zeros(T * k, N, dtype=BF, device="cuda")
    y_pairs = torch.zeros(T * k, N, dtype=BF, device="cuda")
    K.trellis_gemv_grouped(sub.words, sub.suh, sub.svh, x.cuda(), y_full, off2, perm2, k, (T + 1) // 2, 2, 0, e_count, N, Kd, 3, 2)
    K.trellis_gemv_grouped_pairs(sub.words, sub.suh, sub.svh, x.cuda(), y_pairs, off2, perm2, ids.cuda(), T * k, e_begin, k,
                                 (T + 1) // 2, 2, 0, e_count, N, Kd, 3, 2)
    assert torch.equal(y_full, y_pairs)
    local = ((ids >= e_begin) & (ids < e_begin + e_count)).view(-1)
    assert torch.equal(y_full[local.cuda()], y[local.cuda()]) and float(y_pairs[~local.cuda()].abs().max()) == 0.0


@pytest.mark.parametrize("kb,tn,T", [(3, 16, 40), (4, 32, 90), (5, 64, 150), (3, 128, 300), (4, 256, 700)])
def test_grouped_expert_gemm_matches_the_per_pair_reference(K, kb, tn, T):
    """Tile list + grouped input transform + grouped tensor-core product (gate_up then SwiGLU + down) for a skewed plan:
    one expert holds a third of the rows (several tiles), some hold none, a slice of the experts is local."""
    from r4dx_b200.models.moe import ExpertStack
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(kb)
    E, I, H, k = 7, 128, 256, 2
    e_begin, e_count = 1, 5                                   # experts 1..5 are local; 0 and 6 live elsewhere
    gu = [trellis.random_weight(2 * I, H, kb, seed=e, sigma=0.06) for e in range(E)]
    dn = [trellis.random_weight(H, I, kb, seed=50 + e, sigma=0.06) for e in range(E)]
    sg = ExpertStack.from_list([w.to("cuda") for w in gu[e_begin:e_begin + e_count]])
    sd = ExpertStack.from_list([w.to("cuda") for w in dn[e_begin:e_begin + e_count]])
    x = torch.randn(T, H, generator=g).to(BF)
    ids = torch.randint(0, E, (T, k), generator=g).to(torch.int32)
    ids[:, 1] = (ids[:, 0] + 1 + torch.randint(0, E - 1, (T,), generator=g).to(torch.int32)) % E
    ids[: T // 3, 0] = 2
    ids[: T // 3, 1] = torch.where(ids[: T // 3, 1] == 2, torch.tensor(3, dtype=torch.int32), ids[: T // 3, 1])
    ids[ids == 4] = 5                                          # expert 4 gets nothing
    ids[:, 1] = torch.where(ids[:, 1] == ids[:, 0], (ids[:, 0] + 1) % E, ids[:, 1])
    P = T * k
    off = torch.zeros(e_count + 1, dtype=torch.int32, device="cuda")
    perm = torch.zeros(P, dtype=torch.int32, device="cuda")
    K.moe_plan(ids.cuda(), P, E, e_begin, e_count, off, perm)
    tiles = torch.zeros(2 * (P // tn + e_count + 1), dtype=torch.int32, device="cuda")
    nt = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.moe_tiles(off, e_count, tn, tiles, nt)
    o = off.cpu().tolist()
    want = [(e, o[e] + j * tn) for e in range(e_count) for j in range((o[e + 1] - o[e] + tn - 1) // tn)]
    assert int(nt.item()) == len(want)
    assert tiles.cpu().view(-1, 2)[:len(want)].tolist() == [list(w) for w in want]
    xh = torch.zeros(P, H, dtype=torch.float16, device="cuda")
    gu_pairs = torch.zeros(P, 2 * I, dtype=BF, device="cuda")
    y_pairs = torch.zeros(P, H, dtype=BF, device="cuda")
    K.trellis_input_grouped(x.cuda(), sg.suh, xh, off, perm, P, k, 0)
    K.trellis_gemm_grouped(sg.words, sg.svh, xh, gu_pairs, off, perm, tiles, nt, P, e_count, 2 * I, H, kb, tn)
    xh2 = xh.view(-1)[:P * I].view(P, I)
    K.trellis_input_grouped(gu_pairs, sd.suh, xh2, off, perm, P, 1, 1)
    K.trellis_gemm_grouped(sd.words, sd.svh, xh2, y_pairs, off, perm, tiles, nt, P, e_count, H, I, kb, tn)
    K.check_gemm_status(y_pairs.device)
    checked = 0
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            got_gu, got_y = gu_pairs[t * k + j].float().cpu(), y_pairs[t * k + j].float().cpu()
            if not (e_begin <= e < e_begin + e_count):
                assert got_gu.abs().max().item() == 0 and got_y.abs().max().item() == 0      # not ours: untouched
                continue
            ref_gu = trellis.linear_reference(gu[e], x[t:t + 1].float())[0]
            assert (got_gu - ref_gu).abs().max().item() < 0.03 * ref_gu.abs().max().item() + 1e-3
            a = got_gu.to(BF).float()
            m = (torch.nn.functional.silu(a[:I]) * a[I:]).to(BF).float()
            ref_y = trellis.linear_reference(dn[e], m[None])[0]
            assert (got_y - ref_y).abs().max().item() < 0.03 * ref_y.abs().max().item() + 1e-3
            checked += 1
    assert checked > T


def test_topk_lse_summary_and_device_rep_penalty(K):
    from r4dx_b200.runtime.sampler import SampleParams, sample_canonical, sample_from_summary
    g = torch.Generator().manual_seed(12)
    logits = (torch.randn(3, 30000, generator=g) * 3)
    logits[1, 17] = logits[1, 29000] = 20.0                      # tie at the top
    vals, ids, lse = K.topk_lse(logits.cuda(), 64, 0.8, 5)
    for t in range(3):
        order = sorted(range(30000), key=lambda i: (-float(logits[t, i]), i))[:64]
        assert ids[t].cpu().tolist() == [i + 5 for i in order]
        assert torch.equal(vals[t].cpu(), logits[t][order])
        assert abs(float(lse[t]) - float(torch.logsumexp(logits[t].double() / 0.8, 0))) < 1e-3
    p = SampleParams(temperature=0.8, top_k=40, top_p=0.9)
    tok = sample_from_summary(vals[0].cpu(), ids[0].cpu() - 5, float(lse[0]), p, 0.37)
    assert tok == sample_canonical(logits[0], p, 0.37)
    row = torch.tensor([2.0, -2.0, 1.0, 0.5], device="cuda")
    K.repetition_penalty(row, torch.tensor([0, 1, 1, 0], dtype=torch.int32, device="cuda"), 2.0)
    assert row.cpu().tolist() == [1.0, -4.0, 1.0, 0.5]


@pytest.mark.parametrize("T,N,Kd,group", [(1, 256, 512, 64), (5, 384, 1024, 128), (8, 96, 256, 32)])
def test_w8a16_gemv(K, T, N, Kd, group):
    from r4dx_b200.quant import w4a16
    g = torch.Generator().manual_seed(N + T)
    W = torch.randn(N, Kd, generator=g) * 0.05
    w = w4a16.quantize_w8(W, group)
    Wd = w4a16.dequantize_w8(w)
    x = torch.randn(T, Kd, generator=g).to(BF)
    ref = x.float() @ Wd.T
    wd = w4a16.W8Weight(w.wq.cuda(), w.ws.cuda(), w.N, w.K, w.group)
    got = K.w8a16_gemv(wd, x.cuda(), out_f32=True).cpu()
    assert torch.allclose(got, ref, atol=2e-2 * ref.abs().max().item(), rtol=1e-2)
    got_bf = K.w8a16_gemv(wd, x.cuda()).float().cpu()
    assert torch.allclose(got_bf, ref, atol=3e-2 * ref.abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_rotate_rows_in_place(K, mode):
    g = torch.Generator().manual_seed(mode)
    x = torch.randn(7, 512, generator=g).to(BF)
    s = (torch.randint(0, 2, (512,), generator=g).float() * 2 - 1).to(torch.float16)
    xf = x.float()
    if mode == 0:
        ref = R.fwht(xf)
    elif mode == 1:
        ref = R.fwht(xf * s.float())
    else:
        ref = R.fwht(xf) * s.float()
    y = x.cuda().clone()
    K.rotate_rows(y, s.cuda() if mode else None, mode)
    assert torch.allclose(y.float().cpu(), ref, atol=3e-2, rtol=2e-2)
    if mode == 0:      # the normalised transform is its own inverse
        K.rotate_rows(y, None, 0)
        assert torch.allclose(y.float().cpu(), xf, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("kb", [3, 4, 5])
def test_gpu_viterbi_encoder_matches_the_host_encoder_in_quality(K, kb):
    """Same search on both sides; the regularisation signs differ, so compare quality, not bits."""
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(kb)
    W = torch.randn(128, 256, generator=g) * 0.03
    wc, err_cpu = trellis.quantize(W, kb, seed=1)
    wg, err_gpu = trellis.quantize_cuda(W, kb, seed=1)
    assert abs(err_gpu - err_cpu) < 0.1 * err_cpu, (err_gpu, err_cpu)
    assert err_gpu < {3: 0.04, 4: 0.012, 5: 0.004}[kb]
    rec = trellis.reconstruct(TrellisWeightCpu(wg))
    rel = ((rec - W).pow(2).sum() / W.pow(2).sum()).item()
    assert abs(rel - err_gpu) < 0.25 * err_gpu + 1e-4, (rel, err_gpu)      # the reported error is the real reconstruction error
    # and the device kernels read the GPU-made words like any other weight
    x = torch.randn(2, 256, generator=g).to(BF)
    y = K.trellis_gemv(wg, x.cuda()).float().cpu()
    ref = x.float() @ rec.T
    assert torch.allclose(y, ref, atol=3e-2 * ref.abs().max().item(), rtol=3e-2)


def TrellisWeightCpu(w):
    from r4dx_b200.quant.trellis import TrellisWeight
    return TrellisWeight(w.words.cpu(), w.suh.cpu(), w.svh.cpu(), w.N, w.K, w.kb)


def test_sigmoid_router_matches_reference(K):
    g = torch.Generator().manual_seed(13)
    T, E, k = 7, 32, 4
    logits = torch.randn(T, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.3
    ids = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, k, device="cuda")
    for b, scale in ((None, 1.0), (bias, 2.5)):
        K.moe_router_sigmoid(logits.cuda(), b.cuda() if b is not None else None, k, True, scale, ids, w)
        rid, rw = R.moe_route_sigmoid(logits, b, k, True, scale)
        assert torch.equal(ids.cpu().long(), rid)
        assert torch.allclose(w.cpu(), rw, rtol=1e-2, atol=4e-3)


def test_short_conv_across_calls_matches_reference(K):
    """Decode-sized calls, a partly rejected speculative window and a prefill-sized call, one state ring: every output
    equals the reference convolution over the committed sequence."""
    g = torch.Generator().manual_seed(21)
    H, L = 384, 3
    wt = (torch.randn(H, L, generator=g) * 0.5).to(BF)
    ring = torch.zeros(32, H, dtype=BF, device="cuda")
    state = None
    pos = 0

    def call(T, commit):
        nonlocal state, pos
        bcx = torch.randn(T, 3 * H, generator=g).to(BF)
        out = torch.zeros(T, H, dtype=BF, device="cuda")
        K.short_conv(bcx.cuda(), wt.cuda(), ring, torch.tensor([pos], dtype=torch.int32, device="cuda"), out, T)
        ref, _ = R.short_conv(bcx.float(), wt.float(), state, round_bf16=True)
        assert torch.allclose(out.float().cpu(), ref, rtol=2e-2, atol=2e-2), (T, pos)
        _, state = R.short_conv(bcx[:commit].float(), wt.float(), state, round_bf16=True)   # only the committed rows advance the state
        pos += commit

    call(1, 1)
    call(5, 5)
    call(8, 3)          # a verify window of 8 rows of which 3 are accepted: the next call overwrites the other slots
    call(1, 1)
    call(16, 2)         # the widest window
    call(3, 3)
    call(45, 45)        # prefill-sized: the ring update is the second launch
    call(2, 2)
    call(64, 64)        # a multiple of the ring length
    call(1, 1)


def test_viterbi_quantized_layer_times_like_a_random_code_layer(K):
    """The benchmarks use random code words in the trellis layout.  A layer quantized from N(0, 0.02) weights by the
    Viterbi encoder has the same shapes and bytes, and the kernels' work does not depend on the code values: the
    weight-streaming kernel's time for the two differs by less than 2 % (median of repeated cold launches)."""
    from r4dx_b200.quant import trellis
    N, Kd, kb = 2048, 2048, 4
    g = torch.Generator().manual_seed(0)
    W = torch.randn(N, Kd, generator=g) * 0.02
    tq, _ = trellis.quantize_cuda(W, kb, seed=3)
    tr = trellis.random_weight(N, Kd, kb, seed=4, device="cuda")
    assert tq.words.numel() == tr.words.numel() and tq.kb == tr.kb
    x = torch.randn(1, Kd, generator=g).to(BF).cuda()
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")

    def med(w):
        y = torch.empty(1, N, dtype=BF, device="cuda")
        ts = []
        for i in range(60):
            flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            K.trellis_gemv(w, x, out=y)
            e1.record()
            torch.cuda.synchronize()
            if i >= 10:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    tqd = trellis.TrellisWeight(tq.words.cuda(), tq.suh.cuda(), tq.svh.cuda(), tq.N, tq.K, tq.kb)
    a, b = med(tqd), med(tr)
    a2, b2 = med(tqd), med(tr)                      # interleaved repeats guard against drift between the two series
    ta, tb = min(a, a2), min(b, b2)
    assert abs(ta - tb) <= 0.02 * max(ta, tb) + 0.0003, (ta, tb)     # 2 % plus the event timer's 0.3 us granularity


@pytest.mark.parametrize("T,N,Kd,group", [(20, 256, 512, 64), (300, 384, 1024, 128)])
def test_linear_tc_w8a16_matches_fp32_reference(K, T, N, Kd, group):
    from r4dx_b200.quant import w4a16
    g = torch.Generator().manual_seed(T)
    W = torch.randn(N, Kd, generator=g) * 0.05
    w = w4a16.quantize_w8(W, group)
    Wd = w4a16.dequantize_w8(w)
    x = torch.randn(T, Kd, generator=g).to(BF)
    res = torch.randn(T, N, generator=g).to(BF)
    ref = x.half().float() @ Wd.T
    y = K.linear_tc(w.to("cuda"), x.cuda(), out_f32=True)
    K.check_gemm_status(y.device)
    assert torch.allclose(y.cpu(), ref, atol=2e-2, rtol=1e-2)
    y2 = K.linear_tc(w.to("cuda"), x.cuda(), residual=res.cuda())
    assert torch.allclose(y2.float().cpu(), ref + res.float(), atol=6e-2, rtol=2e-2)
