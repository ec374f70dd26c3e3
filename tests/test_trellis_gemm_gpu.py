"""tcgen05 trellis GEMM vs fp32 references (needs a B200)."""
import pytest
import torch

from r4dx_b200.ops import reference as R

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def K():
    from r4dx_b200.ops import kernels
    return kernels


def test_input_transform(K):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 512, generator=g).to(BF)
    suh = (torch.randn(512, generator=g)).to(torch.float16)
    out = K.trellis_input(x.cuda(), suh.cuda())
    ref = R.fwht(x.float() * suh.float()[None])
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2, rtol=1e-2)
    gu = torch.randn(3, 1024, generator=g).to(BF)
    out2 = K.trellis_input(gu.cuda(), suh.cuda(), fused_silu_mul=True)
    act = R.silu_mul(gu.float()).to(BF).float()
    assert torch.allclose(out2.float().cpu(), R.fwht(act * suh.float()[None]), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("T,tn", [(16, 16), (40, 64), (128, 128), (300, 128), (512, 256), (700, 512), (1024, 512)])
def test_dense_tensor_core_path(K, T, tn):
    """Dense fp16 A operand: isolates TMA / UMMA descriptors / TMEM epilogue from the trellis decode."""
    g = torch.Generator().manual_seed(T)
    N, Kd = 256, 384
    W = (torch.randn(N, Kd, generator=g) * 0.5).to(torch.float16)
    xh = torch.randn(T, Kd, generator=g).to(torch.float16)
    svh = (torch.randn(N, generator=g)).to(torch.float16)
    y = K.dense_gemm_hadamard(W.cuda(), svh.cuda(), xh.cuda(), tn=tn)
    K.check_gemm_status("cuda")
    ref = R.fwht(xh.float() @ W.float().T) * svh.float()[None]
    err = (y.float().cpu() - ref).abs().max().item()
    assert err < 0.02 * ref.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("kb", [3, 4, 5])
@pytest.mark.parametrize("T,tn", [(16, 16), (100, 128), (512, 256), (600, 512)])
def test_trellis_gemm_matches_reference_and_gemv(K, kb, T, tn):
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(kb * 100 + T)
    N, Kd = 384, 512
    tw = trellis.random_weight(N, Kd, kb, seed=kb, sigma=0.02)
    x = torch.randn(T, Kd, generator=g).to(BF)
    res = torch.randn(T, N, generator=g).to(BF)
    twd = tw.to("cuda")
    xh = K.trellis_input(x.cuda(), twd.suh)
    y = K.trellis_gemm(twd, xh, tn=tn)
    K.check_gemm_status("cuda")
    ref = trellis.linear_reference(tw, x.float())
    scale = ref.abs().max().item()
    assert (y.float().cpu() - ref).abs().max().item() < 0.02 * scale + 1e-3
    y2 = K.trellis_gemm(twd, xh, residual=res.cuda(), tn=tn)
    assert (y2.float().cpu() - (ref + res.float())).abs().max().item() < 0.02 * (scale + 4) + 1e-3
    # the small-batch kernel must agree with the tensor-core kernel on the same rows
    y8 = K.trellis_gemv(twd, x[:8].cuda())
    assert (y8.float() - y[:8].float()).abs().max().item() < 0.02 * scale + 1e-3


@pytest.mark.parametrize("kb,T,N,Kd,tn", [(4, 300, 256, 512, 128), (5, 1024, 384, 1024, 512), (3, 700, 128, 256, 256)])
def test_trellis_gemm_8bit_operands_match_the_reference_within_their_rounding(kb, T, N, Kd, tn):
    """e4m3 activations (one scale per row) times e4m3 code values against the fp32 reference of the same weights.
    Three mantissa bits on both operands: the error is a few percent of the output scale, far below a wrong layout (~1),
    and close to the 16-bit kernel's result."""
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(kb + T)
    w = trellis.random_weight(N, Kd, kb, seed=5, sigma=0.05)
    x = torch.randn(T, Kd, generator=g).to(torch.bfloat16)
    ref = trellis.linear_reference(w, x.float())
    wd = w.to("cuda")
    xh = K.trellis_input(x.cuda(), wd.suh)
    xq, sc = K.quantize_rows_e4m3(xh)
    back = (xq.view(torch.float8_e4m3fn).float() * sc[:, None]).cpu()
    assert (back - xh.float().cpu()).abs().max().item() <= 0.07 * xh.float().abs().max().item()     # half an e4m3 step of the row maximum
    y8 = K.trellis_gemm_f8(wd, xq, sc, tn=tn).float().cpu()
    K.check_gemm_status("cuda")
    y16 = K.trellis_gemm(wd, xh).float().cpu()
    scale = ref.abs().max().item()
    rms = lambda a: a.pow(2).mean().sqrt().item()
    assert rms(y8 - ref) < 0.05 * rms(ref), (rms(y8 - ref), rms(ref))
    assert (y8 - ref).abs().max().item() < 0.15 * scale
    assert rms(y16 - ref) < rms(y8 - ref)                                    # the 16-bit path is the more exact one
    res = torch.randn(T, N, generator=g).to(torch.bfloat16)
    y8r = K.trellis_gemm_f8(wd, xq, sc, residual=res.cuda(), tn=tn).float().cpu()
    assert (y8r - (y8 + res.float())).abs().max().item() < 0.02 * scale + 0.05
