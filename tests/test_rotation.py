"""Residual-stream rotation: the fold is exact in fp32, the container round-trips it, the kernel matches the math."""
import json
import os

import pytest
import torch

from r4dx_b200.config import tiny_hybrid_config
from r4dx_b200.models.oracle import OracleModel, init_weights
from r4dx_b200.quant import rotation as rot


def _spec(cfg, block=64, seed=11):
    return rot.make_spec("q2a", seed, cfg.hidden_size, block)


def test_q_is_orthogonal_and_qt_inverts_it():
    spec = rot.make_spec("q2a", 3, 5120)
    assert (spec.block, spec.nblk) == (1024, 5)
    t = rot.rotation_tensors(spec)
    rot.check_rotation_tensors(spec, t["rotation.signs"], t["rotation.mix"])
    x = torch.randn(7, 5120, dtype=torch.float64)
    y = rot.apply_q(x, spec, t["rotation.signs"].double(), t["rotation.mix"].double())
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    back = rot.apply_qt(y, spec, t["rotation.signs"].double(), t["rotation.mix"].double())
    assert torch.allclose(back, x, atol=1e-5)
    # the same seed gives the same tensors; another seed does not
    t2 = rot.rotation_tensors(rot.make_spec("q2a", 3, 5120))
    assert torch.equal(t["rotation.mix"], t2["rotation.mix"]) and torch.equal(t["rotation.signs"], t2["rotation.signs"])
    assert not torch.equal(t["rotation.signs"], rot.rotation_tensors(rot.make_spec("q2a", 4, 5120))["rotation.signs"])


def test_rotation_spreads_an_outlier_channel():
    spec = rot.make_spec("q2a", 1, 2048)
    t = rot.rotation_tensors(spec)
    x = torch.zeros(1, 2048)
    x[0, 37] = 100.0
    y = rot.apply_q(x, spec, t["rotation.signs"], t["rotation.mix"])
    assert y.abs().max().item() < 100.0 / 20          # 100 / sqrt(1024) = 3.1 per channel, times a mix entry below 1


def test_folded_model_equals_the_unrotated_model_in_fp32():
    """The gate for the fold table: logits of the rotated weight set (entry Q, exit Q^T, norms folded away) equal the
    unrotated model's, for a prompt and for decode steps with state carried over."""
    cfg = tiny_hybrid_config()
    w = init_weights(cfg, 0)
    for k in w:
        if k.endswith("layernorm"):
            w[k] = w[k] + 0.3 * torch.randn(w[k].shape, generator=torch.Generator().manual_seed(len(k)))   # norms that matter
    spec = _spec(cfg)
    assert spec.nblk > 1
    wr = rot.fold_rotation(cfg, w, spec)
    assert all(float(wr[k].abs().max()) == 0.0 for k in wr if k.endswith("input_layernorm") or k.endswith("post_attention_layernorm"))
    a, b = OracleModel(cfg, w), OracleModel(cfg, wr)
    ids = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(2))
    la, sa = a.forward(ids)
    lb, sb = b.forward(ids)
    assert (la - lb).abs().max().item() < 2e-4 * la.abs().max().item()
    for t in (5, 9):
        la, sa = a.forward(torch.tensor([t]), sa)
        lb, sb = b.forward(torch.tensor([t]), sb)
        assert (la - lb).abs().max().item() < 2e-4 * la.abs().max().item()
    # captured features come back in the un-rotated basis
    _, _, _, ca = a.forward(ids, return_hidden=True, capture_layers=[1])
    _, _, _, cb = b.forward(ids, return_hidden=True, capture_layers=[1])
    assert (ca[1] - cb[1]).abs().max().item() < 2e-4 * ca[1].abs().max().item()


def test_unsupported_families_are_refused():
    from r4dx_b200.config import tiny_moe_config
    cfg = tiny_moe_config()
    with pytest.raises(ValueError):
        rot.fold_rotation(cfg, init_weights(cfg, 0), rot.make_spec("q2a", 0, cfg.hidden_size))
    with pytest.raises(ValueError):
        rot.RotationSpec.from_meta({"kind": "hadamard1024x5", "seed": 1, "hidden": 256, "block": 64}, 256)
    with pytest.raises(ValueError):
        rot.RotationSpec.from_meta({"kind": "q2a", "seed": -1, "hidden": 256, "block": 64}, 256)


def test_converter_writes_a_rotated_container(tmp_path):
    from r4dx_b200.cli.convert import main as convert
    from r4dx_b200.quant.container import Container
    from r4dx_b200.quant.weights import dequantize_weight_set, load_weight_set
    out = str(tmp_path / "rot.r4dxb")
    assert convert(["--input", "random:tiny", "--output", out, "--layouts", "bf16", "--lm-head", "bf16", "--rotate", "q2a",
                    "--rotation-seed", "0x2A", "--rotation-block", "64"]) == 0
    meta = json.loads(Container(out).metadata["rotation"])
    assert meta == {"kind": "q2a", "seed": 42, "hidden": 256, "block": 64}
    cfg, q = load_weight_set(out)
    assert q["rotation.mix"].dtype == torch.float32 and q["rotation.mix"].shape == (4, 4)
    # the rotated bf16 container serves the same function as the plain one (bf16 rounding of the folded weights apart)
    plain = str(tmp_path / "plain.r4dxb")
    assert convert(["--input", "random:tiny", "--output", plain, "--layouts", "bf16", "--lm-head", "bf16"]) == 0
    _, qp = load_weight_set(plain)
    a, b = OracleModel(cfg, dequantize_weight_set(qp)), OracleModel(cfg, dequantize_weight_set(q))
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(3))
    la, _ = a.forward(ids)
    lb, _ = b.forward(ids)
    assert (la - lb).abs().max().item() < 0.03 * la.abs().max().item()
    # tensors only
    only = str(tmp_path / "rot.safetensors")
    assert convert(["--input", "random:tiny", "--output", str(tmp_path / "unused"), "--rotate", "q2a", "--rotation-out", only]) == 0
    from safetensors.torch import load_file
    assert set(load_file(only)) == {"rotation.signs", "rotation.mix"} and not os.path.exists(str(tmp_path / "unused"))


@pytest.mark.gpu
@pytest.mark.parametrize("H,B", [(5120, 1024), (256, 64), (2048, 1024), (1536, 512)])
def test_rotate_residual_kernel_matches_the_reference(H, B):
    from r4dx_b200.ops import kernels as K
    spec = rot.make_spec("q2a", 7, H, B)
    t = rot.rotation_tensors(spec)
    x = torch.randn(5, H, generator=torch.Generator().manual_seed(H)).to(torch.bfloat16)
    signs, mix = t["rotation.signs"].cuda(), t["rotation.mix"].cuda()
    y = K.rotate_residual(x.cuda().clone(), signs, mix).float().cpu()
    ref = rot.apply_q(x.float(), spec, t["rotation.signs"], t["rotation.mix"])
    assert torch.allclose(y, ref, atol=2e-2, rtol=2e-2)
    back = K.rotate_residual(y.to(torch.bfloat16).cuda(), signs, mix, inverse=True).float().cpu()
    ref_back = rot.apply_qt(y.to(torch.bfloat16).float(), spec, t["rotation.signs"], t["rotation.mix"])
    assert torch.allclose(back, ref_back, atol=2e-2, rtol=2e-2)
    assert torch.allclose(back, x.float(), atol=6e-2, rtol=3e-2)


@pytest.mark.gpu
def test_rotated_quantized_model_matches_its_oracle_on_the_gpu():
    """Trellis-quantized rotated tiny model: prefill, chunked prefill and decode against the CPU oracle of the same set."""
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.quant.weights import dequantize_weight_set, quantize_weight_set
    cfg = tiny_hybrid_config()
    w = rot.fold_rotation(cfg, init_weights(cfg, 0), _spec(cfg))
    q = quantize_weight_set(cfg, w)
    oracle = OracleModel(cfg, dequantize_weight_set(q), fp8_kv=True)
    qd = {k: (v.to("cuda") if hasattr(v, "to") else v) for k, v in q.items()}
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(9)).to(torch.int32)
    ref, _ = oracle.forward(ids.long())
    m = HybridModel(cfg, qd, max_ctx=128)
    assert m.rot is not None
    m.prefill_small(ids)
    la = m.buf.logits[(40 - 1) % 8].float().cpu()
    scale = ref[-1].abs().max().item()
    assert (la - ref[-1]).abs().max().item() < 0.06 * scale
    m2 = HybridModel(cfg, qd, max_ctx=128)
    m2.prefill(ids, chunk=24)
    lb = m2.buf.logits[0].float().cpu()
    assert (lb - ref[-1]).abs().max().item() < 0.06 * scale
    assert int(la.argmax()) == int(lb.argmax())
