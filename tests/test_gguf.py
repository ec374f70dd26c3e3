"""GGUF reader: container parsing, block dequantisation against scalar restatements of the formats, and the import of a
Llama-style checkpoint (with the rotary row permutation of that architecture) through the converter."""
import numpy as np
import torch

from r4dx_b200.quant import gguf as G


def _f16(x):
    return np.float16(x).astype(np.float32)


def test_block_formats_match_scalar_decoders():
    rng = np.random.default_rng(0)
    # Q4_0 / Q4_1 / Q5_0 / Q8_0: three blocks each
    for gtype in (G.GGML_Q4_0, G.GGML_Q4_1, G.GGML_Q5_0, G.GGML_Q8_0):
        per, size = G.BLOCK[gtype]
        raw = rng.integers(0, 256, size=(3, size), dtype=np.uint8)
        raw[:, :2] = np.array([0.0123], np.float16).view(np.uint8)            # a finite scale
        if gtype == G.GGML_Q4_1:
            raw[:, 2:4] = np.array([-0.5], np.float16).view(np.uint8)
        got = G.dequantize(raw.reshape(-1), gtype).reshape(3, per)
        for b in range(3):
            d = _f16(raw[b, :2].view(np.float16)[0])
            exp = np.zeros(32, np.float32)
            if gtype == G.GGML_Q8_0:
                exp = raw[b, 2:].view(np.int8).astype(np.float32) * d
            elif gtype == G.GGML_Q5_0:
                qh = int(raw[b, 2:6].view(np.uint32)[0])
                for j in range(16):
                    q = int(raw[b, 6 + j])
                    exp[j] = (((q & 0xF) | (((qh >> j) & 1) << 4)) - 16) * d
                    exp[j + 16] = (((q >> 4) | (((qh >> (j + 16)) & 1) << 4)) - 16) * d
            else:
                hdr = 2 if gtype == G.GGML_Q4_0 else 4
                m = _f16(raw[b, 2:4].view(np.float16)[0]) if gtype == G.GGML_Q4_1 else 0.0
                for j in range(16):
                    q = int(raw[b, hdr + j])
                    lo, hi = q & 0xF, q >> 4
                    exp[j], exp[j + 16] = ((lo - 8) * d, (hi - 8) * d) if gtype == G.GGML_Q4_0 else (lo * d + m, hi * d + m)
            assert np.allclose(got[b], exp, rtol=1e-6, atol=1e-7), gtype


def test_k_quants_match_scalar_decoders():
    rng = np.random.default_rng(1)
    # Q4_K
    raw = rng.integers(0, 256, size=(2, 144), dtype=np.uint8)
    raw[:, 0:2] = np.array([0.01], np.float16).view(np.uint8)
    raw[:, 2:4] = np.array([0.02], np.float16).view(np.uint8)
    got = G.dequantize(raw.reshape(-1), G.GGML_Q4_K).reshape(2, 256)
    for b in range(2):
        d, dmin = _f16(raw[b, 0:2].view(np.float16)[0]), _f16(raw[b, 2:4].view(np.float16)[0])
        s = raw[b, 4:16].astype(int)

        def sm(j):
            if j < 4:
                return s[j] & 63, s[j + 4] & 63
            return (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)

        exp, q, at = np.zeros(256, np.float32), raw[b, 16:], 0
        for c in range(4):
            (s1, m1), (s2, m2) = sm(2 * c), sm(2 * c + 1)
            for l in range(32):
                exp[at + l] = d * s1 * (int(q[32 * c + l]) & 0xF) - dmin * m1
                exp[at + 32 + l] = d * s2 * (int(q[32 * c + l]) >> 4) - dmin * m2
            at += 64
        assert np.allclose(got[b], exp, rtol=1e-5, atol=1e-6)
    # Q6_K
    raw = rng.integers(0, 256, size=(2, 210), dtype=np.uint8)
    raw[:, 208:210] = np.array([0.003], np.float16).view(np.uint8)
    got = G.dequantize(raw.reshape(-1), G.GGML_Q6_K).reshape(2, 256)
    for b in range(2):
        d = _f16(raw[b, 208:210].view(np.float16)[0])
        ql, qh, sc = raw[b, :128].astype(int), raw[b, 128:192].astype(int), raw[b, 192:208].view(np.int8).astype(int)
        exp = np.zeros(256, np.float32)
        for n in range(2):
            for l in range(32):
                i = l // 16
                a, h = ql[64 * n:], qh[32 * n:]
                q1 = ((a[l] & 0xF) | ((h[l] & 3) << 4)) - 32
                q2 = ((a[l + 32] & 0xF) | (((h[l] >> 2) & 3) << 4)) - 32
                q3 = ((a[l] >> 4) | (((h[l] >> 4) & 3) << 4)) - 32
                q4 = ((a[l + 32] >> 4) | (((h[l] >> 6) & 3) << 4)) - 32
                for gi, qv in enumerate((q1, q2, q3, q4)):
                    exp[128 * n + 32 * gi + l] = d * sc[8 * n + i + 2 * gi] * qv
        assert np.allclose(got[b], exp, rtol=1e-5, atol=1e-6)


def test_llama_gguf_imports_to_the_same_model(tmp_path):
    """Internal weights -> HF layout -> a GGUF file as a llama-architecture exporter would write it (rotary rows interleaved,
    F32 / F16 / Q8_0 tensors, metadata) -> import: the oracle's logits match up to the file's quantisation."""
    from r4dx_b200.config import tiny_llama_config
    from r4dx_b200.models.oracle import OracleModel, init_weights
    from r4dx_b200.quant import hf_import as HI
    cfg = tiny_llama_config()
    w = init_weights(cfg, 1)
    hf = HI.export_hf_weights(cfg, w)

    def permute(t, heads):            # [head][2][d/2] -> [head][d/2][2]
        return t.reshape(heads, 2, t.shape[0] // heads // 2, t.shape[1]).transpose(1, 2).reshape(t.shape)

    rev = {v: k for k, v in G._LAYER_NAMES.items()}
    tensors = {"token_embd.weight": (hf["model.embed_tokens.weight"].numpy(), G.GGML_F16),
               "output_norm.weight": (hf["model.norm.weight"].numpy(), G.GGML_F32),
               "output.weight": (hf["lm_head.weight"].numpy(), G.GGML_Q8_0)}
    for i in range(cfg.num_hidden_layers):
        for mine, theirs in rev.items():
            key = f"model.layers.{i}.{mine}.weight"
            if key not in hf:
                continue
            t = hf[key]
            if theirs == "attn_q":
                t = permute(t, cfg.num_attention_heads)
            if theirs == "attn_k":
                t = permute(t, cfg.num_key_value_heads)
            tensors[f"blk.{i}.{theirs}.weight"] = (t.contiguous().numpy(), G.GGML_F32 if t.dim() == 1 else G.GGML_Q8_0)
    md = {"general.architecture": "llama", "llama.block_count": cfg.num_hidden_layers, "llama.embedding_length": cfg.hidden_size,
          "llama.feed_forward_length": cfg.intermediate_size, "llama.attention.head_count": cfg.num_attention_heads,
          "llama.attention.head_count_kv": cfg.num_key_value_heads, "llama.rope.freq_base": float(cfg.rope_theta),
          "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), "llama.context_length": 4096,
          "tokenizer.ggml.tokens": ["a", "b"]}
    path = str(tmp_path / "m.gguf")
    G.write_gguf(path, md, tensors)
    g = G.GgufFile(path)
    assert g.metadata["llama.block_count"] == cfg.num_hidden_layers and g.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    assert g.tensors["blk.0.attn_q.weight"].shape == (cfg.q_dim, cfg.hidden_size)
    g.close()
    cfg2, back = G.import_gguf(path)
    assert cfg2.head_dim == cfg.head_dim and cfg2.rotary_dim == cfg.head_dim and not cfg2.qk_norm and not cfg2.tie_word_embeddings
    assert torch.allclose(back["text.layers.1.attn.qg"], w["text.layers.1.attn.qg"], atol=float(w["text.layers.1.attn.qg"].abs().max()) / 127)       # half a Q8_0 step, with slack
    ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(0))
    la, _ = OracleModel(cfg, w).forward(ids)
    lb, _ = OracleModel(cfg2, back).forward(ids)
    assert (la - lb).abs().max() < 0.03 * la.abs().max()
    # the converter takes the file directly
    from r4dx_b200.cli.convert import main as convert_main
    assert convert_main(["--input", path, "--output", str(tmp_path / "m.r4dxb"), "--layers", "1"]) == 0


def test_moe_gguf_with_stacked_experts_imports_to_the_same_model(tmp_path):
    """An all-attention MoE decoder written the way such files are (experts stacked per projection, shared expert with its
    gate) -> import: the same weights, the same logits."""
    import dataclasses
    from r4dx_b200.config import tiny_moe_config
    from r4dx_b200.models.oracle import OracleModel, init_weights
    cfg = dataclasses.replace(tiny_moe_config(), layer_types=["full_attention"] * 2, num_hidden_layers=2, attn_output_gate=False,
                              norm_zero_centered=False, partial_rotary_factor=1.0, rope_theta=1.0e6, norm_topk_prob=False)
    from r4dx_b200.quant import hf_import as HI
    w = init_weights(cfg, 3)
    hf = HI.export_hf_weights(cfg, w)                            # the checkpoint's conventions (plain norm scales, split gate / up)
    E, I = cfg.num_experts, cfg.moe_intermediate_size
    f32 = lambda t: (t.contiguous().numpy(), G.GGML_F32)
    tensors = {"token_embd.weight": f32(hf["model.embed_tokens.weight"]), "output_norm.weight": f32(hf["model.norm.weight"]),
               "output.weight": f32(hf["lm_head.weight"])}
    rev = {v: k for k, v in G._LAYER_NAMES.items()}
    for i in range(2):
        L = f"model.layers.{i}."
        for mine, theirs in rev.items():
            if L + mine + ".weight" in hf:
                tensors[f"blk.{i}.{theirs}.weight"] = f32(hf[L + mine + ".weight"])
        m = L + "mlp."
        tensors[f"blk.{i}.ffn_gate_inp.weight"] = f32(hf[m + "gate.weight"])
        tensors[f"blk.{i}.ffn_gate_inp_shexp.weight"] = f32(hf[m + "shared_expert_gate.weight"].reshape(-1))
        for n in ("gate", "up", "down"):
            tensors[f"blk.{i}.ffn_{n}_exps.weight"] = f32(torch.stack([hf[m + f"experts.{e}.{n}_proj.weight"] for e in range(E)]))
            tensors[f"blk.{i}.ffn_{n}_shexp.weight"] = f32(hf[m + f"shared_expert.{n}_proj.weight"])
    a = "qwen2moe"
    md = {"general.architecture": a, f"{a}.block_count": 2, f"{a}.embedding_length": cfg.hidden_size, f"{a}.feed_forward_length": 0,
          f"{a}.attention.head_count": cfg.num_attention_heads, f"{a}.attention.head_count_kv": cfg.num_key_value_heads,
          f"{a}.attention.key_length": cfg.head_dim, f"{a}.rope.freq_base": float(cfg.rope_theta),
          f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), f"{a}.expert_count": E,
          f"{a}.expert_used_count": cfg.num_experts_per_tok, f"{a}.expert_feed_forward_length": I,
          f"{a}.expert_shared_feed_forward_length": cfg.shared_expert_intermediate_size}
    path = str(tmp_path / "moe.gguf")
    G.write_gguf(path, md, tensors)
    cfg2, back = G.import_gguf(path)
    assert cfg2.is_moe and cfg2.num_experts == E and cfg2.shared_expert_intermediate_size == cfg.shared_expert_intermediate_size
    assert cfg2.layer_types == ["full_attention"] * 2 and not cfg2.norm_topk_prob and not cfg2.attn_output_gate
    assert set(back) == set(w)
    for k_ in w:
        assert torch.allclose(back[k_], w[k_], atol=1e-6), k_
    ids = torch.randint(0, cfg.vocab_size, (7,), generator=torch.Generator().manual_seed(0))
    la, _ = OracleModel(cfg, w).forward(ids)
    lb, _ = OracleModel(cfg2, back).forward(ids)
    assert torch.allclose(la, lb, atol=1e-4)
