"""Argument parsers and the converter round trip (CPU)."""
import os

import pytest
import torch

from r4dx_b200.cli.args import cli_parser, convert_parser, server_parser


def test_parsers_accept_the_documented_flags():
    a = cli_parser().parse_args(["--model", "m.r4dxb", "--prompt", "hi", "--max-tokens", "5", "--tp", "2", "--mtp", "3",
                                 "--temperature", "0.7", "--top-k", "40", "--stats", "--think", "off", "--pp", "2", "--hybrid"])
    assert a.tp == 2 and a.mtp == 3 and a.top_k == 40 and a.think == "off" and a.hybrid
    s = server_parser().parse_args(["--model", "m", "--port", "9000", "--max-queue", "3", "--request-log", "x.jsonl",
                                    "--default-temperature", "0.5", "--batch", "4", "--prompt-checkpoint", "off"])
    assert s.port == 9000 and s.max_queue == 3 and s.default_temperature == 0.5 and s.batch == 4
    c = convert_parser().parse_args(["--input", "random:tiny", "--output", "o", "--kb-plan", "kb4", "--selftest"])
    assert c.kb_plan == "kb4" and c.selftest


def test_convert_roundtrip_and_reuse(tmp_path):
    from r4dx_b200.cli import convert
    from r4dx_b200.quant.weights import load_weight_set
    out = str(tmp_path / "tiny.r4dxb")
    assert convert.main(["--input", "random:tiny", "--output", out, "--layers", "1", "--kb-plan", "kb4", "--selftest"]) == 0
    cfg, q = load_weight_set(out)
    assert cfg.num_hidden_layers == 1 and "lm_head" in q
    out2 = str(tmp_path / "tiny2.r4dxb")
    assert convert.main(["--input", "random:tiny", "--output", out2, "--layers", "1", "--kb-plan", "kb4",
                         "--reuse-tensors-from", out]) == 0
    _, q2 = load_weight_set(out2)
    assert torch.equal(q2["text.layers.0.mlp.down"].words, q["text.layers.0.mlp.down"].words)


def test_native_resource_gate_passes_on_the_built_library():
    """Every kernel's ptxas figures are kept beside its object; none may spill beyond the gate's limit."""
    from r4dx_b200.native import build as B
    B.build()
    rep = B.check_resources()
    names = " ".join(k for _, k, _, _, _ in rep)
    assert len(rep) > 100 and "TrellisGemmKernel" in names and "GdnChunkScanKernel" in names
    assert max(r for _, _, r, _, _ in rep) <= 255


def test_converter_builds_a_tiny_model_of_every_family(tmp_path):
    """random:<family> -> container -> reload: config and tensor set survive, for each model family the engine serves."""
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.weights import load_weight_set
    for kind, layers, probe in (("llama", 1, "text.layers.0.attn.qg"), ("gemma", 1, "text.layers.0.post_mlp_out_norm"),
                                ("lfm2", 2, "text.layers.0.conv.in_proj")):
        out = str(tmp_path / f"{kind}.r4dxb")
        assert convert_main(["--input", f"random:{kind}", "--output", out, "--layers", str(layers), "--kb-plan", "kb3"]) == 0
        cfg, w = load_weight_set(out)
        assert cfg.num_hidden_layers == layers and probe in w, (kind, sorted(w)[:8])
    cfg, w = load_weight_set(str(tmp_path / "lfm2.r4dxb"))
    assert cfg.arch == "lfm2_moe" and cfg.moe_router == "sigmoid" and cfg.layer_types == ["conv", "conv"]
    assert "text.layers.1.moe.expert_bias" in w and w["text.layers.1.moe.expert_bias"].dtype.is_floating_point


def test_converter_imports_encoded_trellis_tensors_and_rejects_wrong_ones(tmp_path):
    """--trellis-from: tensors encoded elsewhere are taken as they are after a CPU reconstruction check."""
    import json
    import torch
    from r4dx_b200.cli.convert import load_source, main as convert
    from r4dx_b200.quant.weights import export_trellis_dir, load_weight_set, quantize_weight_set
    from r4dx_b200.quant.trellis import TrellisWeight
    cfg, w = load_source("random:tiny", 0, False, 0)
    q = quantize_weight_set(cfg, w, kb_rule=lambda n: 4)
    body = {k: v for k, v in q.items() if isinstance(v, TrellisWeight) and ".layers.0." in k}
    d = str(tmp_path / "enc")
    export_trellis_dir(body, d)
    out = str(tmp_path / "m.r4dxb")
    assert convert(["--input", "random:tiny", "--output", out, "--trellis-from", d, "--kb-plan", "kb5"]) == 0
    _, back = load_weight_set(out)
    for k, v in body.items():
        assert back[k].kb == 4 and torch.equal(back[k].words, v.words)          # imported, not re-encoded at 5 bits
    other = next(k for k, v in back.items() if isinstance(v, TrellisWeight) and ".layers.1." in k)
    assert back[other].kb == 5
    # a tensor whose codes belong to other weights fails the reconstruction check
    name = next(iter(body))
    bad = dict(body)
    bad[name] = TrellisWeight(torch.roll(body[name].words, 17), body[name].suh, body[name].svh, body[name].N, body[name].K, 4)
    d2 = str(tmp_path / "bad")
    export_trellis_dir(bad, d2)
    with pytest.raises(SystemExit) as e:
        convert(["--input", "random:tiny", "--output", str(tmp_path / "x.r4dxb"), "--trellis-from", d2])
    assert "reconstruction error" in str(e.value)
    man = json.load(open(d + "/trellis_manifest.json"))
    assert man["format"] == "r4dxb-trellis-1" and name in man["tensors"]


def test_converter_keeps_a_vision_tower_and_imports_a_drafter(tmp_path):
    import json
    import torch
    from safetensors.torch import save_file
    from r4dx_b200.cli.convert import main as convert
    from r4dx_b200.models.dflash import load_dflash
    from r4dx_b200.models.vision import VisionConfig
    from r4dx_b200.quant.hf_import import import_hf_vision
    from r4dx_b200.quant.weights import load_weight_set
    # a second-generation drafter checkpoint in the Hugging Face naming, geometry matched to the tiny target (hidden 256)
    H, G, L, V, R, I = 256, 16, 2, 4096, 8, 512
    g = torch.Generator().manual_seed(0)
    n = lambda *s: torch.randn(*s, generator=g) * 0.05
    t = {"fc.weight": n(H, 2 * H), "hidden_norm.weight": 1 + n(H), "norm.weight": 1 + n(H),
         "candidate_selector.hidden_projection.weight": n(R, H), "candidate_selector.predecessor_codebook": n(V, R),
         "candidate_selector.successor_codebook": n(V, R)}
    for i in range(L):
        p = f"layers.{i}."
        t.update({p + "input_layernorm.weight": 1 + n(H), p + "post_attention_layernorm.weight": 1 + n(H),
                  p + "self_attn.q_proj.weight": n(4 * 64, H), p + "self_attn.k_proj.weight": n(2 * 64, H), p + "self_attn.v_proj.weight": n(2 * 64, H),
                  p + "self_attn.o_proj.weight": n(H, 4 * 64), p + "self_attn.q_norm.weight": 1 + n(64), p + "self_attn.k_norm.weight": 1 + n(64),
                  p + "mlp.gate_proj.weight": n(I, H), p + "mlp.up_proj.weight": n(I, H), p + "mlp.down_proj.weight": n(H, I)})
        for mod in ("attention_conv", "mlp_conv"):
            t[p + mod + ".base_kernel"] = n(2, 2, H)
            t[p + mod + ".kernel_projection.weight"] = n(4 * G, H)
    d = tmp_path / "drafter"
    d.mkdir()
    save_file({("model." + k): v.contiguous() for k, v in t.items()}, str(d / "model.safetensors"))
    json.dump({"hidden_size": H, "num_hidden_layers": L, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
               "intermediate_size": I, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "sliding_window": 48,
               "dflash_config": {"target_layer_ids": [0, 2], "mask_token_id": 3, "block_size": 8}}, open(d / "config.json", "w"))
    out = str(tmp_path / "m.r4dxb")
    assert convert(["--input", "random:tiny", "--output", out, "--layouts", "bf16", "--vision", "on", "--dflash-hf", str(d)]) == 0
    cfg, q = load_weight_set(out)
    vw = {k[len("vision."):]: v for k, v in q.items() if k.startswith("vision.")}
    vc = VisionConfig.from_weights(vw)
    assert (vc.depth, vc.hidden_size, vc.num_heads, vc.patch_size, vc.out_hidden_size) == (2, 144, 2, 8, cfg.hidden_size)
    dc, dq = load_dflash(out + ".dflash")
    assert dc.target_layers == (1, 3) and dc.block == 8 and dc.mask_token_id == 3 and dc.rank == R
    assert tuple(dq["layers.1.conv2.base"].shape) == (2, H) and tuple(dq["layers.1.conv3.dyn"].shape) == (2 * G, H)
    assert torch.allclose(dq["layers.0.conv1.base"].float(), t["layers.0.attention_conv.base_kernel"][1].to(torch.bfloat16).float())
    assert tuple(dq["layers.0.gate_up"].wq.shape)[0] == 2 * I
    # Hugging Face vision names map onto the tower's names, the patch kernel is flattened
    hv = import_hf_vision({"model.visual.patch_embed.proj.weight": torch.zeros(144, 3, 2, 8, 8), "model.visual.blocks.0.attn.qkv.bias": torch.zeros(432),
                           "model.visual.merger.linear_fc2.weight": torch.zeros(256, 576), "model.language_model.x": torch.zeros(1)})
    assert set(hv) == {"patch_embed.weight", "blocks.0.qkv.bias", "merger.fc2.weight"} and hv["patch_embed.weight"].shape == (144, 384)


def test_converter_writes_and_reads_the_w8a16_body_layout(tmp_path):
    from r4dx_b200.cli.convert import main as convert
    from r4dx_b200.quant.w4a16 import W8Weight
    from r4dx_b200.quant.weights import dequantize_weight_set, load_weight_set
    out = str(tmp_path / "w8.r4dxb")
    assert convert(["--input", "random:llama", "--output", out, "--layouts", "w8a16", "--selftest"]) == 0
    cfg, q = load_weight_set(out)
    body = [k for k, v in q.items() if isinstance(v, W8Weight)]
    assert len(body) >= 6 * cfg.num_hidden_layers and all(q[k].wq.dtype == torch.uint8 for k in body)
    dq = dequantize_weight_set(q)
    assert dq[body[0]].shape == (q[body[0]].N, q[body[0]].K)


def test_two_stage_split_balanced_by_weight_bytes():
    from r4dx_b200.parallel.pp import choose_split_by_bytes
    assert choose_split_by_bytes([10] * 8) == 4
    assert choose_split_by_bytes([10] * 8, last_stage_extra=20) == 5          # the head rides with stage B: A takes one more layer
    assert choose_split_by_bytes([30, 10, 10, 10, 10, 10]) == 2               # a heavy first layer moves the boundary up
    assert choose_split_by_bytes([1, 1, 1, 100]) == 3
    with pytest.raises(ValueError, match="fits"):
        choose_split_by_bytes([10] * 8, cap=35)
    assert choose_split_by_bytes([10] * 8, cap=40) == 4
    with pytest.raises(ValueError):
        choose_split_by_bytes([5])


def test_plan_only_predicts_what_the_converter_writes(tmp_path, capsys):
    """--plan-only prints tensor count and data bytes from shapes alone; they equal what a real conversion stores."""
    import json
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.weights import load_weight_set
    out = str(tmp_path / "m.r4dxb")
    assert convert_main(["--input", "random:moe", "--output", out, "--layers", "2", "--kb-plan", "mix3.3", "--plan-only"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert not os.path.exists(out) and rep["arch"] == "qwen_hybrid_moe"
    assert convert_main(["--input", "random:moe", "--output", out, "--layers", "2", "--kb-plan", "mix3.3"]) == 0
    cfg, w = load_weight_set(out)
    assert rep["tensors"] == len(w)
    stored = sum(t.nbytes if not isinstance(t, torch.Tensor) else t.numel() * t.element_size() for t in w.values())
    assert rep["data_bytes"] == stored, (rep["data_bytes"], stored)
    assert rep["by_layout"]["trellis"]["tensors"] == sum(type(t).__name__ == "TrellisWeight" for t in w.values())


def test_group_rules_and_manifest_hash_flags(tmp_path):
    import hashlib
    from r4dx_b200.cli.convert import main as convert_main, parse_group_rule
    from r4dx_b200.quant.weights import export_trellis_dir, load_weight_set
    rule = parse_group_rule("^lm_head$=32,attn=128")
    assert rule("lm_head") == 32 and rule("text.layers.0.attn.qg") == 128 and rule("text.layers.0.mlp.down") is None
    with pytest.raises(SystemExit, match="32, 64 or 128"):
        parse_group_rule("x=48")
    out = str(tmp_path / "a.r4dxb")
    assert convert_main(["--input", "random:tiny", "--output", out, "--layers", "1", "--layouts", "w8a16", "--w4a16-group-rule", "^lm_head$=32",
                         "--w8a16-group", "128"]) == 0
    cfg, w = load_weight_set(out)
    assert w["lm_head"].group == 32 and w["text.layers.0.gdn.in_proj_qkv"].group == 128
    # the trellis import directory is pinned by the hash of its manifest
    out2 = str(tmp_path / "b.r4dxb")
    assert convert_main(["--input", "random:tiny", "--output", out2, "--layers", "1", "--kb-plan", "kb3"]) == 0
    d = str(tmp_path / "enc")
    export_trellis_dir(load_weight_set(out2)[1], d)
    sha = hashlib.sha256(open(os.path.join(d, "trellis_manifest.json"), "rb").read()).hexdigest()
    out3 = str(tmp_path / "c.r4dxb")
    with pytest.raises(SystemExit, match="hashes to"):
        convert_main(["--input", "random:tiny", "--output", out3, "--layers", "1", "--kb-plan", "kb3", "--trellis-from", d,
                      "--trellis-manifest-sha256", "0" * 64])
    assert convert_main(["--input", "random:tiny", "--output", out3, "--layers", "1", "--kb-plan", "kb3", "--trellis-from", d,
                         "--trellis-manifest-sha256", sha.upper()]) == 0


def test_reduced_vocabulary_draft_head_is_baked_with_mtp(tmp_path, capsys):
    import json
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant import w4a16
    from r4dx_b200.quant.weights import load_weight_set
    ids_file = tmp_path / "ids.json"
    ids = sorted(set(torch.randint(0, 4096, (300,), generator=torch.Generator().manual_seed(0)).tolist()))
    ids_file.write_text(json.dumps({"ids": ids}))
    out = str(tmp_path / "m.r4dxb")
    assert convert_main(["--input", "random:tiny", "--output", out, "--kb-plan", "kb3", "--mtp", "--draft-vocab-ids", str(ids_file)]) == 0
    cfg, w = load_weight_set(out)
    vid, dh = w["mtp.draft_head.vocab_ids"], w["mtp.draft_head.lm_head"]
    assert vid.dtype == torch.int32 and vid.numel() % 128 == 0 and vid[:len(ids)].tolist() == ids and int(vid[-1]) == ids[-1]
    assert dh.N == vid.numel() and dh.K == cfg.hidden_size
    full = w4a16.dequantize(w["lm_head"])
    part = w4a16.dequantize(dh)
    assert (part - full[vid.long()]).abs().max().item() < 0.02 * full.abs().max().item()      # both are 4-bit roundings of the same rows
    # without an MTP head the flag is ignored, with a note; ids outside the vocabulary are refused
    out2 = str(tmp_path / "n.r4dxb")
    assert convert_main(["--input", "random:tiny", "--output", out2, "--kb-plan", "kb3", "--layers", "1", "--draft-vocab-ids", str(ids_file)]) == 0
    assert "ignored" in capsys.readouterr().err and "mtp.draft_head.lm_head" not in load_weight_set(out2)[1]
    ids_file.write_text(json.dumps([1, 2, 5000]))
    with pytest.raises(SystemExit, match="must lie in"):
        convert_main(["--input", "random:tiny", "--output", out, "--kb-plan", "kb3", "--mtp", "--draft-vocab-ids", str(ids_file)])


def test_converter_keeps_the_audio_embedder(tmp_path):
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.models.audio import FRAME, WEIGHT_NAME, load_audio_embedder
    from r4dx_b200.quant.weights import load_weight_set
    out = str(tmp_path / "g.r4dxb")
    assert convert_main(["--input", "random:gemma", "--output", out, "--layers", "1", "--kb-plan", "kb3", "--audio", "on"]) == 0
    cfg, w = load_weight_set(out)
    assert w[WEIGHT_NAME].shape == (cfg.hidden_size, FRAME) and w[WEIGHT_NAME].dtype == torch.bfloat16
    emb = load_audio_embedder(w)
    assert emb is not None
    with pytest.raises(SystemExit, match="Gemma-style"):
        convert_main(["--input", "random:tiny", "--output", out, "--layers", "1", "--audio", "on"])


def test_one_tensor_selftest_mode(tmp_path, capsys):
    import json
    from safetensors.torch import load_file, save_file
    from r4dx_b200.cli.convert import main as convert_main
    src = str(tmp_path / "w.safetensors")
    w = torch.randn(256, 128, generator=torch.Generator().manual_seed(1)) * 0.02
    save_file({"w": w.to(torch.bfloat16)}, src)
    outp = str(tmp_path / "back.safetensors")
    assert convert_main(["--selftest-input", src, "--kb-plan", "kb4", "--selftest-output", outp]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["layout"] == "TrellisWeight" and rep["kb"] == 4 and 0 < rep["relative_squared_error"] < 6 * 4.0 ** -4
    assert load_file(outp)["w"].shape == (256, 128)
    assert convert_main(["--selftest-input", src, "--selftest-name", "lm_head", "--w4a16-group-rule", "^lm_head$=32"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["layout"] == "W4Weight" and rep["group"] == 32 and rep["relative_squared_error"] < 0.02
    with pytest.raises(SystemExit, match="--input and --output"):
        convert_main(["--kb-plan", "kb4"])


def test_draft_vocabulary_picker(tmp_path, capsys):
    import json
    from r4dx_b200.utils.draft_vocab import main as dv_main, pick_ids
    rep = pick_ids([[5, 5, 5, 7, 7, 9], [5, 11]], size=3, always=[2])
    assert rep["ids"] == [2, 5, 7] and rep["sample_tokens"] == 8 and abs(rep["coverage"] - 6 / 8) < 1e-9
    assert pick_ids([[1, 2, 3]], size=10, vocab_size=3)["ids"] == [1, 2]           # ids outside the vocabulary are dropped
    txt = tmp_path / "a.txt"
    txt.write_text("hello hello world")
    log = tmp_path / "b.jsonl"
    log.write_text(json.dumps({"messages": [{"role": "user", "content": "hello tool"}]}) + "\n")
    out = str(tmp_path / "ids.json")
    assert dv_main(["--text", str(txt), str(log), "--size", "8", "--out", out]) == 0
    ids = json.load(open(out))["ids"]
    assert len(ids) == 8 and ids == sorted(ids) and ord("l") in ids and ord("o") in ids
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert 0 < rep["coverage"] <= 1 and rep["kept"] == 8


def test_bit_allocation_under_a_byte_budget(tmp_path, capsys):
    import json
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.weights import load_weight_set
    from r4dx_b200.utils import alloc_bits as AB
    assert AB.class_of("text.layers.7.moe.experts.12.gate_up") == "text.layers.7.moe.experts.*.gate_up"
    err = {"a": {3: 1.0, 4: 0.2, 5: 0.05}, "b": {3: 0.5, 4: 0.4, 5: 0.39}, "c": {3: 2.0, 4: 0.5, 5: 0.1}}
    size = {"a": 8000, "b": 8000, "c": 80000}
    base = sum(size.values()) * 3 // 8
    assert AB.allocate(err, size, base) == {"a": 3, "b": 3, "c": 3}
    assert AB.allocate(err, size, base + 1000) == {"a": 4, "b": 3, "c": 3}                  # the best error drop per byte first
    assert AB.allocate(err, size, base + 2000) == {"a": 5, "b": 3, "c": 3}
    assert AB.allocate(err, size, base + 12100) == {"a": 5, "b": 3, "c": 4} or AB.allocate(err, size, base + 12100)["c"] == 4
    assert AB.allocate(err, size, 10 ** 9) == {"a": 5, "b": 5, "c": 5}
    with pytest.raises(ValueError, match="budget"):
        AB.allocate(err, size, base - 1)
    plan = str(tmp_path / "plan.json")
    assert AB.main(["--input", "random:moe", "--layers", "1", "--budget-mib", "0.9", "--out", plan]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    doc = json.load(open(plan))
    assert rep["bytes"] <= 0.9 * 2 ** 20 and 3.0 <= rep["bits_per_weight"] <= 5.0 and doc["format"] == "r4dxb-kb-plan-1"
    assert "text.layers.0.moe.experts.*.gate_up" in doc["classes"]
    out = str(tmp_path / "m.r4dxb")
    assert convert_main(["--input", "random:moe", "--layers", "1", "--output", out, "--kb-plan", "kb3", "--kb-plan-file", plan]) == 0
    cfg, w = load_weight_set(out)
    for name, t in w.items():
        if type(t).__name__ == "TrellisWeight":
            assert t.kb == doc["classes"][AB.class_of(name)], name
