"""Argument parsers and the converter round trip (CPU)."""
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
