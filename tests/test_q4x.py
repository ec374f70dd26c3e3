"""qwen4_exp family on the CPU: n-gram ids and table file, the oracle's stream gate, n-gram layer and block-selecting
attention (chunking invariance, the dense limit, the tie rule)."""
import dataclasses

import numpy as np
import pytest
import torch

from r4dx_b200.config import ModelConfig, qwen4_exp_config, tiny_qwen4_exp_config
from r4dx_b200.models.q4x_oracle import Q4xOracle, Q4xState, init_q4x_weights, select_blocks
from r4dx_b200.runtime import ngram as NG


@pytest.fixture(scope="module")
def table(tmp_path_factory):
    cfg = tiny_qwen4_exp_config()
    path = str(tmp_path_factory.mktemp("ngram") / "tiny.r4dx-ngram")
    NG.synthetic_sidecar(path, cfg.vocab_size, cfg.ngram_head_dim, cfg.eos_token_id, seed=3)
    t = NG.NgramTable.open(path, mode="file")
    yield t
    t.close()


def rows_fn(table):
    def f(tokens, history):
        ids = np.asarray(NG.ngram_ids_reference(tokens, table.header, history), dtype=np.int64)
        return table.rows(ids).reshape(len(tokens), -1)
    return f


def test_config_presets_and_json_round_trip():
    for c in (tiny_qwen4_exp_config(), qwen4_exp_config()):
        c.validate()
        assert ModelConfig.from_json(c.to_json()) == c
    c = qwen4_exp_config()
    assert c.is_qwen4_exp and c.ple_layers == [1] and c.num_attention_layers() == 12 and c.ngram_head_dim == 160
    bad = dataclasses.replace(tiny_qwen4_exp_config(), indexer_budget=18)
    with pytest.raises(ValueError):
        bad.validate()
    hf = {"model_type": "qwen4_exp", "text_config": {"model_type": "qwen4_exp", "hidden_size": 256, "num_hidden_layers": 4,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
          "linear_key_head_dim": 64, "linear_value_head_dim": 64, "vocab_size": 4096, "num_experts": 16, "num_experts_per_tok": 4,
          "moe_intermediate_size": 128, "shared_expert_intermediate_size": 128, "hc_count": 4, "hc_lowrank": 32,
          "ple_layer_ids": [2], "ple_embed_dim": 256, "ngram_size": 3, "indexer_budget": 16, "indexer_heads": 2,
          "indexer_head_dim": 64, "output_gate_type": "sigmoid"}}
    import json
    c = ModelConfig.from_json(json.dumps(hf))
    assert c.arch == "qwen4_exp" and c.ple_layers == [1] and c.gdn_gate_act == "sigmoid" and not c.final_norm


def test_ngram_header_round_trip_and_refusals(table, tmp_path):
    h = table.header
    assert NG.NgramHeader.parse(h.pack()) == h
    assert table.verify_sha256()
    raw = bytearray(h.pack())
    raw[0] = ord("X")
    with pytest.raises(NG.NgramError, match="magic"):
        NG.NgramHeader.parse(bytes(raw))
    raw = bytearray(h.pack())
    raw[400] = 1
    with pytest.raises(NG.NgramError, match="padding"):
        NG.NgramHeader.parse(bytes(raw))
    short = tmp_path / "short.r4dx-ngram"
    data = open(table.path, "rb").read()
    short.write_bytes(data[:-h.row_bytes * 3])
    with pytest.raises(NG.NgramError, match="bytes on disk"):
        NG.NgramTable.open(str(short), mode="file")
    t = NG.NgramTable.open(str(short), mode="file", allow_truncated=True)
    with pytest.raises(NG.NgramError, match="could not be read"):
        t.rows(np.asarray([h.rows - 1], dtype=np.int64))          # a short read is an error, never a zero row
    t.close()


def test_ngram_ids_native_equal_reference_for_any_chunking(table):
    h = table.header
    eos = h.eos_token_id
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, 4096, (200,), generator=g).tolist()
    for at in (5, 6, 40, 41, 43, 120):
        toks[at] = eos
    want = NG.ngram_ids_reference(toks, h)
    gen = NG.NgramIds(h)
    assert gen.generate(toks).tolist() == want
    gen.reset()
    got, at = [], 0
    for n in (1, 1, 7, 1, 64, 3, 123):
        got += gen.generate(toks[at:at + n]).tolist()
        at += n
    assert got == want
    # segmentation: right after an end-of-sequence token the 3-gram sees it twice, whatever came before it
    a = NG.ngram_ids_reference([11, eos, 5], h)[2]
    b = NG.ngram_ids_reference([99, eos, 5], h)[2]
    c = NG.ngram_ids_reference([5], h)[0]
    assert a == b == c
    x = NG.ngram_ids_reference([11, 12, 5], h)[2]
    y = NG.ngram_ids_reference([99, 12, 5], h)[2]
    assert x[:8] == y[:8] and x[8:] != y[8:]                      # 2-gram heads ignore the token two back
    for row in want:
        for hd, i in enumerate(row):
            assert h.head_offsets[hd] <= i < h.head_offsets[hd] + h.head_primes[hd]
    with pytest.raises(NG.NgramError):
        gen.generate([-1])
    snap = gen.snapshot()
    r1 = gen.generate([3, 4]).tolist()
    gen.restore(snap)
    assert gen.generate([3, 4]).tolist() == r1


def test_table_placements_agree(table):
    toks = [1, 2, 3, 7, 9, 10]
    a = table.gather_host(toks)
    t2 = NG.NgramTable.open(table.path, mode="pinned", device="cpu")
    b = t2.gather_host(toks)
    t2.close()
    assert a.shape == (6, 256) and torch.equal(a, b)


def test_select_blocks_prefers_recent_blocks_on_ties():
    s = torch.tensor([0.0, 2.0, 0.0, 2.0, 0.0, 1.0, 0.0])
    assert select_blocks(s, 3).tolist() == [1, 3, 5]
    assert select_blocks(s, 4).tolist() == [1, 3, 5, 6]           # among the zero scores the latest block wins
    assert select_blocks(s, 6).tolist() == [1, 2, 3, 4, 5, 6]


@pytest.fixture(scope="module")
def tiny(table):
    cfg = tiny_qwen4_exp_config()
    w = init_q4x_weights(cfg, seed=1)
    return cfg, w, Q4xOracle(cfg, w, rows_fn(table))


def test_oracle_is_chunking_invariant_and_selects_blocks(tiny):
    cfg, w, m = tiny
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (45,), generator=g)
    ids[20] = cfg.eos_token_id
    full, st = m.forward(ids)
    sel = st.selected[3]
    assert sel[10] is None and sel[18] is None                   # up to budget / ratio complete blocks: dense
    assert sel[19] is not None and len(sel[19]) == 16 + 0        # 5 complete blocks, the best 4 kept, no open tail
    assert len(sel[44]) == 16 + 1 and sel[44][-1] == 44 and sel[44] == sorted(sel[44])
    st2 = Q4xState()
    parts = []
    for a, b in ((0, 1), (1, 8), (8, 9), (9, 30), (30, 45)):
        lg, st2 = m.forward(ids[a:b], st2)
        parts.append(lg)
    got = torch.cat(parts, 0)
    assert (got - full).abs().max().item() < 2e-4 * full.abs().max().item() + 1e-5
    assert st2.selected[3][-1] == sel[44]


def test_sparse_attention_equals_dense_while_everything_fits_the_budget(tiny, table):
    cfg, w, _ = tiny
    wide = dataclasses.replace(cfg, indexer_budget=4096)
    dense = dataclasses.replace(cfg, indexer_heads=0)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(9))
    a, _ = Q4xOracle(wide, w, rows_fn(table)).forward(ids)
    b, _ = Q4xOracle(dense, w, rows_fn(table)).forward(ids)
    c, _ = Q4xOracle(cfg, w, rows_fn(table)).forward(ids)
    assert torch.allclose(a, b, atol=1e-5)
    assert (c[:19] - b[:19]).abs().max().item() < 1e-5            # rows that still see everything
    assert (c[30:] - b[30:]).abs().max().item() > 1e-4            # later rows drop blocks


def test_stream_gate_and_ngram_layer_move_the_output(tiny, table):
    cfg, w, m = tiny
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    base, _ = m.forward(ids)
    zero_rows = lambda toks, hist: torch.zeros(len(toks), cfg.ple_embed_dim)
    other, _ = Q4xOracle(cfg, w, zero_rows).forward(ids)
    assert (base - other).abs().max().item() > 1e-4
    # the injection weights are 2 * sigmoid(.): a zero inject projection gives exactly 1 per stream
    w2 = dict(w)
    for k in w:
        if k.endswith(".inject"):
            w2[k] = torch.zeros_like(w[k])
    m2 = Q4xOracle(cfg, w2, rows_fn(table))
    h = torch.randn(3, cfg.hc_count * cfg.hidden_size)
    x, inj = m2.hc_prep("text.layers.0.hc.attn.", h)
    assert x.shape == (3, cfg.hidden_size) and torch.allclose(inj, torch.ones(3, cfg.hc_count))
    out = torch.randn(3, cfg.hidden_size)
    assert torch.allclose(m2.hc_inject(h, out, inj), h + out.repeat(1, cfg.hc_count))


def test_awq_pack_quantized_round_trip_and_view():
    from r4dx_b200.quant import awq
    g = torch.Generator().manual_seed(0)
    w = torch.randn(20, 256, generator=g) * 0.05               # N not a multiple of 8: the zero points pad their last word
    t = awq.quantize(w, 128)
    assert t["weight_packed"].shape == (20, 32) and t["weight_zero_point"].shape == (3, 2) and t["weight_packed"].dtype == torch.int32
    d = awq.dequantize(t["weight_packed"], t["weight_scale"], t["weight_zero_point"], 20, 256, 128)
    assert d.dtype == torch.bfloat16 and (d.float() - w).abs().max().item() < 0.6 * float(t["weight_scale"].float().max())
    # element by element from the definition: nibble j of word c is column 8 c + j; nibble n % 8 of zero-point row n / 8
    for n, k in ((0, 0), (7, 9), (19, 255), (8, 128)):
        q = (int(t["weight_packed"][n, k // 8]) >> (4 * (k % 8))) & 0xF
        zp = (int(t["weight_zero_point"][n // 8, k // 128]) >> (4 * (n % 8))) & 0xF
        want = torch.tensor(float(q - zp) * float(t["weight_scale"][n, k // 128])).to(torch.bfloat16)
        assert d[n, k] == want
    raw = {"a.b." + k_: v for k_, v in t.items()}
    raw["a.norm.weight"] = torch.ones(4)
    view = awq.AwqView(raw)
    assert sorted(view) == ["a.b.weight", "a.norm.weight"] and "a.b.weight_packed" not in view and "a.b.weight" in view
    assert torch.equal(view["a.b.weight"], d) and torch.equal(view["a.norm.weight"], torch.ones(4))
    with pytest.raises(KeyError):
        view["a.b.weight_scale"]
    del raw["a.b.weight_shape"]
    with pytest.raises(ValueError, match="weight_shape"):
        awq.AwqView(raw)
    cfg_ok = '{"quantization_config": {"format": "pack-quantized", "config_groups": {"g0": {"weights": {"num_bits": 4, "strategy": "group", "symmetric": false, "group_size": 128}}}}}'
    assert awq.pack_scheme(cfg_ok) == 128 and awq.pack_scheme("{}") is None
    with pytest.raises(ValueError):
        awq.pack_scheme(cfg_ok.replace('"num_bits": 4', '"num_bits": 8'))


def test_checkpoint_names_round_trip_through_the_importer(tiny):
    from r4dx_b200.quant.hf_import import config_from_hf, export_qwen4_exp, import_hf_weights
    cfg, w, _ = tiny
    hf = export_qwen4_exp(cfg, w)
    assert "model.language_model.layers.3.self_attn.indexer.index_qk_proj.weight" in hf
    assert "model.language_model.layers.1.ple.conv1d.weight" in hf and hf["model.language_model.layers.1.ple.conv1d.weight"].dim() == 3
    assert "model.language_model.layers.0.attn_hyper_connection.block_inject_weight.weight" in hf
    back = import_hf_weights(cfg, hf)
    assert set(back) == set(w)
    for k_ in w:
        assert torch.equal(back[k_], w[k_].float()), k_
    import json
    text = {"model_type": "qwen4_exp", "hidden_size": 256, "num_hidden_layers": 4, "layer_types": cfg.layer_types,
            "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
            "linear_key_head_dim": 64, "linear_value_head_dim": 64, "vocab_size": 4096, "num_experts": 16, "num_experts_per_tok": 4,
            "moe_intermediate_size": 128, "shared_expert_intermediate_size": 128, "hc_count": 4, "hc_lowrank": 32,
            "ple_layer_ids": [2], "ple_embed_dim": 256, "ple_conv_kernel_size": 4, "ngram_size": 3, "indexer_n_heads": 2,
            "indexer_kv_heads": 1, "indexer_head_dim": 64, "indexer_budget": 16, "output_gate_type": "sigmoid", "eos_token_id": 7}
    c2 = config_from_hf(json.dumps({"model_type": "qwen4_exp", "text_config": text}))
    assert c2 == cfg


def test_converter_writes_a_container_that_records_its_ngram_table(tmp_path):
    import json
    from r4dx_b200.cli.convert import main as convert_main
    from r4dx_b200.quant.container import Container
    from r4dx_b200.quant.weights import load_weight_set
    out, side = str(tmp_path / "q4x.r4dxb"), str(tmp_path / "q4x.r4dx-ngram")
    with pytest.raises(SystemExit, match="ngram-sidecar"):
        convert_main(["--input", "random:q4x", "--output", out, "--layers", "2", "--kb-plan", "kb3"])
    with pytest.raises(SystemExit, match="does not support: --rotate, --mtp"):
        convert_main(["--input", "random:q4x", "--output", out, "--layers", "2", "--ngram-sidecar", side, "--rotate", "q2a", "--mtp"])
    assert convert_main(["--input", "random:q4x", "--output", out, "--layers", "2", "--kb-plan", "kb3", "--ngram-sidecar", side]) == 0
    cfg, w = load_weight_set(out)
    assert cfg.is_qwen4_exp and cfg.num_hidden_layers == 2 and cfg.ple_layers == [1]
    assert w["text.layers.0.hc.attn.down"].dtype == torch.bfloat16 and "text.layers.1.ple.conv1d" in w and "text.hc_final.up" in w
    assert type(w["text.layers.0.gdn.in_proj_qkv"]).__name__ == "TrellisWeight"
    rec = json.loads(Container(out).metadata["ngram_sidecar"])
    t = NG.NgramTable.open(side, mode="file")
    assert rec["path"] == "q4x.r4dx-ngram" and rec["rows"] == t.header.rows and rec["sha256"] == t.header.body_sha256.hex()
    assert t.verify_sha256()
    t.close()


def test_table_file_from_a_checkpoints_own_shards(tmp_path, table):
    """A checkpoint directory with the table in four shards over two files + the hash buffers -> the same table file."""
    import json
    from safetensors.torch import save_file
    h = table.header
    body = table.rows(np.arange(h.rows, dtype=np.int64))
    cuts = [0, 1000, 5000, 9000, h.rows]
    pre = "model.language_model.layers.1.ple.ple_embedding."
    f1 = {pre + f"ngram_embedding.shard_{i}.weight": body[cuts[i]:cuts[i + 1]].contiguous() for i in (0, 2)}
    f2 = {pre + f"ngram_embedding.shard_{i}.weight": body[cuts[i]:cuts[i + 1]].contiguous() for i in (1, 3)}
    f2[pre + "layer_multipliers"] = torch.tensor(h.multipliers, dtype=torch.int64)
    f2[pre + "ngram_heads_vocab_sizes"] = torch.tensor(h.head_primes, dtype=torch.int64)
    f2[pre + "ngram_heads_offsets"] = torch.tensor(h.head_offsets, dtype=torch.int64)
    d = tmp_path / "ckpt"
    d.mkdir()
    save_file(f1, str(d / "model-00001.safetensors"))
    save_file(f2, str(d / "embedding-model-00001.safetensors"))
    wm = {k: "model-00001.safetensors" for k in f1}
    wm.update({k: "embedding-model-00001.safetensors" for k in f2})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    (d / "config.json").write_text(json.dumps({"text_config": {"ple_layer_ids": [2], "split_ngram_parts": 4, "eos_token_id": h.eos_token_id}}))
    out = str(tmp_path / "repacked.r4dx-ngram")
    assert NG.main(["repack", "--model-dir", str(d), "--out", out]) == 0
    t = NG.NgramTable.open(out, mode="file")
    assert t.header.rows == h.rows and t.header.head_primes == h.head_primes and t.header.multipliers == h.multipliers
    assert t.header.body_sha256 == h.body_sha256 and t.verify_sha256()
    toks = [5, 6, 7, h.eos_token_id, 8]
    assert torch.equal(t.gather_host(toks), NG.NgramTable.open(table.path, mode="file").gather_host(toks))
    t.close()
    assert NG.main(["verify", "--sidecar", out]) == 0
    (d / "config.json").write_text(json.dumps({"text_config": {"ple_layer_ids": [2], "split_ngram_parts": 5}}))
    with pytest.raises(NG.NgramError, match="expected shard_0..shard_4"):
        NG.repack_from_checkpoint(str(d), out)


def test_calibration_and_kl_report_run_on_the_family(tmp_path, table):
    """Hessians of a 2-layer model (experts that saw fewer rows than input channels get a damped diagonal), KV descales
    of its attention layer, and the KL report of a quantized set, all through the family's own oracle."""
    import json
    from r4dx_b200.quant import calibrate
    from r4dx_b200.quant.calibrate import capture_hessians
    cfg = tiny_qwen4_exp_config()
    w = init_q4x_weights(cfg, seed=2)
    prompts = [torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(s)) for s in range(2)]
    counts = {}
    H = capture_hessians(cfg, w, prompts, ngram_table=table, counts=counts)
    assert counts["text.layers.0.gdn.in_proj_qkv"] == 48 and H["text.layers.0.gdn.in_proj_qkv"].shape == (256, 256)
    ex = [k for k in H if ".experts." in k and k.endswith("gate_up")]
    assert ex and all(counts[k] < 256 for k in ex)                # 48 rows x top-4 over 16 experts: no expert sees 256 rows
    h = H[ex[0]]
    assert torch.equal(h, torch.diag(torch.diagonal(h))) and float(torch.diagonal(h).min()) > 0
    dense = H["text.layers.0.gdn.in_proj_qkv"]                    # 48 rows < 256 channels as well: diagonal, too
    assert torch.equal(dense, torch.diag(torch.diagonal(dense)))
    out = str(tmp_path / "kv.json")
    with pytest.raises(SystemExit, match="ngram-sidecar"):
        calibrate.main(["kv", "--input", "random:q4x", "--tokens", "16", "--prompts", "1", "--out", out])
    assert calibrate.main(["kv", "--input", "random:q4x", "--tokens", "16", "--prompts", "1", "--out", out, "--ngram-sidecar", table.path]) == 0
    kv = json.load(open(out))
    assert list(kv) == ["3"] and len(kv["3"]["k"]) == cfg.num_key_value_heads and min(kv["3"]["k"]) > 0
    from r4dx_b200.utils import kl_report
    import io, contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert kl_report.main(["--input", "random:q4x", "--kb-plan", "kb4", "--tokens", "16", "--prompts", "1", "--layers", "2",
                               "--ngram-sidecar", table.path]) == 0
    rep = json.loads(buf.getvalue().strip().splitlines()[-1])
    assert rep["positions"] == 16 and 0 <= rep["kl_mean"] < 1.0


def test_tie_rule_noise_floor_tool(table, tiny):
    """With exact ties forced (two equal keys blocks cannot be told apart by score) the two tie rules pick different blocks
    on some rows and the report says so; KL of a model against itself under one rule is 0."""
    from r4dx_b200.utils.qsa_noise_floor import noise_floor, select_blocks_oldest
    cfg, w, _ = tiny
    s = torch.tensor([0.0, 2.0, 0.0, 2.0, 0.0, 1.0, 0.0])
    assert select_blocks_oldest(s, 4).tolist() == [0, 1, 3, 5] and select_blocks(s, 4).tolist() == [1, 3, 5, 6]
    w2 = dict(w)
    w2["text.layers.3.attn.indexer.qk"] = torch.zeros_like(w["text.layers.3.attn.indexer.qk"])    # every block scores 0: all ties
    ids = [torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(4))]
    rep = noise_floor(cfg, w2, table, ids)
    assert rep["sparse_rows"] == 21 and rep["rows_where_the_rules_pick_different_blocks"] == 21
    assert rep["kl_mean"] > 0
    rep0 = noise_floor(cfg, w, table, ids)
    assert rep0["rows_where_the_rules_pick_different_blocks"] <= rep["rows_where_the_rules_pick_different_blocks"]


def test_direct_row_reads_equal_buffered_reads(table, tmp_path):
    """O_DIRECT row reads (aligned spans around each row, rows that straddle a sector boundary, the file's last rows) give
    the same rows as buffered reads; a file system that refuses O_DIRECT says so."""
    import shutil
    path = str(tmp_path / "copy.r4dx-ngram")                     # (the default tmp dir may sit on a file system without O_DIRECT)
    shutil.copyfile(table.path, path)
    try:
        t = NG.NgramTable.open(path, mode="file", direct=True, threads=3)
    except NG.NgramError as e:
        assert "O_DIRECT" in str(e)
        pytest.skip("this file system refuses O_DIRECT")
    h = t.header
    ids = np.asarray([0, 1, 11, 12, 13, h.rows - 1, h.rows - 2, 4095 // h.row_bytes, 4096 // h.row_bytes, 1234, 7], dtype=np.int64)
    assert torch.equal(t.rows(ids), table.rows(ids))
    with pytest.raises(NG.NgramError, match="could not be read"):
        t.rows(np.asarray([h.rows], dtype=np.int64))
    t.close()
