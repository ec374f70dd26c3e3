"""r4dxb-convert: fp32/bf16 checkpoint (safetensors + config.json) or a random init -> quantized container.

Two-phase writer (plan, then stream), `.partial` + rename, optional re-open self test with a reconstruction
error bound per tensor, optional reuse of unchanged tensors from an older container guarded by sha256
(reference: src/convert/main.cpp:1-120)."""
from __future__ import annotations

import hashlib
import json
import os
import sys

import torch

from .args import convert_parser


def _kb_rule(plan: str, plan_file: str = None):
    from ..quant.weights import default_kb_rule, moe_kb_rule
    base = {"mix4.5": default_kb_rule, "mix3.3": moe_kb_rule, "kb3": lambda n: 3, "kb4": lambda n: 4, "kb5": lambda n: 5}[plan]
    if not plan_file:
        return base
    from ..utils.alloc_bits import class_of
    doc = json.load(open(plan_file))
    if doc.get("format") != "r4dxb-kb-plan-1" or not isinstance(doc.get("classes"), dict):
        raise SystemExit(f"--kb-plan-file {plan_file}: not a bit-width plan")
    classes = {k: int(v) for k, v in doc["classes"].items()}
    if any(v not in (3, 4, 5) for v in classes.values()):
        raise SystemExit(f"--kb-plan-file {plan_file}: widths must be 3, 4 or 5")
    return lambda name: classes.get(class_of(name), base(name))


def parse_group_rule(text: str):
    """'REGEX=GROUP,REGEX=GROUP' -> name -> group or None (first match wins; groups 32, 64 or 128)."""
    import re
    rules = []
    for part in [p_ for p_ in text.split(",") if p_]:
        if "=" not in part:
            raise SystemExit(f"--w4a16-group-rule: '{part}' is not REGEX=GROUP")
        rx, g = part.rsplit("=", 1)
        if g not in ("32", "64", "128"):
            raise SystemExit(f"--w4a16-group-rule: group {g} is not 32, 64 or 128")
        try:
            rules.append((re.compile(rx), int(g)))
        except re.error as e:
            raise SystemExit(f"--w4a16-group-rule: bad pattern {rx!r}: {e}")
    if not rules:
        return None
    return lambda name: next((g for rx, g in rules if rx.search(name)), None)


def load_source(spec: str, layers: int, mtp: bool, seed: int, raw_out=None):
    """(config, fp32 weights under this engine's names).  ``raw_out``: a dict that receives the checkpoint's own tensors
    when the source is a Hugging Face directory (the vision tower is imported from them)."""
    from ..config import (ModelConfig, small_hybrid_config, tiny_gemma_config, tiny_hybrid_config, tiny_lfm2_config,
                          tiny_llama_config, tiny_moe_config)
    from ..models.oracle import init_weights
    if spec.startswith("random:"):
        # tiny random-init models of every family (reference: tools/convert_ref/make_tiny_*.py)
        from ..config import tiny_qwen4_exp_config
        makers = {"tiny": tiny_hybrid_config, "small": small_hybrid_config, "moe": tiny_moe_config, "llama": tiny_llama_config,
                  "gemma": tiny_gemma_config, "lfm2": tiny_lfm2_config, "q4x": tiny_qwen4_exp_config}
        kind = spec.split(":", 1)[1]
        if kind not in makers:
            raise SystemExit(f"unknown random model {kind!r}; one of {sorted(makers)}")
        cfg = makers[kind]()
        if layers:
            cfg.num_hidden_layers, cfg.layer_types = layers, cfg.layer_types[:layers]
            cfg.ple_layers = [i for i in cfg.ple_layers if i < layers]
        if cfg.is_qwen4_exp:
            from ..models.q4x_oracle import init_q4x_weights
            return cfg, init_q4x_weights(cfg, seed)
        return cfg, init_weights(cfg, seed, with_mtp=mtp)
    if spec.endswith(".gguf"):
        from ..quant.gguf import import_gguf
        cfg, w = import_gguf(spec)
        if layers:
            cfg.num_hidden_layers, cfg.layer_types = layers, cfg.layer_types[:layers]
            w = {k: v for k, v in w.items() if not k.startswith("text.layers.") or int(k.split(".")[2]) < layers}
        return cfg, w
    from safetensors import safe_open
    d = spec if os.path.isdir(spec) else os.path.dirname(spec)
    cfg_text = open(os.path.join(d, "config.json")).read()
    files = [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith(".safetensors")] if os.path.isdir(spec) else [spec]
    w = {}
    for f in files:
        with safe_open(f, "pt") as sf:
            for k in sf.keys():
                w[k] = sf.get_tensor(k)
    if any(k.startswith("text.layers.") for k in w):       # already in this engine's naming
        return ModelConfig.from_json(cfg_text), w
    # a Hugging Face checkpoint: read its config.json and rename / reshape the tensors
    from ..quant.hf_import import config_from_hf, import_hf_weights
    from ..quant import awq
    group = awq.pack_scheme(cfg_text)
    if group is not None:
        w = awq.AwqView(w, group)            # int4 pack-quantized linears read as bf16 weights, dequantized when touched
    if raw_out is not None:
        raw_out.update({k: w[k] for k in w if "visual." in k or "vision_tower." in k} if group is not None else w)
    cfg = config_from_hf(cfg_text)
    if layers:
        cfg.num_hidden_layers, cfg.layer_types = layers, cfg.layer_types[:layers]
    return cfg, import_hf_weights(cfg, w)


def plan_container(cfg, w, layout: str, kb_rule, head_group: int, lm_head: str = "w4a16", keep=()) -> dict:
    """What the converter would write, from shapes alone: per tensor the layout, the bit width and the stored bytes (the same
    rules as ``quantize_weight_set`` + ``save_weight_set``; reference: src/convert/main.cpp --plan-only)."""
    from ..quant.weights import F32_NAMES, is_quantized_linear
    plan, by_layout = {}, {}
    for name, t in w.items():
        shape = tuple(t.shape)
        numel = 1
        for d in shape:
            numel *= d
        leaf = name.split(".")[-1]
        kept = any(s_ in name for s_ in keep)
        if name == "lm_head" and lm_head != "bf16" and layout != "bf16" and not kept:
            N, K = shape
            lay, bits, nbytes = "w4a16", 4, N * K // 2 + N * (K // head_group) * 4
        elif not kept and is_quantized_linear(name) and layout == "trellis" and len(shape) == 2 and shape[0] % 128 == 0 and shape[1] % 128 == 0:
            N, K = shape
            kb = kb_rule(name)
            lay, bits, nbytes = "trellis", kb, N * K * kb // 8 + 2 * K + 2 * N
        elif not kept and is_quantized_linear(name) and layout == "w8a16" and len(shape) == 2 and shape[0] % 128 == 0 and shape[1] % 128 == 0:
            N, K = shape
            lay, bits, nbytes = "w8a16", 8, N * K + N * (K // head_group) * 2
        elif not kept and is_quantized_linear(name) and layout == "w4a16" and len(shape) == 2:
            N, K = shape
            lay, bits, nbytes = "w4a16", 4, N * K // 2 + N * (K // head_group) * 4
        elif leaf in F32_NAMES or name.startswith("rotation."):
            lay, bits, nbytes = "f32", 32, numel * 4
        else:
            lay, bits, nbytes = "bf16", 16, numel * 2
        plan[name] = {"layout": lay, "bits": bits, "shape": list(shape), "bytes": nbytes}
        agg = by_layout.setdefault(lay, {"tensors": 0, "bytes": 0})
        agg["tensors"] += 1
        agg["bytes"] += nbytes
    return {"tensors": len(plan), "data_bytes": sum(v["bytes"] for v in plan.values()), "by_layout": by_layout, "plan": plan}


def _selftest_one(args) -> int:
    """Quantizes one tensor through the same code path a conversion takes and reports how well it reconstructs
    (reference: src/convert/main.cpp:223-226 has the same one-tensor mode for its layouts)."""
    from safetensors.torch import load_file, save_file
    from ..config import tiny_hybrid_config
    from ..quant.weights import dequantize_weight_set, quantize_weight_set
    t = load_file(args.selftest_input).get("w")
    if t is None or t.dim() != 2:
        raise SystemExit("--selftest-input: the file must hold one 2-D tensor named \"w\"")
    name = args.selftest_name
    layout = args.layouts.split(",")[0]
    q = quantize_weight_set(tiny_hybrid_config(), {name: t.float()}, layout=layout, kb_rule=_kb_rule(args.kb_plan),
                            head_group=args.lm_head_group, seed=args.seed, group_rule=parse_group_rule(args.w4a16_group_rule),
                            w8_group=args.w8a16_group or None)
    back = dequantize_weight_set(q)[name]
    err = float(((back - t.float()) ** 2).sum() / (t.float() ** 2).sum().clamp_min(1e-30))
    stored = q[name]
    rep = {"name": name, "layout": type(stored).__name__ if not isinstance(stored, torch.Tensor) else str(stored.dtype).replace("torch.", ""),
           "shape": list(t.shape), "relative_squared_error": err,
           "bytes": stored.nbytes if not isinstance(stored, torch.Tensor) else stored.numel() * stored.element_size()}
    if hasattr(stored, "kb"):
        rep["kb"] = stored.kb
    if hasattr(stored, "group"):
        rep["group"] = stored.group
    if args.selftest_output:
        save_file({"w": back.to(torch.bfloat16).contiguous()}, args.selftest_output)
    print(json.dumps(rep))
    return 0


def main(argv=None) -> int:
    args = convert_parser().parse_args(argv)
    from ..quant.container import Container
    from ..quant.weights import dequantize_weight_set, load_weight_set, quantize_weight_set, save_weight_set
    if args.threads:
        torch.set_num_threads(args.threads)
    if args.selftest_input:
        return _selftest_one(args)
    if not args.input or not args.output:
        raise SystemExit("--input and --output are required")
    raw = {}
    cfg, w = load_source(args.input, args.layers, args.mtp, args.seed, raw_out=raw)
    if cfg.is_qwen4_exp:
        # text only, its own residual structure: the flags below do not apply (reference: docs/qwen4exp.md "Convert" refuses the same)
        bad = [f for f, on in (("--rotate", args.rotate != "none"), ("--vision on", args.vision == "on"), ("--mtp", args.mtp),
                               ("--dflash-hf", bool(args.dflash_hf)), ("--reuse-tensors-from", bool(args.reuse_tensors_from))) if on]
        if bad:
            raise SystemExit("qwen4_exp does not support: " + ", ".join(bad))
        if not args.ngram_sidecar:
            raise SystemExit("qwen4_exp: --ngram-sidecar FILE is required (the container records the n-gram table it was built for)")
    keep = [s for s in args.keep_bf16.split(",") if s]
    layout = args.layouts.split(",")[0]
    if args.plan_only:
        rep = plan_container(cfg, w, layout, _kb_rule(args.kb_plan, args.kb_plan_file), args.lm_head_group, args.lm_head, keep)
        plan = rep.pop("plan")
        rep["largest"] = [[n, v["layout"], v["bytes"]] for n, v in sorted(plan.items(), key=lambda kv: -kv[1]["bytes"])[:5]]
        rep["arch"] = cfg.arch
        print(json.dumps(rep))
        return 0
    src = {k: v for k, v in w.items()}
    extra_meta = {}
    if args.rotate != "none":
        # the fold happens in fp32 before anything is quantized; the container carries the rotation tensors and their seed
        from ..quant import rotation as rot
        try:
            spec = rot.make_spec(args.rotate, args.rotation_seed, cfg.hidden_size, args.rotation_block or None)
            if args.rotation_out:
                from safetensors.torch import save_file
                save_file(rot.rotation_tensors(spec), args.rotation_out, metadata={"rotation": json.dumps(spec.to_meta())})
                print(f"wrote {args.rotation_out}: rotation tensors only", file=sys.stderr)
                return 0
            src = rot.fold_rotation(cfg, src, spec)
        except ValueError as e:
            raise SystemExit(f"--rotate {args.rotate}: {e}")
        w = src                                  # hashes, reuse and the self test refer to the folded weights
        extra_meta["rotation"] = json.dumps(spec.to_meta())
    hessians = None
    if args.hessians:
        from safetensors.torch import load_file
        hessians = {k: v for k, v in load_file(args.hessians).items() if v.dim() == 2}
    imatrix = None
    if args.imatrix:
        from safetensors.torch import load_file
        imatrix = {k: v for k, v in load_file(args.imatrix).items() if v.dim() == 1}
    imported = {}
    if args.trellis_from and args.trellis_manifest_sha256:
        mpath = os.path.join(args.trellis_from, "trellis_manifest.json")
        try:
            got = hashlib.sha256(open(mpath, "rb").read()).hexdigest()
        except OSError as e:
            raise SystemExit(f"--trellis-from {args.trellis_from}: {e}")
        if got != args.trellis_manifest_sha256.lower():
            raise SystemExit(f"--trellis-manifest-sha256: {mpath} hashes to {got}")
    if args.trellis_from:
        # already-encoded body linears: taken as they are (checked against the checkpoint), everything else is quantized here
        from ..quant.weights import import_trellis_dir
        if args.rotate != "none":
            raise SystemExit("--trellis-from cannot be combined with --rotate: the imported codes were fitted to the unrotated weights")
        try:
            imported, errs = import_trellis_dir(args.trellis_from, src, verify=args.trellis_verify == "full")
        except (OSError, ValueError) as e:
            raise SystemExit(f"--trellis-from {args.trellis_from}: {e}")
        src = {k: v for k, v in src.items() if k not in imported}
        worst = max(errs.items(), key=lambda kv: kv[1]) if errs else ("", 0.0)
        extra_meta["trellis_import"] = json.dumps({"dir": os.path.abspath(args.trellis_from), "tensors": len(imported),
                                                   "verify": args.trellis_verify, "worst": worst[1], "worst_tensor": worst[0]})
        print(f"imported {len(imported)} trellis tensors from {args.trellis_from} (worst reconstruction error {worst[1]:.4f} at {worst[0]})",
              file=sys.stderr)
    q = quantize_weight_set(cfg, src, layout=layout, kb_rule=_kb_rule(args.kb_plan, args.kb_plan_file), head_group=args.lm_head_group, seed=args.seed,
                            encoder=args.encoder, hessians=hessians, imatrix=imatrix, search=args.quant == "search",
                            group_rule=parse_group_rule(args.w4a16_group_rule), w8_group=args.w8a16_group or None,
                            ldlq_damp=args.ldlq_damp)
    q.update(imported)
    if args.vision == "on":
        # the tower stays bf16 under "vision."; a random source gets a small random tower of the serving code's test geometry
        if raw:
            from ..quant.hf_import import import_hf_vision
            vw = import_hf_vision(raw)
            if not vw:
                raise SystemExit("--vision on: the checkpoint has no visual.* tensors")
        else:
            from ..models.vision import VisionConfig, init_vision_weights
            vw = init_vision_weights(VisionConfig(depth=2, hidden_size=144, num_heads=2, intermediate_size=256, patch_size=8,
                                                  out_hidden_size=cfg.hidden_size, num_position_embeddings=64), args.seed)
        for k, v in vw.items():
            q["vision." + k] = v.to(torch.bfloat16)
    if args.audio == "on":
        # the encoder-free audio embedder rides along in bf16 (reference: src/convert/main.cpp:184-186, --audio on copies
        # model.embed_audio.* as audio.*); a random source gets a random projection of the serving code's shape
        from ..models.audio import FRAME, WEIGHT_NAME
        if cfg.arch != "gemma":
            raise SystemExit("--audio on: the audio front end belongs to the Gemma-style family")
        found = {}
        for k, v in raw.items():
            for pre in ("model.embed_audio.", "embed_audio."):
                if k.startswith(pre):
                    found["audio.embed_audio." + k[len(pre):]] = v.to(torch.bfloat16)
        if not found:
            if raw:
                raise SystemExit("--audio on: the checkpoint has no embed_audio.* tensors")
            gen = torch.Generator().manual_seed(args.seed + 5)
            found[WEIGHT_NAME] = (torch.randn(cfg.hidden_size, FRAME, generator=gen) * 0.02).to(torch.bfloat16)
        if WEIGHT_NAME not in found or tuple(found[WEIGHT_NAME].shape) != (cfg.hidden_size, FRAME):
            raise SystemExit(f"--audio on: {WEIGHT_NAME} must be [{cfg.hidden_size}, {FRAME}]")
        q.update(found)
    if args.draft_vocab_ids:
        # reduced-vocabulary head for the MTP drafter's own drafts (the verify pass still scores the full vocabulary, so the
        # output stays exact; reference: src/convert/main.cpp:165-169).  Ignored without --mtp, as there.
        if args.mtp and any(k.startswith("mtp.") for k in w):
            from ..quant import w4a16 as W4
            raw_ids = json.load(open(args.draft_vocab_ids))
            ids = sorted({int(i) for i in (raw_ids["ids"] if isinstance(raw_ids, dict) else raw_ids)})
            if not ids or ids[0] < 0 or ids[-1] >= cfg.vocab_size:
                raise SystemExit(f"--draft-vocab-ids: ids must lie in [0, {cfg.vocab_size})")
            while len(ids) % 128:
                ids.append(ids[-1])                  # padded with a repeat of the last id: the lowest index wins ties, same token
            sel = torch.tensor(ids, dtype=torch.long)
            rows = w["lm_head"].float()[sel]
            q["mtp.draft_head.lm_head"] = rows.to(torch.bfloat16) if args.lm_head == "bf16" else W4.quantize(rows, args.lm_head_group)
            q["mtp.draft_head.vocab_ids"] = sel.to(torch.int32)
        else:
            print("--draft-vocab-ids ignored: the container has no MTP head (--mtp)", file=sys.stderr)
    for k in list(q):
        if any(s in k for s in keep):
            q[k] = w[k].to(torch.bfloat16)
    if args.lm_head == "bf16":
        q["lm_head"] = w["lm_head"].to(torch.bfloat16)
    if args.kv_calib:
        cal = json.load(open(args.kv_calib))
        for name, amax in cal.items():
            q[name] = torch.tensor(amax, dtype=torch.float32) / 448.0
    reused = 0
    if args.reuse_tensors_from and os.path.exists(args.reuse_tensors_from):
        old = Container(args.reuse_tensors_from)
        src_hash = json.loads(old.metadata.get("source_sha256", "{}"))
        _, oldq = load_weight_set(args.reuse_tensors_from)
        for k, v in w.items():
            h = hashlib.sha256(v.detach().float().contiguous().numpy().tobytes()).hexdigest()
            if src_hash.get(k) == h and k in oldq:
                q[k] = oldq[k]
                reused += 1
    if cfg.is_qwen4_exp:
        from ..runtime import ngram as NG
        if not os.path.exists(args.ngram_sidecar):
            if not args.input.startswith("random:"):
                raise SystemExit(f"--ngram-sidecar {args.ngram_sidecar}: no such file")
            NG.synthetic_sidecar(args.ngram_sidecar, cfg.vocab_size, cfg.ngram_head_dim, cfg.eos_token_id, seed=args.seed)
        t = NG.NgramTable.open(args.ngram_sidecar, mode="file")
        hd = t.header
        t.close()
        if hd.heads * hd.head_dim != cfg.ple_embed_dim or hd.eos_token_id != cfg.eos_token_id:
            raise SystemExit("--ngram-sidecar: the table's geometry or end-of-sequence id does not match the model")
        # recorded, never rehashed at load: name (relative to the container when they share a directory), rows, sha256 of the body
        same_dir = os.path.dirname(os.path.abspath(args.ngram_sidecar)) == os.path.dirname(os.path.abspath(args.output))
        extra_meta["ngram_sidecar"] = json.dumps({"path": os.path.basename(args.ngram_sidecar) if same_dir else os.path.abspath(args.ngram_sidecar),
                                                  "rows": hd.rows, "row_bytes": hd.row_bytes, "sha256": hd.body_sha256.hex()})
    hashes = {k: hashlib.sha256(v.detach().float().contiguous().numpy().tobytes()).hexdigest() for k, v in w.items()}
    extra_meta.update({"source_sha256": json.dumps(hashes), "converter": "r4dxb-convert 0.1", "kb_plan": args.kb_plan})
    save_weight_set(args.output, cfg, q, extra_meta)
    print(f"wrote {args.output}: {len(q)} tensors, {reused} reused", file=sys.stderr)
    if args.dflash_hf:
        # the drafter rides next to the container: <output>.dflash holds its config and source weights (quantized at load)
        from ..models.dflash import save_dflash
        from ..quant.dflash_hf import import_dflash_hf
        try:
            dcfg, dw = import_dflash_hf(args.dflash_hf, w["text.embed_tokens"], cfg.vocab_size)
        except (KeyError, ValueError) as e:
            raise SystemExit(f"--dflash-hf {args.dflash_hf}: {e}")
        if dcfg.hidden != cfg.hidden_size:
            raise SystemExit(f"--dflash-hf: drafter hidden size {dcfg.hidden} != target hidden size {cfg.hidden_size}")
        if max(dcfg.target_layers) >= cfg.num_hidden_layers + 1:
            raise SystemExit(f"--dflash-hf: target layers {dcfg.target_layers} exceed the target's {cfg.num_hidden_layers} layers")
        save_dflash(args.output + ".dflash", dcfg, dw)
        print(f"wrote {args.output}.dflash: {dcfg.layers} layers, taps at layers {list(dcfg.target_layers)}", file=sys.stderr)
    if args.selftest:
        _, back = load_weight_set(args.output)
        dq = dequantize_weight_set(back)
        worst = 0.0
        for k, v in w.items():
            if v.dim() == 2 and k in dq:
                rel = float(((dq[k] - v.float()) ** 2).sum() / (v.float() ** 2).sum().clamp_min(1e-30))
                worst = max(worst, rel)
        print(f"selftest: worst relative squared error {worst:.4f}", file=sys.stderr)
        if worst > 0.2:
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
