"""LoadTextModel: flags -> TextModel (reference dispatch: src/model/tp_model.cpp:1271-1275)."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..config import ModelConfig, qwen_hybrid_27b_config, small_hybrid_config, tiny_hybrid_config


def load_text_model(args, device: Optional[str] = None):
    """Returns (TextModel, tokenizer, chat_template)."""
    from ..models.hybrid import HybridModel
    from ..parallel.shard import shard_weight_set
    from ..quant.weights import load_weight_set, quantize_weight_set, synthetic_weight_set
    from ..runtime.text_model import LocalTextModel
    from ..runtime.tokenizer import load_tokenizer
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = device or f"cuda:{local}"
    torch.cuda.set_device(torch.device(device))
    comm = None
    pp = getattr(args, "pp", 1)
    hybrid = bool(getattr(args, "hybrid", False))
    ep = getattr(args, "ep", 1)
    if hybrid and not (pp == 2 and args.tp == 2):
        raise SystemExit("--hybrid is pipelined prefill + tensor-parallel decode on two ranks: use --pp 2 --tp 2 --hybrid")
    if pp > 1 and not hybrid and args.tp > 1:
        raise SystemExit("--pp 2 with --tp N needs --hybrid (pipelined prefill, then tensor-parallel decode)")
    if ep > 1 and (args.tp > 1 or pp > 1):
        raise SystemExit("--ep N runs data-parallel attention with expert-parallel experts: it does not combine with --tp / --pp")
    ranks_needed = max(args.tp, pp, ep)
    if ranks_needed > 1:
        if world != ranks_needed:
            raise SystemExit(f"this configuration needs {ranks_needed} ranks "
                             f"(python -m torch.distributed.run --nproc-per-node {ranks_needed} ...)")
        import torch.distributed as dist
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device(device))
    model_arg = args.model or "synthetic:tiny"
    if model_arg.startswith("synthetic:"):
        kind = model_arg.split(":", 1)[1]
        gcfg = {"tiny": tiny_hybrid_config, "small": small_hybrid_config, "27b": qwen_hybrid_27b_config}[kind]()
        if args.layers:
            gcfg.num_hidden_layers = args.layers
            gcfg.layer_types = gcfg.layer_types[:args.layers]
        cfg = gcfg.shard(args.tp, rank) if args.tp > 1 else gcfg
        if pp > 1:
            # the pipeline stages run full-width layers of the same model the tensor-parallel ranks hold shards of
            full = synthetic_weight_set(gcfg, device=device, seed=0)
            weights = shard_weight_set(gcfg, full, args.tp, rank) if args.tp > 1 else full
        else:
            full = None
            weights = synthetic_weight_set(cfg, device=device, seed=0)
        model_id = f"synthetic-{kind}"
    else:
        gcfg, full = load_weight_set(model_arg, device=device)
        cfg = gcfg.shard(args.tp, rank) if args.tp > 1 else gcfg
        weights = shard_weight_set(gcfg, full, args.tp, rank)
        model_id = os.path.splitext(os.path.basename(model_arg))[0]
    if gcfg.is_qwen4_exp:
        return _load_qwen4_exp(args, gcfg, weights, model_arg, model_id, device)
    if pp > 1:
        return _load_pipeline(args, gcfg, cfg, weights, full, model_id, device, rank, world, hybrid)
    if ep > 1:
        return _load_expert_parallel(args, gcfg, weights, model_id, device, rank, world)
    if args.tp > 1:
        from ..parallel.tp_comm import make_comm, spin_limit_for_ms
        comm = make_comm(args.tp, rank, device, mode=args.tp_mode, hidden=gcfg.hidden_size,
                         spin_limit=spin_limit_for_ms(getattr(args, "tp_ar_timeout_ms", 500)))
    model = HybridModel(cfg, weights, max_ctx=args.max_ctx, device=device, comm=comm)
    drafter = None
    if args.mtp > 0 and any(k.startswith("mtp.") for k in weights):
        from ..models.mtp import MtpDrafter
        drafter = MtpDrafter(model, weights, use_draft_head=getattr(args, "mtp_draft_head", "on") == "on")
    if getattr(args, "ngram", 0) > 0 and drafter is None:
        from ..models.ngram import NgramDrafter
        drafter = NgramDrafter()
    if getattr(args, "dflash", None):
        from ..models.dflash import DflashDrafter, load_dflash
        dcfg, dweights = load_dflash(args.dflash)
        drafter = DflashDrafter(model, dcfg, dweights)
    tk, tpl = load_tokenizer(args.tokenizer_dir, gcfg.vocab_size)
    local = LocalTextModel(model, model_id=model_id, global_config=gcfg, drafter=drafter,
                           prefill_chunk=getattr(args, "prefill_chunk", 0))
    if args.tp > 1:
        # rank 0 leads (tokenizer, sampling, front door); the others replay its commands (see runtime/tp_model.py)
        import torch.distributed as dist
        from ..parallel.tp_group import FaultSpec, RankGroup
        from ..runtime.tp_model import TpTextModel
        ctl = dist.new_group(backend="gloo")
        group = RankGroup(rank, world, group=ctl, fault=FaultSpec.parse(getattr(args, "tp_fault", "") or ""))
        return TpTextModel(local, group, ctl_group=ctl, comm=comm), tk, tpl
    return local, tk, tpl


def _load_qwen4_exp(args, gcfg, weights, model_arg: str, model_id: str, device):
    """The 4-stream MoE family: one GPU, text only, its n-gram table next to the container (or --ngram-sidecar)."""
    import json
    from ..models.q4x import Qwen4ExpModel
    from ..quant.container import Container
    from ..runtime import ngram as NG
    from ..runtime.text_model import LocalTextModel
    from ..runtime.tokenizer import load_tokenizer
    bad = [f for f, on in (("--tp", args.tp > 1), ("--pp", getattr(args, "pp", 1) > 1), ("--ep", getattr(args, "ep", 1) > 1),
                           ("--mtp", getattr(args, "mtp", 0) > 0), ("--dflash", bool(getattr(args, "dflash", None))),
                           ("--ngram", getattr(args, "ngram", 0) > 0), ("--vision on", getattr(args, "vision", "off") == "on")) if on]
    if bad:
        raise SystemExit("qwen4_exp does not support: " + ", ".join(bad))
    table = None
    if gcfg.ple_layers:
        path = getattr(args, "ngram_sidecar", None)
        if not path:
            rec = json.loads(Container(model_arg).metadata.get("ngram_sidecar", "{}"))
            if not rec:
                raise SystemExit("this container records no n-gram table; pass --ngram-sidecar FILE")
            path = rec["path"] if os.path.isabs(rec["path"]) else os.path.join(os.path.dirname(os.path.abspath(model_arg)), rec["path"])
        placement = getattr(args, "ngram_placement", "device")
        try:
            try:
                # rows read from the file bypass the page cache where the file system allows it (the full table is 95 GiB)
                table = NG.NgramTable.open(path, mode=placement, device=device, direct=(placement == "file"))
            except NG.NgramError as e:
                if "O_DIRECT" not in str(e):
                    raise
                print(f"n-gram table: {e}; reading through the page cache", flush=True)
                table = NG.NgramTable.open(path, mode=placement, device=device)
        except (OSError, NG.NgramError) as e:
            raise SystemExit(f"n-gram table {path}: {e}")
        if not getattr(args, "ngram_sidecar", None) and rec.get("sha256") and table.header.body_sha256.hex() != rec["sha256"]:
            raise SystemExit(f"n-gram table {path} is not the one this container was converted with (sha256 in its header differs)")
    model = Qwen4ExpModel(gcfg, weights, ngram_table=table, max_ctx=args.max_ctx, device=device)
    tk, tpl = load_tokenizer(args.tokenizer_dir, gcfg.vocab_size)
    return LocalTextModel(model, model_id=model_id, global_config=gcfg), tk, tpl


def _facade(local, rank: int, world: int, args, comm=None):
    """Leader/follower facade over ``world`` ranks (rank 0 serves; the others replay its calls)."""
    import torch.distributed as dist
    from ..parallel.tp_group import FaultSpec, RankGroup
    from ..runtime.tp_model import TpTextModel
    ctl = dist.new_group(backend="gloo")
    group = RankGroup(rank, world, group=ctl, fault=FaultSpec.parse(getattr(args, "tp_fault", "") or ""))
    return TpTextModel(local, group, ctl_group=ctl, comm=comm)


def _load_pipeline(args, gcfg, cfg, weights, full, model_id, device, rank, world, hybrid):
    """``--pp 2``: two-stage layer split (prefill pipelined over chunks, decode through both stages);
    with ``--hybrid --tp 2`` the pipeline serves long prompts and decode runs tensor-parallel after a reshard."""
    from ..models.hybrid import HybridModel
    from ..parallel.pp import default_split
    from ..runtime.pp_model import HybridPpTextModel, LayerSplitTextModel
    from ..runtime.tokenizer import load_tokenizer
    split = args.pp_split or default_split(gcfg)
    if not args.pp_split and getattr(args, "pp_balance", "layers") == "bytes":
        from ..parallel.pp import choose_split_by_bytes, layer_bytes
        src = full if full is not None else weights
        nb = lambda name: 0 if name not in src else (src[name].nbytes if not isinstance(src[name], torch.Tensor)
                                                     else src[name].numel() * src[name].element_size())
        split = choose_split_by_bytes(layer_bytes(gcfg, src), nb("text.embed_tokens"), nb("lm_head"))
    if not 0 < split < gcfg.num_hidden_layers:
        raise SystemExit(f"--pp-split {split} must leave both stages at least one of the {gcfg.num_hidden_layers} layers")
    rng = (0, split) if rank == 0 else (split, gcfg.num_hidden_layers)
    # the stage runs full-width layers: the unsharded weights (a synthetic set is re-created unsharded)
    stage_w = full if full is not None else weights
    # the pipeline stages keep state for prompts only: with --hybrid-ctx they hold fewer positions than the decode model, and
    # longer prompts take the tensor-parallel prefill (reference: docs/usage.md "--hybrid-ctx N": the stage-KV capacity)
    stage_ctx = min(args.max_ctx, getattr(args, "hybrid_ctx", 0) or args.max_ctx) if hybrid else args.max_ctx
    stage = HybridModel(gcfg, stage_w, max_ctx=stage_ctx, device=device, layer_range=rng)
    chunk = getattr(args, "prefill_chunk", 0) or 1024
    tk, tpl = load_tokenizer(args.tokenizer_dir, gcfg.vocab_size)
    if not hybrid:
        local = LayerSplitTextModel(stage, rank, split, gcfg, model_id=model_id, chunk=chunk)
        return _facade(local, rank, world, args), tk, tpl
    from ..parallel.tp_comm import make_comm, spin_limit_for_ms
    comm = make_comm(args.tp, rank, device, mode=args.tp_mode, hidden=gcfg.hidden_size,
                     spin_limit=spin_limit_for_ms(getattr(args, "tp_ar_timeout_ms", 500)))
    tp_model = HybridModel(cfg, weights, max_ctx=args.max_ctx, device=device, comm=comm)
    local = HybridPpTextModel(tp_model, stage, rank, world, split, gcfg, model_id=model_id, chunk=chunk,
                              min_rows=getattr(args, "pp_min_rows", 512), prefill_chunk=getattr(args, "prefill_chunk", 0))
    return _facade(local, rank, world, args, comm=comm), tk, tpl


def _load_expert_parallel(args, gcfg, weights, model_id, device, rank, world):
    """``--ep N`` (mixture-of-experts models): every rank keeps the attention / recurrent layers whole and a slice of the
    experts; tokens travel to their experts and back inside the dispatch / combine kernels.  Every rank runs the same
    requests here (the leader serves, followers replay), so the ranks' rows are identical copies."""
    from ..models.hybrid import HybridModel
    from ..parallel.ep import EpComm
    from ..parallel.tp_comm import spin_limit_for_ms
    from ..runtime.text_model import LocalTextModel
    from ..runtime.tokenizer import load_tokenizer
    if not gcfg.is_moe:
        raise SystemExit("--ep needs a mixture-of-experts model")
    if gcfg.num_experts % world:
        raise SystemExit(f"--ep {world} must divide the {gcfg.num_experts} experts")
    from ..models.hybrid import MAX_ROWS
    comm = EpComm(world, rank, device, gcfg, max_rows=MAX_ROWS, spin_limit=spin_limit_for_ms(getattr(args, "tp_ar_timeout_ms", 500)))
    model = HybridModel(gcfg, weights, max_ctx=args.max_ctx, device=device, comm=comm)
    tk, tpl = load_tokenizer(args.tokenizer_dir, gcfg.vocab_size)
    local = LocalTextModel(model, model_id=model_id, global_config=gcfg, prefill_chunk=getattr(args, "prefill_chunk", 0))
    return _facade(local, rank, world, args), tk, tpl
