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
    if args.tp > 1:
        if world != args.tp:
            raise SystemExit(f"--tp {args.tp} needs {args.tp} ranks (python -m torch.distributed.run --nproc-per-node {args.tp} ...)")
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
        weights = synthetic_weight_set(cfg, device=device, seed=0)
        model_id = f"synthetic-{kind}"
    else:
        gcfg, full = load_weight_set(model_arg, device=device)
        cfg = gcfg.shard(args.tp, rank) if args.tp > 1 else gcfg
        weights = shard_weight_set(gcfg, full, args.tp, rank)
        model_id = os.path.splitext(os.path.basename(model_arg))[0]
    if args.tp > 1:
        from ..parallel.tp_comm import make_comm, spin_limit_for_ms
        comm = make_comm(args.tp, rank, device, mode=args.tp_mode, hidden=gcfg.hidden_size,
                         spin_limit=spin_limit_for_ms(getattr(args, "tp_ar_timeout_ms", 500)))
    model = HybridModel(cfg, weights, max_ctx=args.max_ctx, device=device, comm=comm)
    drafter = None
    if args.mtp > 0 and any(k.startswith("mtp.") for k in weights):
        from ..models.mtp import MtpDrafter
        drafter = MtpDrafter(model, weights)
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
