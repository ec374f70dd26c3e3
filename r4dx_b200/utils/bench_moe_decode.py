"""Batched decode throughput of the hybrid MoE geometry (hidden 2048, 512 experts top-10 + shared expert):
``--batch`` concurrent sequences, attention and the recurrent layers data-parallel (each rank owns batch / world
sequences), routed experts expert-parallel with the in-kernel all-to-all.  Device-timed, max over ranks.

    python -m r4dx_b200.utils.bench_moe_decode --batch 64 --ctx 2048                       # one GPU
    python -m torch.distributed.run --nproc-per-node 8 -m r4dx_b200.utils.bench_moe_decode --batch 64
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--prefill", type=int, default=0, help="one GPU: time a cold prefill of this many tokens instead of decode steps")
    ap.add_argument("--real-prefill", type=int, default=0, metavar="P",
                    help="batched decode: every slot is prefilled with P random tokens (real caches and recurrent state) "
                         "instead of being positioned at --ctx with empty caches")
    ap.add_argument("--single", action="store_true", help="one sequence through the CUDA-graph decode path (one GPU)")
    ap.add_argument("--family", default="qwen_moe", choices=["qwen_moe", "lfm2", "qwen4_exp"],
                    help="lfm2: the short-conv + attention MoE geometry (40 layers, 64 experts top-4); qwen4_exp: 4-stream "
                         "residual, block-selecting attention, n-gram layer, 512 experts of inner width 640; both --single only")
    ap.add_argument("--positioned", action="store_true", help="qwen4_exp: skip the real prefill, start at --ctx with empty caches")
    ap.add_argument("--ngram-first-prime", type=int, default=1_000_000,
                    help="qwen4_exp: per-head vocabulary of the synthetic device table (16 heads; 20,000,000 is the full 95 GiB table)")
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(dev))
    from r4dx_b200.config import lfm2_moe_config, qwen_hybrid_moe_config
    from r4dx_b200.models.batch import BatchModel
    from r4dx_b200.parallel.ep import EpComm, NcclEpBaseline
    from r4dx_b200.quant.weights import moe_kb_rule, synthetic_weight_set
    if a.family == "lfm2":
        if not a.single or world > 1:
            raise SystemExit("--family lfm2 runs with --single on one GPU")
        cfg = lfm2_moe_config(layers=min(a.layers, 40))
    elif a.family == "qwen4_exp":
        if not a.single or world > 1:
            raise SystemExit("--family qwen4_exp runs with --single on one GPU")
        from r4dx_b200.config import qwen4_exp_config
        cfg = qwen4_exp_config(min(a.layers, 48))
    else:
        cfg = qwen_hybrid_moe_config(a.layers)
    e_per = cfg.num_experts // world
    w = synthetic_weight_set(cfg, device=dev, seed=0, kb_rule=moe_kb_rule, expert_range=(rank * e_per, e_per))
    if a.prefill:
        from r4dx_b200.models.hybrid import HybridModel
        from r4dx_b200.ops import kernels as K
        m = HybridModel(cfg, w, max_ctx=a.prefill + 64, device=dev)
        ids = torch.randint(0, cfg.vocab_size, (a.prefill,), dtype=torch.int32)
        m.prefill(ids[:min(a.prefill, 4096)])
        m.reset()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        m.prefill(ids)
        e1.record()
        torch.cuda.synchronize()
        K.check_gemm_status(dev)
        ms = e0.elapsed_time(e1)
        print(json.dumps({"metric": f"prefill tok/s, {a.family} geometry", "tokens": a.prefill, "layers": cfg.num_hidden_layers,
                          "ms": ms, "tok_s": a.prefill / (ms / 1e3)}))
        return
    if a.single and a.family == "qwen4_exp":
        # really prefilled context (1024-row chunks on the tensor cores), then graph decode
        from r4dx_b200.models.q4x import Qwen4ExpModel
        from r4dx_b200.runtime import ngram as NG
        hd = NG.make_header(cfg.vocab_size, cfg.ngram_head_dim, cfg.eos_token_id, seed=0, first_prime_after=a.ngram_first_prime)
        table = NG.NgramTable.synthetic_device(hd, dev)
        m = Qwen4ExpModel(cfg, w, ngram_table=table, max_ctx=a.ctx + a.steps + a.warmup + 64, device=dev)
        ids = torch.randint(0, cfg.vocab_size, (a.ctx,), dtype=torch.int32)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if a.positioned:
            m.pos, tok, pre_ms = a.ctx, 17, float("nan")       # empty caches at the position: for launch lists under a profiler
        else:
            m.prefill(ids)                  # untimed: allocates the chunk workspaces at their final size, loads every kernel
            m.reset()
            torch.cuda.synchronize()
            e0.record()
            tok = m.prefill(ids)
            e1.record()
            torch.cuda.synchronize()
            pre_ms = e0.elapsed_time(e1)
        m.enable_graphs((1,))
        m.decode_begin(tok)
        for _ in range(a.warmup):
            m.decode_step_graph()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            m.decode_step_graph()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
        print(json.dumps({"metric": "batch-1 decode tok/s, qwen4_exp geometry", "ctx": a.ctx, "layers": cfg.num_hidden_layers,
                          "ms_per_step": ms, "tok_s": 1e3 / ms, "prefill_tok_s": a.ctx / (pre_ms / 1e3),
                          "weights_gib": m.weight_bytes() / 2**30, "ngram_table_gib": table.body.numel() * 2 / 2**30,
                          "sparse_rows": bool(a.ctx + 1 > cfg.indexer_budget + cfg.indexer_ratio - 1),
                          "reference_published_tok_s": 57.5 if a.ctx >= 2000 else 50.3, "reference_published_prefill_tok_s": "231-450"}))
        return
    if a.single:
        from r4dx_b200.models.hybrid import HybridModel
        m = HybridModel(cfg, w, max_ctx=a.ctx + a.steps + a.warmup + 64, device=dev)
        m.pos = a.ctx
        m.enable_graphs((1,))
        m.decode_begin(17)
        for _ in range(a.warmup):
            m.decode_step_graph()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            m.decode_step_graph()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
        ref = {"qwen_moe": 50.3, "lfm2": 72.7}[a.family]       # the reference's published trellis numbers (2 GPUs of its kind)
        print(json.dumps({"metric": f"batch-1 decode tok/s, {a.family} geometry", "ctx": a.ctx, "layers": cfg.num_hidden_layers,
                          "ms_per_step": ms, "tok_s": 1e3 / ms, "reference_published_tok_s": ref}))
        return
    B = a.batch // world
    comm = None
    if world > 1:
        comm = (EpComm if a.comm == "fused" else NcclEpBaseline)(world, rank, dev, cfg, max_rows=max(B, 8))
    bm = BatchModel(cfg, w, slots=B, slot_ctx=max(a.ctx, a.real_prefill) + a.steps + a.warmup + 16, device=dev, comm=comm)
    slots = list(range(B))
    g = torch.Generator().manual_seed(rank)
    if a.real_prefill:
        toks = [bm.import_slot(s, torch.randint(0, cfg.vocab_size, (a.real_prefill,), generator=g, dtype=torch.int32)) for s in slots]
    else:
        for s in slots:
            bm.position_slot(s, a.ctx)
        toks = torch.randint(0, cfg.vocab_size, (B,), generator=g).tolist()
    for _ in range(a.warmup):
        toks = bm.decode_batch(slots, toks)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        toks = bm.decode_batch(slots, toks)
    e1.record()
    torch.cuda.synchronize()
    if comm is not None:
        comm.check_healthy()
    worst = max(b.max_rows_of_an_expert() for b in bm.moe.values()) if world == 1 else 0
    t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t[0])
        print(json.dumps({"metric": "batched decode tok/s, hybrid MoE geometry", "batch": a.batch, "world": world, "comm": a.comm,
                          "ctx": a.real_prefill or a.ctx, "slots_prefilled": bool(a.real_prefill), "layers": a.layers, "ms_per_step": ms, "tok_s": a.batch / (ms / 1e3),
                          "max_rows_of_an_expert_last_step": worst}))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
