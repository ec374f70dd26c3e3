"""Runs a few eager decode steps of a synthetic model for kernel profiling.

    python -m r4dx_b200.utils.profile_step --layers 64 --ctx 8192 --steps 1

The model is positioned at ``--ctx`` without a prefill (the KV cache holds zeros, which costs the
same to read), one untimed step warms every kernel up, then ``--steps`` steps run between
cudaProfilerStart/Stop so that a profiler started with ``--profile-from-start off`` captures
exactly those launches.  Prints the device time of the profiled steps.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--model", default="27b", choices=["27b", "small", "lfm2"])
    ap.add_argument("--tp", type=int, default=1, help="rank 0's shard of this tensor-parallel degree with the no-op communicator: "
                    "the kernels of one rank at its real shapes, nothing exchanged (results are wrong by design)")
    ap.add_argument("--graph", type=int, default=0, help="also time this many CUDA-graph replays of the step")
    ap.add_argument("--chunk", type=int, default=0, help="rows per prefill chunk (0: the model's own choice)")
    ap.add_argument("--prefill", type=int, default=0, help="profile one chunked prefill of this many tokens instead of decode steps")
    a = ap.parse_args()
    from r4dx_b200.config import lfm2_moe_config, qwen_hybrid_27b_config, small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.quant.weights import synthetic_weight_set
    if a.model == "lfm2":
        from r4dx_b200.quant.weights import moe_kb_rule
        cfg = lfm2_moe_config(layers=min(a.layers, 40))
        w = synthetic_weight_set(cfg, device="cuda", seed=0, kb_rule=moe_kb_rule)
    else:
        cfg = qwen_hybrid_27b_config(a.layers) if a.model == "27b" else small_hybrid_config(a.layers)
        comm = None
        if a.tp > 1:
            from r4dx_b200.parallel.tp_emulated import NoopComm
            comm = NoopComm(a.tp, 0, "cuda:0", None)
            cfg = cfg.shard(a.tp, 0)
        w = synthetic_weight_set(cfg, device="cuda", seed=0)
    m = HybridModel(cfg, w, max_ctx=max(a.ctx, a.prefill) + 64 + a.rows * (a.steps + 2 + a.graph),
                    **({"comm": comm} if a.model != "lfm2" and comm is not None else {}))
    if a.prefill:
        ids = torch.randint(0, cfg.vocab_size, (a.prefill,), dtype=torch.int32)
        kw = {"chunk": a.chunk} if a.chunk else {}
        m.prefill(ids[:max(4096, a.chunk)], **kw)          # warm-up (allocates the chunk buffers)
        m.reset()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()
        e0.record()
        m.prefill(ids, **kw)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"prefill of {a.prefill} tokens, {a.layers} layers, tp shard {a.tp}, chunk {a.chunk or 'auto'}: {e0.elapsed_time(e1):.2f} ms")
        return
    m.pos = a.ctx
    ids = torch.randint(0, cfg.vocab_size, (a.rows,), dtype=torch.int32)
    m.feed(ids)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    e0.record()
    for _ in range(a.steps):
        m.feed(ids)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"eager {a.steps} step(s) of {a.rows} row(s): {e0.elapsed_time(e1) / a.steps:.3f} ms/step")
    if a.graph and a.rows == 1:
        m.enable_graphs((1,))
        m.decode_begin(int(ids[0]))
        for _ in range(3):
            m.decode_step_graph()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.graph):
            m.decode_step_graph()
        e1.record()
        torch.cuda.synchronize()
        print(f"graph replay, tp shard {a.tp}: {e0.elapsed_time(e1) / a.graph:.3f} ms/step")


if __name__ == "__main__":
    main()
