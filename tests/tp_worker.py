"""Child of tests/test_tp_gpu.py: one rank of a tensor-parallel run of a small hybrid model.

Every rank builds the same full synthetic weight set and keeps its shard.  The SAME shard then runs under both
communicators of one process group - library collectives between kernels (NcclComm) and collectives inside the compute
kernels (FusedComm) - and the full logits rows are compared: last row of a prefill, an 8-row speculative window, a chunked
prefill that really takes several chunks, 12 greedy decode steps under teacher forcing.  Rank 0 also runs the unsharded
model as the outer reference."""
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# Fused vs library path on identical shards, whole model: the two differ in where partial sums are rounded to bf16 (the
# fused epilogue adds fp32 partials and rounds once, the library path rounds every partial, reduces, and rounds the add
# again), and eight such points in a 4-layer stack move a logit by up to a few bf16 steps.  The per-operation checks
# below are the tight ones: there the only difference left is one rounding, and the bound is a count of bf16 steps.
TOL_PATHS = float(os.environ.get("R4DXB_TP_TOL", "0.03"))
# sharded vs unsharded model: different split of every sum
TOL_REF = 0.05


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from r4dx_b200.config import small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_comm import NcclComm
    from r4dx_b200.parallel.tp_fused import FusedComm
    from r4dx_b200.quant.weights import synthetic_weight_set
    gcfg = dataclasses.replace(small_hybrid_config(layers=4), linear_num_key_heads=8, linear_num_value_heads=16)
    full = synthetic_weight_set(gcfg, device=dev, seed=3, sigma=0.05)
    cfg = gcfg.shard(world, rank)
    shard = shard_weight_set(gcfg, full, world, rank)
    fused = FusedComm(world, rank, dev, n=gcfg.hidden_size)
    fused.self_test()
    m_f = HybridModel(cfg, shard, max_ctx=640, device=dev, comm=fused)
    m_n = HybridModel(cfg, shard, max_ctx=640, device=dev, comm=NcclComm(world, rank, dev))
    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(0, gcfg.vocab_size, (90,), generator=gen, dtype=torch.int32)
    ids3 = torch.randint(0, gcfg.vocab_size, (450,), generator=gen, dtype=torch.int32)
    worst = {}

    def full_rows(m, rows):
        """Logits rows of this rank's vocabulary shard -> the full rows on every rank."""
        mine = m.buf.logits[rows].float().contiguous()
        parts = torch.empty(world, *mine.shape, device=dev)
        dist.all_gather_into_tensor(parts, mine)
        return parts.permute(1, 0, 2).reshape(mine.shape[0], -1)[:, :gcfg.vocab_size]

    def compare(what, a, b, tol):
        scale = max(a.abs().max().item(), 1e-6)
        d = (a - b).abs().max().item() / scale
        worst[what] = max(worst.get(what, 0.0), d)
        assert d <= tol, (what, d, tol)

    # -- per-operation checks ------------------------------------------------------------------------------------------
    from r4dx_b200.ops import kernels as K
    BF = torch.bfloat16
    g2 = torch.Generator().manual_seed(100 + rank)
    # (a) the push all-reduce of bare rows against an fp32 library all-reduce of the same inputs: one rounding apart
    rows = torch.randn(5, gcfg.hidden_size, generator=g2).to(BF).to(dev)
    want = rows.float()
    dist.all_reduce(want)
    got = rows.clone()
    fused.all_reduce_rows(got)
    torch.cuda.synchronize()
    step = 2.0 ** -8 * want.abs().clamp_min(1e-3)                    # one bf16 step at each element's magnitude
    assert bool(((got.float() - want).abs() <= step).all()), "push all-reduce is more than one bf16 step from the fp32 sum"
    every = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(every, got)
    assert all(torch.equal(e, every[0]) for e in every), "ranks hold different bits after the push all-reduce"
    # (b) the fused row-parallel product (+ residual) against the fp32 sum of every rank's own product
    lin = m_f.lin["text.layers.0.mlp.down"]
    xin = (torch.randn(3, 2 * cfg.intermediate_size, generator=torch.Generator().manual_seed(5)) * 0.5).to(BF).to(dev)
    res0 = torch.randn(3, gcfg.hidden_size, generator=torch.Generator().manual_seed(6)).to(BF).to(dev)
    part = torch.empty(3, gcfg.hidden_size, dtype=BF, device=dev)
    lin(xin, out=part, prologue=K.PRO_SILU_MUL)
    want = part.float()
    dist.all_reduce(want)
    want = want + res0.float()
    got = res0.clone()
    fused.row_parallel_linear(lin, xin, got, prologue=K.PRO_SILU_MUL)
    torch.cuda.synchronize()
    fused.check_healthy()
    # every rank's reference partial was rounded to bf16 once (half a step each), the fused result once at the end
    bound = (0.5 * world + 1.0) * 2.0 ** -8 * torch.maximum(want.abs(), part.float().abs().max() * torch.ones_like(want))
    assert bool(((got.float() - want).abs() <= bound).all()), ("fused product", ((got.float() - want).abs() / bound).max().item())
    # (c) the vocabulary merge: the global best value with the lowest id among equals
    ids_t = torch.tensor([rank * 100 + 7, 5, 1000 - rank], dtype=torch.int32, device=dev)
    vals_t = torch.tensor([1.0 + rank, 2.0, 3.0], dtype=torch.float32, device=dev)
    fused.merge_argmax(ids_t, vals_t)
    torch.cuda.synchronize()
    assert ids_t.tolist() == [(world - 1) * 100 + 7, 5, 1000 - (world - 1)] and vals_t.tolist() == [float(world), 2.0, 3.0], (ids_t, vals_t)

    # 0. the fused collectives inside a captured graph: greedy generation with graph replay, tokens equal on every rank
    toks_graph = m_f.generate_greedy(ids, 6, use_graph=True)
    m_f.reset()
    # 1. one-chunk prefill, last row
    t_f, t_n = m_f.prefill(ids), m_n.prefill(ids)
    assert toks_graph[0] == t_f
    row_f, row_n = full_rows(m_f, [m_f.last_row]), full_rows(m_n, [m_n.last_row])
    compare("prefill", row_f, row_n, TOL_PATHS)
    # 2. 12 decode steps on both, teacher-forced with the fused model's tokens
    toks = [t_f]
    for j in range(12):
        m_n.feed(torch.tensor([toks[-1]], dtype=torch.int32))
        m_f.feed(torch.tensor([toks[-1]], dtype=torch.int32))
        compare("decode", full_rows(m_f, [0]), full_rows(m_n, [0]), TOL_PATHS)
        toks.append(int(m_f.buf.next_ids[0].item()))
    # 3. an 8-row window on top
    win = torch.tensor(toks[-8:], dtype=torch.int32)
    m_f.feed(win); m_n.feed(win)
    compare("window", full_rows(m_f, list(range(8))), full_rows(m_n, list(range(8))), TOL_PATHS)
    fused.check_healthy()
    # 4. chunked prefill: 450 tokens in 64-row chunks (8 chunks, two rounds through the double-buffered receive halves and
    #    a short tail), then in 384-row chunks whose token tiles span several owners
    for chunk in (64, 384):
        m_f.reset(); m_n.reset()
        calls0 = getattr(fused, "pf_calls", 0)
        a, b = m_f.prefill(ids3, chunk=chunk), m_n.prefill(ids3, chunk=chunk)
        compare(f"prefill chunk {chunk}", full_rows(m_f, [m_f.last_row]), full_rows(m_n, [m_n.last_row]), TOL_PATHS)
        fused.check_healthy()
        layers_rp = 2 * gcfg.num_hidden_layers                      # row-parallel products per chunk
        want_chunks = (450 + chunk - 1) // chunk - (1 if 450 % chunk and 450 % chunk <= 8 else 0)
        if fused.pf_calls < calls0:          # larger chunk buffers were allocated: the counter started again
            calls0 = 0
        assert fused.pf_calls - calls0 == want_chunks * layers_rp, (fused.pf_calls - calls0, want_chunks, layers_rp)
    # 5. recovery leaves a working communicator: zero everything, self-test, and the same prefill again
    fused.recover()
    m_f.reset()
    again = m_f.prefill(ids3, chunk=384)
    compare("after recover", full_rows(m_f, [m_f.last_row]), full_rows(m_n, [m_n.last_row]), TOL_PATHS)
    # every rank must hold the same tokens
    gathered = [None] * world
    dist.all_gather_object(gathered, (toks, toks_graph, a, again))
    assert all(g == gathered[0] for g in gathered), f"ranks disagree: {gathered}"
    # the sharded model against the unsharded one (every rank takes part in the gathers)
    m_f.reset()
    m_f.prefill(ids3, chunk=384)
    row3 = full_rows(m_f, [m_f.last_row])
    if rank == 0:
        ref = HybridModel(gcfg, full, max_ctx=640, device=dev)
        ref.prefill(ids)
        ref_row = ref.buf.logits[[ref.last_row]].float()
        compare("vs unsharded prefill", ref_row, row_f, TOL_REF)
        d_f = (ref_row - row_f).abs().max().item()
        d_n = (ref_row - row_n).abs().max().item()
        # the fused path must not sit farther from the unsharded model than the library path does (plus slack for noise)
        assert d_f <= 1.5 * d_n + 0.005 * ref_row.abs().max().item(), ("fused farther from the unsharded model than nccl", d_f, d_n)
        ref.reset()
        ref.prefill(ids3, chunk=384)
        compare("vs unsharded long prefill", ref.buf.logits[[ref.last_row]].float(), row3, TOL_REF)
        print("worst relative logit differences:", {k: round(v, 5) for k, v in worst.items()}, flush=True)
        print(fused.stats.line())
        print(f"TP_OK world={world}", flush=True)
    # leave without tearing NCCL down: communicators referenced by captured graphs can stall the teardown
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
