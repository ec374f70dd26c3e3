"""Tensor parallelism at 2, 4 and 8 ranks on ONE GPU: the ranks are threads of this process, every collective is a
host-side rendezvous (no kernel waits for another kernel).  Checks the sharding of every tensor - KV-head replication at
8 ranks included - and the per-rank call sequence against the unsharded model."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu


def _near_best(lg: torch.Tensor, tok: int, tol: float, what: str) -> None:
    lg = lg.float()
    gap = lg.max().item() - lg[tok].item()
    assert gap <= tol * lg.abs().max().item(), (what, tok, int(lg.argmax()), gap)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_match_the_unsharded_model(world):
    from r4dx_b200.config import small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_emulated import EmulatedWorld
    from r4dx_b200.quant.weights import synthetic_weight_set
    dev = "cuda:0"
    gcfg = dataclasses.replace(small_hybrid_config(layers=4), linear_num_key_heads=8, linear_num_value_heads=16)
    full = synthetic_weight_set(gcfg, device=dev, seed=3, sigma=0.05)
    ids = torch.randint(0, gcfg.vocab_size, (90,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    ref = HybridModel(gcfg, full, max_ctx=512, device=dev)
    ref_first = ref.prefill(ids)
    ref_logits = ref.buf.logits[getattr(ref, "last_row", 0)].float().clone()

    def rank_body(rank, comm):
        cfg = gcfg.shard(world, rank)
        m = HybridModel(cfg, shard_weight_set(gcfg, full, world, rank), max_ctx=512, device=dev, comm=comm)
        m.overlap_siblings = False                       # everything on the one shared stream
        toks = m.generate_greedy(ids, 8, use_graph=False)
        shard_logits = None
        m.reset()
        first = m.prefill(ids)
        shard_logits = m.buf.logits[getattr(m, "last_row", 0)].float().clone()
        return toks, first, shard_logits, comm.stats.all_reduces

    got = EmulatedWorld(world, dev).run(rank_body)
    toks = got[0][0]
    assert all(g[0] == toks for g in got), "ranks disagree on the tokens"
    assert all(g[3] > 0 for g in got)
    # the concatenated vocabulary shards are the unsharded logits row, up to the rounding of the split sums
    row = torch.cat([g[2] for g in got])[:gcfg.vocab_size]
    scale = ref_logits.abs().max().item()
    assert (row - ref_logits).abs().max().item() <= 0.05 * scale
    _near_best(ref_logits, got[0][1], 0.04, "prefill")
    _near_best(ref_logits, toks[0], 0.04, "first token")
    # teacher forcing: every token the sharded ranks picked is (nearly) the unsharded model's best
    for j in range(1, len(toks)):
        lg = ref.decode_step_logits(toks[j - 1]).view(-1)
        _near_best(lg, toks[j], 0.04, f"decode {j}")


def test_lockstep_check_stops_ranks_that_feed_different_tokens():
    """The race detector: with the fingerprint exchange on, a rank that stages a different token is caught on the host before
    the ranks meet in a collective; with equal calls nothing fires."""
    from r4dx_b200.config import small_hybrid_config
    from r4dx_b200.models.hybrid import HybridModel
    from r4dx_b200.parallel.shard import shard_weight_set
    from r4dx_b200.parallel.tp_comm import TpDivergenceError
    from r4dx_b200.parallel.tp_emulated import EmulatedWorld
    from r4dx_b200.quant.weights import synthetic_weight_set
    dev, world = "cuda:0", 2
    gcfg = dataclasses.replace(small_hybrid_config(layers=2), linear_num_key_heads=8, linear_num_value_heads=16)
    full = synthetic_weight_set(gcfg, device=dev, seed=3, sigma=0.05)

    def body(bad):
        def rank_body(rank, comm):
            m = HybridModel(gcfg.shard(world, rank), shard_weight_set(gcfg, full, world, rank), max_ctx=64, device=dev, comm=comm)
            m.overlap_siblings = False
            m.lockstep_checks = True
            m.feed(torch.tensor([5, 6, 7], dtype=torch.int32))
            m.feed(torch.tensor([9 if (bad and rank == 1) else 8], dtype=torch.int32))
            return m.pos
        return EmulatedWorld(world, dev).run(rank_body)

    assert body(False) == [4, 4]
    with pytest.raises(TpDivergenceError):
        body(True)
