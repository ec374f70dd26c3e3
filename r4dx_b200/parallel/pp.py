"""Pipeline-parallel prefill over NCCL point-to-point, and the reshard into the tensor-parallel decode layout.

Two stages: stage A (rank 0) owns the embedding and layers [0, split), stage B (rank 1) owns layers
[split, N) and the head.  Chunk c+1 runs on A while chunk c runs on B; the hand-off is the residual stream
of the chunk (one [T, hidden] bf16 tensor) sent with ``isend`` / ``irecv`` into double buffers, so the copy
overlaps the next chunk's compute.  Each stage keeps the KV cache / GDN state of its own layers (the
reference moves the same carry, plus KV blocks, through pinned host slots:
reference src/model/pp_model.cpp:441-513, pp_channel.h:52-110).

After the prompt, ``reshard_to_tp`` hands every tensor-parallel rank its head slice of every layer's state,
derived from the same shard rules as the weights (reference: src/model/reshard_plan.h:1-18), so decode can
continue tensor-parallel ("hybrid" mode: PP prefill, TP decode).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..models.hybrid import KV_BLOCK, MAX_ROWS, HybridModel
from .shard import shard_plan

BF = torch.bfloat16


def default_split(cfg: ModelConfig) -> int:
    """Stage A gets slightly fewer layers than half: stage B also runs the head."""
    n = cfg.num_hidden_layers
    return max(1, (n * 29) // 64) if n >= 8 else n // 2


def layer_bytes(cfg: ModelConfig, weights) -> List[int]:
    """Device bytes of every layer's tensors in a weight set (quantized layouts count their packed bytes)."""
    out = [0] * cfg.num_hidden_layers
    for name, t in weights.items():
        if name.startswith("text.layers."):
            i = int(name.split(".")[2])
            if i < len(out):
                out[i] += t.nbytes if not isinstance(t, torch.Tensor) else t.numel() * t.element_size()
    return out


def choose_split_by_bytes(per_layer: List[int], first_stage_extra: int = 0, last_stage_extra: int = 0, cap: int = 0) -> int:
    """The layer boundary k (stage A = layers [0, k), stage B = the rest) that balances the two stages' weight bytes; stage A
    also carries ``first_stage_extra`` (embedding table), stage B ``last_stage_extra`` (head).  With ``cap`` > 0 a split
    whose larger stage exceeds it is refused (the model does not fit two devices of that size).
    (reference: src/model/qwen4exp_container.h:5-9 places its two stages by the same rule.)"""
    n = len(per_layer)
    if n < 2:
        raise ValueError("a two-stage split needs at least two layers")
    total = sum(per_layer)
    best_k, best_gap, run = 1, None, 0
    for k in range(1, n):
        run += per_layer[k - 1]
        a, b = run + first_stage_extra, total - run + last_stage_extra
        gap = abs(a - b)
        if best_gap is None or gap < best_gap:
            best_k, best_gap = k, gap
    a = sum(per_layer[:best_k]) + first_stage_extra
    b = total - sum(per_layer[:best_k]) + last_stage_extra
    if cap and max(a, b) > cap:
        raise ValueError(f"no two-stage split fits {cap} bytes per device: the best one needs {max(a, b)}")
    return best_k


class PipelinePrefill:
    def __init__(self, stage: HybridModel, rank: int, split: int, chunk: int = 1024, group=None):
        self.stage, self.rank, self.split, self.chunk, self.group = stage, rank, split, chunk, group
        H = stage.cfg.hidden_size
        self.bufs = [torch.empty(chunk, H, dtype=BF, device=stage.device) for _ in range(2)]
        self.stats = {"chunks": 0, "bytes": 0}

    def prefill(self, ids: torch.Tensor) -> int:
        """Both ranks call this with the same ids; returns the greedy next token (known on both)."""
        st, n = self.stage, ids.numel()
        ids = ids.to(torch.int32)
        cb = st._chunk_buffers(min(self.chunk, max(n, MAX_ROWS + 1)))
        C = cb["C"]
        chunks = [(s, min(n, s + C)) for s in range(0, n, C)]
        pending: List = [None, None]
        tok = torch.zeros(1, dtype=torch.int32, device=st.device)
        for c, (s, e) in enumerate(chunks):
            T = e - s
            buf = self.bufs[c % 2]
            cb["positions"][:T].copy_(torch.arange(st.pos, st.pos + T, dtype=torch.int32, device=st.device))
            if self.rank == 0:
                if pending[c % 2] is not None:
                    pending[c % 2].wait()                      # the buffer's previous send has left
                cb["ids"][:T].copy_(ids[s:e].to(st.device), non_blocking=True)
                st.forward_chunk(T, want_logits=False)
                buf[:T].copy_(cb["x"][:T])
                pending[c % 2] = dist.isend(buf[:T], dst=1, group=self.group)
            else:
                dist.recv(buf[:T], src=0, group=self.group)
                cb["x"][:T].copy_(buf[:T])
                st.forward_chunk(T, want_logits=(e == n), skip_embed=True)
            self.stats["chunks"] += 1
            self.stats["bytes"] += T * buf.shape[1] * 2
        for p in pending:
            if p is not None:
                p.wait()
        if self.rank == 1:
            tok.copy_(st.buf.next_ids[:1])
        dist.broadcast(tok, src=1, group=self.group)
        return int(tok.item())


class LayerSplitDecode:
    """Static two-stage layer split for decode (models whose weights do not fit one GPU): stage A runs its layers on
    the new rows and hands the residual rows to stage B, which finishes the stack, runs the head and tells both ranks
    the token.  The stages keep the KV cache / recurrent state of their own layers, exactly as the pipelined prefill
    left them, so ``PipelinePrefill.prefill`` followed by ``step`` needs no state movement
    (reference: src/model/qwen4exp_stage.cpp, qwen35moe_stage.cpp run their two big MoE models this way, with the
    residual bounced through host memory; here it is one NCCL send over NVLink)."""

    def __init__(self, stage: HybridModel, rank: int, group=None):
        self.stage, self.rank, self.group = stage, rank, group
        self.tok = torch.zeros(1, dtype=torch.int32, device=stage.device)

    def step(self, token: int) -> int:
        st = self.stage
        b = st.buf
        T = st._stage(torch.tensor([token], dtype=torch.int32), st.pos)
        b.n_replay.fill_(st.pending_rows)
        if self.rank == 0:
            st.forward_rows(T, want_logits=False)
            dist.send(b.x[:T], dst=1, group=self.group)
        else:
            dist.recv(b.x[:T], src=0, group=self.group)
            st.forward_rows(T, want_logits=True, skip_embed=True)
            self.tok.copy_(b.next_ids[:1])
        st.pending_rows = T
        st.pos += T
        dist.broadcast(self.tok, src=1, group=self.group)
        return int(self.tok.item())


def _channel_ranges(gcfg: ModelConfig, world: int, rank: int) -> List[Tuple[int, int]]:
    return shard_plan(gcfg, world, rank)["gdn.conv1d_weight"][1]


def reshard_to_tp(gcfg: ModelConfig, stage: HybridModel, tp_model: HybridModel, world: int, rank: int, stage_ranks: Dict[int, int],
                  group=None) -> None:
    """Moves full-head per-layer state from the stage that produced it into every rank's head-sliced decode model.

    ``stage_ranks``: layer -> rank holding that layer's full state.  World must equal the number of ranks in the
    group; every rank calls this.  Copies are plain NCCL send/recv of the slices (local slices are copied)."""
    pos = stage.pos
    stage.commit_pending() if stage.pending_rows else None
    plan_of = {r: shard_plan(gcfg, world, r) for r in range(world)}
    used_blocks = (pos + KV_BLOCK - 1) // KV_BLOCK
    for layer in range(gcfg.num_hidden_layers):
        owner = stage_ranks[layer]
        for dst in range(world):
            pl = plan_of[dst]
            if gcfg.is_attention_layer(layer):
                (a, b), = pl["attn.k"][1]
                h0, h1 = a // gcfg.head_dim, b // gcfg.head_dim
                pieces = [lambda m: m.kv[layer][:used_blocks, h0:h1]] if False else None
                if rank == owner:
                    src = stage.kv[layer][:used_blocks, h0:h1].contiguous()
                    if dst == rank:
                        tp_model.kv[layer][:used_blocks].copy_(src)
                    else:
                        dist.send(src, dst=dst, group=group)
                elif rank == dst:
                    tmp = torch.empty_like(tp_model.kv[layer][:used_blocks])
                    dist.recv(tmp, src=owner, group=group)
                    tp_model.kv[layer][:used_blocks].copy_(tmp)
            else:
                (v0, v1), = pl["gdn.in_proj_a"][1]
                ch = torch.cat([torch.arange(a, b) for a, b in pl["gdn.conv1d_weight"][1]])
                if rank == owner:
                    s_state = stage.gdn_state[layer][v0:v1].contiguous()
                    s_ring = stage.ring[layer][:, ch.to(stage.device)].contiguous()
                    if dst == rank:
                        tp_model.gdn_state[layer].copy_(s_state)
                        tp_model.ring[layer].copy_(s_ring)
                    else:
                        dist.send(s_state, dst=dst, group=group)
                        dist.send(s_ring, dst=dst, group=group)
                elif rank == dst:
                    t1 = torch.empty_like(tp_model.gdn_state[layer])
                    t2 = torch.empty_like(tp_model.ring[layer])
                    dist.recv(t1, src=owner, group=group)
                    dist.recv(t2, src=owner, group=group)
                    tp_model.gdn_state[layer].copy_(t1)
                    tp_model.ring[layer].copy_(t2)
    tp_model.pos = pos
    tp_model.pending_rows = 0
    tp_model.buf.n_replay.zero_()
