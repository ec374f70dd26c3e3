"""Tensor-parallel sharding of a (quantized) weight set for world 1/2/4/8.

Rules (reference: src/model/tp/tp_shard.h:37-107, generalised beyond world 2):
  column-parallel, per fused segment, contiguous head blocks per rank:
      attn.qg (per-head q|gate rows), attn.k / attn.v (KV heads; replicated when world > KV heads),
      gdn.in_proj_qkv ([q | k | v] segments), gdn.in_proj_z, gdn.in_proj_a/b, gdn.conv1d_weight,
      mlp.gate_up ([gate | up] segments), lm_head (vocab rows)
      conv.in_proj ([B | C | x] segments, the rank's channel block of each), conv.weight,
      moe.experts.E.gate_up of the short-conv MoE family ([gate | up] segments; every rank keeps all experts)
  row-parallel (K split): attn.o, gdn.out_proj, conv.out_proj, mlp.down, moe.experts.E.down (short-conv MoE family)
  replicated: embeddings, norms
Trellis tensors split only at multiples of 128 in either dimension, so a shard is a set of whole
128-row blocks (column-parallel) or a contiguous K range inside every block (row-parallel); the
Hadamard sandwich stays block-local and the per-rank partial outputs of a row-parallel shard
simply add up.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config import ModelConfig
from ..quant.trellis import TrellisWeight
from ..quant.w4a16 import W4Weight


def _ranges_to_index(ranges: List[Tuple[int, int]]) -> torch.Tensor:
    return torch.cat([torch.arange(a, b) for a, b in ranges])


def slice_trellis_rows(tw: TrellisWeight, ranges: List[Tuple[int, int]]) -> TrellisWeight:
    """Keeps output rows in ``ranges`` (each a multiple of 128)."""
    for a, b in ranges:
        if a % 128 or b % 128:
            raise ValueError("trellis row ranges must be multiples of 128")
    per_block = (tw.K // 16) * 8 * 8 * tw.kb
    blocks = tw.words.view(tw.N // 128, per_block)
    bidx = _ranges_to_index([(a // 128, b // 128) for a, b in ranges]).to(tw.words.device)
    ridx = _ranges_to_index(ranges).to(tw.svh.device)
    return TrellisWeight(blocks[bidx].reshape(-1).contiguous(), tw.suh, tw.svh[ridx].contiguous(), int(ridx.numel()), tw.K, tw.kb)


def slice_trellis_cols(tw: TrellisWeight, world: int, rank: int) -> TrellisWeight:
    """Keeps the rank's contiguous K range (row-parallel)."""
    if (tw.K // 128) % world:
        raise ValueError("K/128 not divisible by the tp world")
    ks = tw.K // world
    k0 = rank * ks
    v = tw.words.view(tw.N // 128, tw.K // 16, 8 * 8 * tw.kb)
    return TrellisWeight(v[:, k0 // 16:(k0 + ks) // 16].reshape(-1).contiguous(), tw.suh[k0:k0 + ks].contiguous(), tw.svh,
                         tw.N, ks, tw.kb)


def slice_rows(t, ranges: List[Tuple[int, int]]):
    if isinstance(t, TrellisWeight):
        return slice_trellis_rows(t, ranges)
    idx = _ranges_to_index(ranges)
    if isinstance(t, W4Weight):
        idx = idx.to(t.wq.device)
        return W4Weight(t.wq[idx].contiguous(), t.wsz[idx].contiguous(), int(idx.numel()), t.K, t.group)
    return t[idx.to(t.device)].contiguous()


def slice_cols(t, world: int, rank: int):
    if isinstance(t, TrellisWeight):
        return slice_trellis_cols(t, world, rank)
    if isinstance(t, W4Weight):
        ks = t.K // world
        return W4Weight(t.wq[:, rank * ks // 8:(rank + 1) * ks // 8].contiguous(),
                        t.wsz[:, rank * ks // t.group:(rank + 1) * ks // t.group].contiguous(), t.N, ks, t.group)
    ks = t.shape[1] // world
    return t[:, rank * ks:(rank + 1) * ks].contiguous()


def shard_plan(cfg: ModelConfig, world: int, rank: int) -> Dict[str, tuple]:
    """name suffix -> ("rows", ranges) | ("cols",) | ("rep",) for one layer's tensors."""
    c = cfg
    D = c.head_dim
    hq = c.num_attention_heads // world
    q0 = rank * hq
    if c.num_key_value_heads >= world:
        hkv = c.num_key_value_heads // world
        kv0 = rank * hkv
    else:
        hkv = 1
        kv0 = rank // (world // c.num_key_value_heads)
    Dk, Dv = c.linear_key_head_dim, c.linear_value_head_dim
    hk = c.linear_num_key_heads // world
    hv = c.linear_num_value_heads // world
    kd, vd = c.key_dim, c.value_dim
    qkv = [(rank * hk * Dk, (rank + 1) * hk * Dk), (kd + rank * hk * Dk, kd + (rank + 1) * hk * Dk),
           (2 * kd + rank * hv * Dv, 2 * kd + (rank + 1) * hv * Dv)]
    I = c.intermediate_size
    isz = I // world if I else 0
    qs = (2 if c.attn_output_gate else 1) * D
    plan = {
        "attn.qg": ("rows", [(q0 * qs, (q0 + hq) * qs)]),
        "attn.k": ("rows", [(kv0 * D, (kv0 + hkv) * D)]),
        "attn.v": ("rows", [(kv0 * D, (kv0 + hkv) * D)]),
        "attn.k_descale": ("rows", [(kv0, kv0 + hkv)]),
        "attn.v_descale": ("rows", [(kv0, kv0 + hkv)]),
        "attn.o": ("cols",),
        "gdn.in_proj_qkv": ("rows", qkv),
        "gdn.conv1d_weight": ("rows", qkv),
        "gdn.in_proj_z": ("rows", [(rank * hv * Dv, (rank + 1) * hv * Dv)]),
        "gdn.in_proj_a": ("rows", [(rank * hv, (rank + 1) * hv)]),
        "gdn.in_proj_b": ("rows", [(rank * hv, (rank + 1) * hv)]),
        "gdn.A_log": ("rows", [(rank * hv, (rank + 1) * hv)]),
        "gdn.dt_bias": ("rows", [(rank * hv, (rank + 1) * hv)]),
        "gdn.out_proj": ("cols",),
        "mlp.gate_up": ("rows", [(rank * isz, (rank + 1) * isz), (I + rank * isz, I + (rank + 1) * isz)]),
        "mlp.down": ("cols",),
    }
    if c.has_conv_layers:
        H, hc = c.hidden_size, c.hidden_size // world
        plan["conv.in_proj"] = ("rows", [(s_ * H + rank * hc, s_ * H + (rank + 1) * hc) for s_ in range(3)])
        plan["conv.weight"] = ("rows", [(rank * hc, (rank + 1) * hc)])
        plan["conv.out_proj"] = ("cols",)
        if c.num_experts:
            MI = c.moe_intermediate_size
            mi = MI // world
            plan["moe.expert.gate_up"] = ("rows", [(rank * mi, (rank + 1) * mi), (MI + rank * mi, MI + (rank + 1) * mi)])
            plan["moe.expert.down"] = ("cols",)
    return plan


def shard_weight_set(cfg: ModelConfig, w: Dict[str, object], world: int, rank: int) -> Dict[str, object]:
    """Rank-local weights matching ``cfg.shard(world, rank)`` from the full set."""
    if world == 1:
        return dict(w)
    plan = shard_plan(cfg, world, rank)
    vs = cfg.vocab_size // world
    out: Dict[str, object] = {}
    for name, t in w.items():
        if name == "lm_head":
            out[name] = slice_rows(t, [(rank * vs, (rank + 1) * vs)])
            continue
        rule = None
        if ".moe.experts." in name and "moe.expert.gate_up" in plan:
            rule = plan["moe.expert." + name.rsplit(".", 1)[1]]
        for suffix, r in ([] if rule is not None else plan.items()):
            if name.endswith("." + suffix):
                rule = r
                break
        if rule is None or rule[0] == "rep":
            out[name] = t
        elif rule[0] == "rows":
            out[name] = slice_rows(t, rule[1])
        else:
            out[name] = slice_cols(t, world, rank)
    return out
