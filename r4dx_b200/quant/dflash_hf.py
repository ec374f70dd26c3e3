"""Import of a block-diffusion drafter checkpoint in the Hugging Face layout (safetensors + config.json).

Tensor names of the source (``DFlashDraftModel`` / ``DFlash2DraftModel``):

    fc.weight [H, F*H]   hidden_norm.weight   norm.weight
    layers.i.{input_layernorm,post_attention_layernorm}.weight
    layers.i.self_attn.{q,k,v,o}_proj.weight   layers.i.self_attn.{q,k}_norm.weight
    layers.i.mlp.{gate,up,down}_proj.weight
    layers.i.{attention,mlp}_conv.base_kernel [2, 2, H]              (second generation only)
    layers.i.{attention,mlp}_conv.kernel_projection.weight [4*H/16, H]
    candidate_selector.{hidden_projection.weight, predecessor_codebook, successor_codebook}

A first-generation checkpoint has no conv and no selector tensors: it gets identity convs (tap 0 = 1, tap 1 = 0, no
dynamic part) and a zero selector, which make those stages no-ops.  ``dflash_config.target_layer_ids`` are indices into
the source's ``hidden_states``; the residual stream ENTERING layer id + 1 is that tensor, so the stored layers are ids + 1.
The mask row is the target model's embedding of ``mask_token_id`` (the drafter file carries no embedding).

(reference: src/convert/dflash2_hf.hpp, docs/dflash2.md sections 13.1-13.2 and 14.1 for the names and conventions.)
"""
from __future__ import annotations

import json
import os
from typing import Dict, Tuple

import torch

from ..models.dflash import DflashConfig


def _read_dir(d: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors import safe_open
    cfg = json.load(open(os.path.join(d, "config.json")))
    w: Dict[str, torch.Tensor] = {}
    for f in sorted(os.listdir(d)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(d, f), "pt") as sf:
                for k in sf.keys():
                    w[k[6:] if k.startswith("model.") else k] = sf.get_tensor(k)
    return cfg, w


def config_from_hf(hf: dict, n_taps: int) -> DflashConfig:
    dc = hf.get("dflash_config", {})
    ids = dc.get("target_layer_ids", hf.get("target_layer_ids"))
    if not ids or len(ids) != n_taps:
        raise ValueError(f"target_layer_ids {ids} do not match the fc width ({n_taps} taps)")
    heads = hf["num_attention_heads"]
    return DflashConfig(
        layers=hf["num_hidden_layers"], hidden=hf["hidden_size"], heads=heads, kv_heads=hf.get("num_key_value_heads", heads),
        head_dim=hf.get("head_dim", hf["hidden_size"] // heads), intermediate=hf["intermediate_size"],
        window=hf.get("sliding_window") or dc.get("window", 2048), block=dc.get("block_size", hf.get("block_size", 16)),
        rank=dc.get("selector_rank", 256), target_layers=tuple(int(i) + 1 for i in ids),
        mask_token_id=int(dc.get("mask_token_id", hf.get("mask_token_id", 0))), rope_theta=float(hf.get("rope_theta", 1.0e6)),
        eps=float(hf.get("rms_norm_eps", 1e-6)), cands=dc.get("selector_top_k", 16))


def import_dflash_hf(d: str, target_embed: torch.Tensor, vocab: int) -> Tuple[DflashConfig, Dict[str, torch.Tensor]]:
    """(config, fp32 weights under this engine's drafter names) from the checkpoint directory ``d``."""
    hf, t = _read_dir(d)
    H = hf["hidden_size"]
    fc = t["fc.weight"].float()
    if fc.shape[0] != H or fc.shape[1] % H:
        raise ValueError(f"fc.weight {tuple(fc.shape)} is not [hidden, taps * hidden]")
    c = config_from_hf(hf, fc.shape[1] // H)
    G = H // 16
    f = lambda name: t[name].float()
    w: Dict[str, torch.Tensor] = {"fc": fc, "inject_norm": f("hidden_norm.weight"), "out_norm": f("norm.weight"),
                                  "mask_embed": target_embed[c.mask_token_id].float().clone()}
    second_gen = "candidate_selector.hidden_projection.weight" in t
    if second_gen:
        w["selector_hidden"] = f("candidate_selector.hidden_projection.weight")
        w["pred"] = f("candidate_selector.predecessor_codebook").contiguous()
        w["succ"] = f("candidate_selector.successor_codebook").contiguous()
        c.rank = w["selector_hidden"].shape[0]
    else:
        w["selector_hidden"] = torch.zeros(c.rank, H)
        w["pred"] = torch.zeros(vocab, c.rank)
        w["succ"] = torch.zeros(vocab, c.rank)
    for i in range(c.layers):
        s, p = f"layers.{i}.", f"layers.{i}."
        w[p + "in_norm"], w[p + "post_norm"] = f(s + "input_layernorm.weight"), f(s + "post_attention_layernorm.weight")
        w[p + "q_norm"], w[p + "k_norm"] = f(s + "self_attn.q_norm.weight"), f(s + "self_attn.k_norm.weight")
        for ours, theirs in (("wq", "q_proj"), ("wk", "k_proj"), ("wv", "v_proj"), ("wo", "o_proj")):
            w[p + ours] = f(s + f"self_attn.{theirs}.weight")
        w[p + "gate_up"] = torch.cat([f(s + "mlp.gate_proj.weight"), f(s + "mlp.up_proj.weight")], 0)
        w[p + "down"] = f(s + "mlp.down_proj.weight")
        for j0, mod in ((0, "attention_conv"), (2, "mlp_conv")):
            if s + mod + ".base_kernel" in t:
                base = f(s + mod + ".base_kernel")                     # [2 convs, 2 taps, H]
                proj = f(s + mod + ".kernel_projection.weight")        # [2 convs * 2 taps * G, H]
                if base.shape != (2, 2, H) or proj.shape != (4 * G, H):
                    raise ValueError(f"{s}{mod}: unexpected conv tensor shapes {tuple(base.shape)}, {tuple(proj.shape)}")
                for j in range(2):
                    w[p + f"conv{j0 + j}.base"] = base[j].contiguous()
                    w[p + f"conv{j0 + j}.dyn"] = proj[j * 2 * G:(j + 1) * 2 * G].contiguous()
            else:
                for j in range(2):
                    w[p + f"conv{j0 + j}.base"] = torch.cat([torch.ones(1, H), torch.zeros(1, H)], 0)
                    w[p + f"conv{j0 + j}.dyn"] = torch.zeros(2 * G, H)
    shapes = {"wq": (c.heads * c.head_dim, H), "wk": (c.kv_heads * c.head_dim, H), "gate_up": (2 * c.intermediate, H)}
    for n_, sh in shapes.items():
        if tuple(w["layers.0." + n_].shape) != sh:
            raise ValueError(f"layers.0.{n_}: shape {tuple(w['layers.0.' + n_].shape)} does not match the config's {sh}")
    return c, w
