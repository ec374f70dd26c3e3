"""Hugging Face checkpoint names and layouts -> this engine's weight set.

``config_from_hf`` reads a ``config.json`` (dense hybrid, hybrid MoE, Llama-style, Gemma-style) into a ``ModelConfig``;
``import_hf_weights`` renames and reshapes the tensors:

* gated attention: ``q_proj`` already holds per-head ``[q | gate]`` rows -> ``attn.qg``; ``k/v/o_proj`` -> ``attn.k/v/o``;
* Gated DeltaNet: either separate ``in_proj_qkv / in_proj_z / in_proj_a / in_proj_b`` tensors, or the packed
  ``in_proj_qkvz`` (per key head: q, k, its value heads' v, their z) and ``in_proj_ba`` (per key head: b's then a's),
  which are unpacked into ``[q heads | k heads | v heads]`` rows, z rows, a rows, b rows;
  ``conv1d.weight [C, 1, 4]`` -> ``[C, 4]``;
* MLP: ``gate_proj`` and ``up_proj`` are stacked into ``gate_up`` (gate rows first);
* MoE: ``mlp.gate`` -> ``moe.router``, ``mlp.experts.E.*`` -> ``moe.experts.E.*``, ``mlp.shared_expert*`` -> shared expert;
* norms: the engine stores every RMSNorm weight zero-centred (scale = 1 + w); families whose checkpoints hold the plain
  scale (Llama-style) get ``w - 1``; Gemma-style checkpoints are zero-centred already;
* embeddings: multiplied by the family's embedding scale; a tied head becomes its own (unscaled) ``lm_head`` tensor.

``export_hf_weights`` is the inverse (used by the round-trip test and for handing weights to other tools)
(reference: src/model/container.cpp:92-491 name tables, src/convert/main.cpp import paths).
"""
from __future__ import annotations

import json
import math
from typing import Dict

import torch

from ..config import ModelConfig


def config_from_hf(text: str) -> ModelConfig:
    d = json.loads(text)
    t = d.get("text_config", d)
    mt = (t.get("model_type") or d.get("model_type") or "").lower()
    H, L = t["hidden_size"], t["num_hidden_layers"]
    heads = t["num_attention_heads"]
    common = dict(hidden_size=H, num_hidden_layers=L, num_attention_heads=heads,
                  num_key_value_heads=t.get("num_key_value_heads", heads), head_dim=t.get("head_dim", H // heads),
                  intermediate_size=t.get("intermediate_size", 0), rms_norm_eps=t.get("rms_norm_eps", 1e-6),
                  vocab_size=t["vocab_size"], tie_word_embeddings=bool(t.get("tie_word_embeddings", d.get("tie_word_embeddings", False))),
                  max_position_embeddings=t.get("max_position_embeddings", 262144))
    if "llama" in mt or "nanbeige" in mt or "mistral" in mt:
        cfg = ModelConfig(arch="llama", layer_types=["full_attention"] * L, attn_output_gate=False, qk_norm=False,
                          norm_zero_centered=False, partial_rotary_factor=1.0, rope_theta=t.get("rope_theta", 5.0e5),
                          mtp_num_hidden_layers=0, **common)
    elif "lfm2" in mt:
        types = t.get("layer_types") or ["full_attention" if i % 4 == 2 else "conv" for i in range(L)]
        rope = t.get("rope_parameters") or {}
        cfg = ModelConfig(arch="lfm2_moe", layer_types=list(types), attn_output_gate=False, qk_norm=True, norm_zero_centered=False,
                          partial_rotary_factor=1.0, rope_theta=t.get("rope_theta", rope.get("rope_theta", 1.0e6)),
                          mtp_num_hidden_layers=0, num_experts=t.get("num_experts", 0),
                          num_experts_per_tok=t.get("num_experts_per_tok", 0), moe_intermediate_size=t.get("moe_intermediate_size", 0),
                          shared_expert_intermediate_size=0, norm_topk_prob=bool(t.get("norm_topk_prob", True)),
                          moe_router="sigmoid", moe_expert_bias=bool(t.get("use_expert_bias", True)),
                          routed_scaling_factor=float(t.get("routed_scaling_factor", 1.0)),
                          num_dense_layers=t.get("num_dense_layers", 0), short_conv_taps=t.get("conv_L_cache", 3),
                          **{**common, "rms_norm_eps": t.get("norm_eps", 1e-5), "tie_word_embeddings": True})
    elif mt == "qwen4_exp" or t.get("hc_count", 0):
        # 4-stream gated residual, block-selecting attention, one n-gram layer (reference: src/convert/qwen4exp_layout.cpp:60-108
        # reads these keys; ple_layer_ids is 1-based there)
        rope = t.get("rope_parameters") or {}
        types = t.get("layer_types") or ["full_attention" if (i + 1) % int(t.get("full_attention_interval", 4)) == 0 else "linear_attention"
                                         for i in range(L)]
        cfg = ModelConfig(arch="qwen4_exp", layer_types=list(types), attn_output_gate=True,
                          partial_rotary_factor=t.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25)),
                          rope_theta=t.get("rope_theta", rope.get("rope_theta", 1.0e7)),
                          linear_num_key_heads=t["linear_num_key_heads"], linear_num_value_heads=t["linear_num_value_heads"],
                          linear_key_head_dim=t["linear_key_head_dim"], linear_value_head_dim=t["linear_value_head_dim"],
                          linear_conv_kernel_dim=t.get("linear_conv_kernel_dim", 4), mtp_num_hidden_layers=0,
                          num_experts=t["num_experts"], num_experts_per_tok=t.get("num_experts_per_tok", 10),
                          moe_intermediate_size=t["moe_intermediate_size"],
                          shared_expert_intermediate_size=t.get("shared_expert_intermediate_size", 0),
                          norm_topk_prob=bool(t.get("norm_topk_prob", True)), hc_count=t["hc_count"], hc_lowrank=t["hc_lowrank"],
                          ple_layers=[int(i) - 1 for i in t.get("ple_layer_ids", [])], ple_embed_dim=t.get("ple_embed_dim", 0),
                          ple_conv_kernel=t.get("ple_conv_kernel_size", 4), ple_conv_dilation=t.get("ngram_size", 3),
                          indexer_heads=t.get("indexer_n_heads", t.get("indexer_heads", 4)), indexer_dim=t.get("indexer_head_dim", 128),
                          indexer_ratio=t.get("indexer_compress_ratio", 4), indexer_budget=t.get("indexer_budget", 2048),
                          gdn_gate_act=t.get("output_gate_type", "sigmoid"), final_norm=False,
                          eos_token_id=int(t.get("eos_token_id", d.get("eos_token_id", 248044)) or 248044),
                          **{**common, "tie_word_embeddings": False})
        if t.get("indexer_kv_heads", 1) != 1:
            raise ValueError("qwen4_exp: the indexer is built for one key head")
    elif "gemma" in mt:
        pattern = t.get("sliding_window_pattern", 6)
        cfg = ModelConfig(arch="gemma", layer_types=["full_attention"] * L, attn_output_gate=False, qk_norm=True,
                          partial_rotary_factor=1.0, rope_theta=t.get("rope_theta", 1.0e6), mtp_num_hidden_layers=0,
                          sandwich_norm=True, mlp_act="gelu_tanh", sliding_window=t.get("sliding_window", 1024),
                          sliding_global_every=pattern, rope_local_theta=t.get("rope_local_base_freq", 1.0e4),
                          embed_scale=math.sqrt(H), **{**common, "tie_word_embeddings": True})
    else:
        interval = int(t.get("full_attention_interval", 4))
        types = t.get("layer_types") or ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(L)]
        rope = t.get("rope_parameters") or {}
        cfg = ModelConfig(arch="qwen_hybrid_moe" if t.get("num_experts", 0) else "qwen_hybrid", layer_types=list(types),
                          attn_output_gate=bool(t.get("attn_output_gate", True)),
                          partial_rotary_factor=t.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25)),
                          rope_theta=t.get("rope_theta", rope.get("rope_theta", 1.0e7)),
                          linear_num_key_heads=t.get("linear_num_key_heads", 0), linear_num_value_heads=t.get("linear_num_value_heads", 0),
                          linear_key_head_dim=t.get("linear_key_head_dim", 0), linear_value_head_dim=t.get("linear_value_head_dim", 0),
                          linear_conv_kernel_dim=t.get("linear_conv_kernel_dim", 4),
                          mtp_num_hidden_layers=t.get("mtp_num_hidden_layers", 0), num_experts=t.get("num_experts", 0),
                          num_experts_per_tok=t.get("num_experts_per_tok", 0), moe_intermediate_size=t.get("moe_intermediate_size", 0),
                          shared_expert_intermediate_size=t.get("shared_expert_intermediate_size", 0),
                          norm_topk_prob=bool(t.get("norm_topk_prob", True)), **common)
    cfg.validate()
    return cfg


def _unpack_qkvz(cfg: ModelConfig, qkvz: torch.Tensor, ba: torch.Tensor):
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    g = Hv // Hk
    K = qkvz.shape[1]
    per = 2 * Dk + 2 * g * Dv
    x = qkvz.view(Hk, per, K)
    q, k = x[:, :Dk], x[:, Dk:2 * Dk]
    v, z = x[:, 2 * Dk:2 * Dk + g * Dv], x[:, 2 * Dk + g * Dv:]
    qkv = torch.cat([q.reshape(Hk * Dk, K), k.reshape(Hk * Dk, K), v.reshape(Hv * Dv, K)], 0)
    y = ba.view(Hk, 2 * g, K)
    b, a = y[:, :g].reshape(Hv, K), y[:, g:].reshape(Hv, K)
    return qkv.contiguous(), z.reshape(Hv * Dv, K).contiguous(), a.contiguous(), b.contiguous()


def _pack_qkvz(cfg: ModelConfig, qkv: torch.Tensor, z: torch.Tensor, a: torch.Tensor, b: torch.Tensor):
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    g = Hv // Hk
    K = qkv.shape[1]
    q = qkv[:Hk * Dk].view(Hk, Dk, K)
    k = qkv[Hk * Dk:2 * Hk * Dk].view(Hk, Dk, K)
    v = qkv[2 * Hk * Dk:].view(Hk, g * Dv, K)
    zz = z.view(Hk, g * Dv, K)
    qkvz = torch.cat([q, k, v, zz], 1).reshape(-1, K)
    ba = torch.cat([b.view(Hk, g, K), a.view(Hk, g, K)], 1).reshape(-1, K)
    return qkvz.contiguous(), ba.contiguous()


def _norm_in(cfg: ModelConfig, w: torch.Tensor) -> torch.Tensor:
    return w.float() if cfg.norm_zero_centered else w.float() - 1.0


def _norm_out(cfg: ModelConfig, w: torch.Tensor) -> torch.Tensor:
    return w.float() if cfg.norm_zero_centered else w.float() + 1.0


def _layer_norm_names(cfg: ModelConfig):
    """(internal name, HF name) of the per-layer RMSNorms."""
    if cfg.sandwich_norm:       # HF Gemma: post_attention_layernorm is the norm of the attention OUTPUT
        return [("input_layernorm", "input_layernorm"), ("post_attn_out_norm", "post_attention_layernorm"),
                ("post_attention_layernorm", "pre_feedforward_layernorm"), ("post_mlp_out_norm", "post_feedforward_layernorm")]
    return [("input_layernorm", "input_layernorm"), ("post_attention_layernorm", "post_attention_layernorm")]


def import_hf_weights(cfg: ModelConfig, hf: Dict[str, torch.Tensor], prefix: str = "model.") -> Dict[str, torch.Tensor]:
    """HF-named tensors -> the engine's fp32 weight set (what ``quantize_weight_set`` and the CPU oracle take)."""
    def get(name: str) -> torch.Tensor:
        for pre in (prefix, "model.language_model.", "language_model.model.", ""):
            if pre + name in hf:
                return hf[pre + name].float()
        raise KeyError(f"checkpoint has no tensor {prefix}{name}")

    def has(name: str) -> bool:
        return any(pre + name in hf for pre in (prefix, "model.language_model.", "language_model.model.", ""))

    def gate_up(base: str) -> torch.Tensor:
        return torch.cat([get(base + "gate_proj.weight"), get(base + "up_proj.weight")], 0).contiguous()

    if cfg.arch == "lfm2_moe":
        return _import_lfm2(cfg, get, has)
    if cfg.is_qwen4_exp:
        return _import_qwen4_exp(cfg, get, has, hf)
    out: Dict[str, torch.Tensor] = {}
    emb = get("embed_tokens.weight")
    out["text.embed_tokens"] = emb * cfg.embed_scale
    out["text.final_norm"] = _norm_in(cfg, get("norm.weight"))
    out["lm_head"] = hf["lm_head.weight"].float() if "lm_head.weight" in hf else emb.clone()
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", f"layers.{i}."
        for mine, theirs in _layer_norm_names(cfg):
            out[p + mine] = _norm_in(cfg, get(s + theirs + ".weight"))
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            out[p + "attn.qg"] = get(a + "q_proj.weight")
            out[p + "attn.k"], out[p + "attn.v"], out[p + "attn.o"] = get(a + "k_proj.weight"), get(a + "v_proj.weight"), get(a + "o_proj.weight")
            if cfg.qk_norm:
                out[p + "attn.q_norm"] = _norm_in(cfg, get(a + "q_norm.weight"))
                out[p + "attn.k_norm"] = _norm_in(cfg, get(a + "k_norm.weight"))
            out[p + "attn.k_descale"] = torch.ones(cfg.num_key_value_heads)
            out[p + "attn.v_descale"] = torch.ones(cfg.num_key_value_heads)
        else:
            g = s + "linear_attn."
            if has(g + "in_proj_qkvz.weight"):
                qkv, z, a_, b_ = _unpack_qkvz(cfg, get(g + "in_proj_qkvz.weight"), get(g + "in_proj_ba.weight"))
            else:
                qkv, z = get(g + "in_proj_qkv.weight"), get(g + "in_proj_z.weight")
                a_, b_ = get(g + "in_proj_a.weight"), get(g + "in_proj_b.weight")
            out[p + "gdn.in_proj_qkv"], out[p + "gdn.in_proj_z"], out[p + "gdn.in_proj_a"], out[p + "gdn.in_proj_b"] = qkv, z, a_, b_
            out[p + "gdn.conv1d_weight"] = get(g + "conv1d.weight").reshape(cfg.conv_dim, -1)
            out[p + "gdn.A_log"], out[p + "gdn.dt_bias"] = get(g + "A_log"), get(g + "dt_bias")
            out[p + "gdn.norm_weight"] = get(g + "norm.weight")           # the gated norm's weight is a plain scale
            out[p + "gdn.out_proj"] = get(g + "out_proj.weight")
        m = s + "mlp."
        if cfg.is_moe:
            out[p + "moe.router"] = get(m + "gate.weight")
            if cfg.shared_expert_intermediate_size:
                out[p + "moe.shared_gate"] = get(m + "shared_expert_gate.weight").reshape(1, -1)
                out[p + "moe.shared.gate_up"], out[p + "moe.shared.down"] = gate_up(m + "shared_expert."), get(m + "shared_expert.down_proj.weight")
            for e in range(cfg.num_experts):
                out[p + f"moe.experts.{e}.gate_up"] = gate_up(m + f"experts.{e}.")
                out[p + f"moe.experts.{e}.down"] = get(m + f"experts.{e}.down_proj.weight")
        else:
            out[p + "mlp.gate_up"], out[p + "mlp.down"] = gate_up(m), get(m + "down_proj.weight")
    return out


_Q4X_GATE = (("norm", "hc_norm.weight"), ("down", "input_mix_weight_down.weight"), ("up", "input_mix_weight_up.weight"),
             ("inject", "block_inject_weight.weight"))
_Q4X_PLE = ("key_proj", "value_proj", "norm_key", "norm_query", "norm_conv")


def _import_qwen4_exp(cfg: ModelConfig, get, has, hf) -> Dict[str, torch.Tensor]:
    """qwen4_exp checkpoint names -> container names (reference: src/convert/qwen4exp_layout.cpp:140-228 is the same
    table).  Norm weights keep the checkpoint's zero-centred convention; the n-gram table itself (``*.ple.ple_embedding.*``)
    is not part of the weight set: it becomes the table file (``runtime/ngram.py``)."""
    out: Dict[str, torch.Tensor] = {"text.embed_tokens": get("embed_tokens.weight")}
    if "lm_head.weight" not in hf:
        raise KeyError("qwen4_exp checkpoint without lm_head.weight (the head is not tied in this family)")
    out["lm_head"] = hf["lm_head.weight"].float()
    for mine, theirs in _Q4X_GATE[:3]:
        out["text.hc_final." + mine] = get("hyper_connection_mixer." + theirs)
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", f"layers.{i}."
        for blk in ("attn", "mlp"):
            for mine, theirs in _Q4X_GATE:
                out[p + f"hc.{blk}.{mine}"] = get(s + f"{blk}_hyper_connection.{theirs}")
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            out[p + "attn.qg"], out[p + "attn.o"] = get(a + "q_proj.weight"), get(a + "o_proj.weight")
            out[p + "attn.k"], out[p + "attn.v"] = get(a + "k_proj.weight"), get(a + "v_proj.weight")
            out[p + "attn.q_norm"], out[p + "attn.k_norm"] = get(a + "q_norm.weight"), get(a + "k_norm.weight")
            out[p + "attn.k_descale"] = torch.ones(cfg.num_key_value_heads)
            out[p + "attn.v_descale"] = torch.ones(cfg.num_key_value_heads)
            out[p + "attn.indexer.qk"] = get(a + "indexer.index_qk_proj.weight")
            out[p + "attn.indexer.q_norm"] = get(a + "indexer.q_layernorm.weight")
            out[p + "attn.indexer.k_norm"] = get(a + "indexer.k_layernorm.weight")
        else:
            g = s + "linear_attn."
            for name in ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "out_proj"):
                out[p + "gdn." + name] = get(g + name + ".weight")
            out[p + "gdn.conv1d_weight"] = get(g + "conv1d.weight").reshape(cfg.conv_dim, -1)
            out[p + "gdn.A_log"], out[p + "gdn.dt_bias"] = get(g + "A_log"), get(g + "dt_bias")
            out[p + "gdn.norm_weight"] = get(g + "norm.weight")
        if i in cfg.ple_layers:
            for name in _Q4X_PLE:
                out[p + "ple." + name] = get(s + f"ple.{name}.weight")
            out[p + "ple.conv1d"] = get(s + "ple.conv1d.weight").reshape(cfg.hc_count * cfg.hidden_size, -1)
        m = s + "mlp."
        out[p + "moe.router"] = get(m + "gate.weight")
        out[p + "moe.shared_gate"] = get(m + "shared_expert_gate.weight").reshape(1, -1)
        gu = lambda b: torch.cat([get(b + "gate_proj.weight"), get(b + "up_proj.weight")], 0).contiguous()
        out[p + "moe.shared.gate_up"], out[p + "moe.shared.down"] = gu(m + "shared_expert."), get(m + "shared_expert.down_proj.weight")
        for e in range(cfg.num_experts):
            out[p + f"moe.experts.{e}.gate_up"] = gu(m + f"experts.{e}.")
            out[p + f"moe.experts.{e}.down"] = get(m + f"experts.{e}.down_proj.weight")
    return out


def export_qwen4_exp(cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str = "model.language_model.") -> Dict[str, torch.Tensor]:
    """Container names -> the checkpoint's names (round-trip tests and synthetic checkpoints)."""
    H, I = cfg.hidden_size, cfg.moe_intermediate_size
    out: Dict[str, torch.Tensor] = {prefix + "embed_tokens.weight": w["text.embed_tokens"], "lm_head.weight": w["lm_head"]}
    for mine, theirs in _Q4X_GATE[:3]:
        out[prefix + "hyper_connection_mixer." + theirs] = w["text.hc_final." + mine]
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", prefix + f"layers.{i}."
        for blk in ("attn", "mlp"):
            for mine, theirs in _Q4X_GATE:
                out[s + f"{blk}_hyper_connection.{theirs}"] = w[p + f"hc.{blk}.{mine}"]
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            for mine, theirs in (("qg", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "o_proj"), ("q_norm", "q_norm"), ("k_norm", "k_norm")):
                out[a + theirs + ".weight"] = w[p + "attn." + mine]
            out[a + "indexer.index_qk_proj.weight"] = w[p + "attn.indexer.qk"]
            out[a + "indexer.q_layernorm.weight"], out[a + "indexer.k_layernorm.weight"] = w[p + "attn.indexer.q_norm"], w[p + "attn.indexer.k_norm"]
        else:
            g = s + "linear_attn."
            for name in ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "out_proj"):
                out[g + name + ".weight"] = w[p + "gdn." + name]
            out[g + "conv1d.weight"] = w[p + "gdn.conv1d_weight"].reshape(cfg.conv_dim, 1, -1)
            out[g + "A_log"], out[g + "dt_bias"], out[g + "norm.weight"] = w[p + "gdn.A_log"], w[p + "gdn.dt_bias"], w[p + "gdn.norm_weight"]
        if i in cfg.ple_layers:
            for name in _Q4X_PLE:
                out[s + f"ple.{name}.weight"] = w[p + "ple." + name]
            out[s + "ple.conv1d.weight"] = w[p + "ple.conv1d"].reshape(cfg.hc_count * H, 1, -1)
        m = s + "mlp."
        out[m + "gate.weight"], out[m + "shared_expert_gate.weight"] = w[p + "moe.router"], w[p + "moe.shared_gate"]
        S = cfg.shared_expert_intermediate_size

        def split(base: str, gu: torch.Tensor, down: torch.Tensor, inner: int):
            out[base + "gate_proj.weight"], out[base + "up_proj.weight"], out[base + "down_proj.weight"] = gu[:inner], gu[inner:], down
        split(m + "shared_expert.", w[p + "moe.shared.gate_up"], w[p + "moe.shared.down"], S)
        for e in range(cfg.num_experts):
            split(m + f"experts.{e}.", w[p + f"moe.experts.{e}.gate_up"], w[p + f"moe.experts.{e}.down"], I)
    return out


def _import_lfm2(cfg: ModelConfig, get, has) -> Dict[str, torch.Tensor]:
    """Short-conv + attention MoE checkpoints: ``operator_norm`` / ``ffn_norm`` per layer, ``embedding_norm`` at the end, conv
    mixers ``conv.{in_proj,conv,out_proj}``, dense ``feed_forward.{w1 gate, w3 up, w2 down}``, experts either stacked 3-D
    (``experts.gate_up_proj`` [E, 2I, H], ``experts.down_proj`` [E, H, I]) or one module per expert; the head is tied
    (reference: docs/lfm2-plan.md:44-57)."""
    out: Dict[str, torch.Tensor] = {}
    emb = get("embed_tokens.weight")
    out["text.embed_tokens"] = emb
    out["text.final_norm"] = _norm_in(cfg, get("embedding_norm.weight"))
    out["lm_head"] = get("lm_head.weight") if has("lm_head.weight") else emb.clone()
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", f"layers.{i}."
        out[p + "input_layernorm"] = _norm_in(cfg, get(s + "operator_norm.weight"))
        out[p + "post_attention_layernorm"] = _norm_in(cfg, get(s + "ffn_norm.weight"))
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            out[p + "attn.qg"], out[p + "attn.k"] = get(a + "q_proj.weight"), get(a + "k_proj.weight")
            out[p + "attn.v"], out[p + "attn.o"] = get(a + "v_proj.weight"), get(a + "out_proj.weight")
            out[p + "attn.q_norm"] = _norm_in(cfg, get(a + "q_layernorm.weight"))
            out[p + "attn.k_norm"] = _norm_in(cfg, get(a + "k_layernorm.weight"))
            out[p + "attn.k_descale"] = torch.ones(cfg.num_key_value_heads)
            out[p + "attn.v_descale"] = torch.ones(cfg.num_key_value_heads)
        else:
            c = s + "conv."
            out[p + "conv.in_proj"], out[p + "conv.out_proj"] = get(c + "in_proj.weight"), get(c + "out_proj.weight")
            out[p + "conv.weight"] = get(c + "conv.weight").reshape(cfg.hidden_size, -1)
        f = s + "feed_forward."
        if not cfg.layer_is_moe(i):
            out[p + "mlp.gate_up"] = torch.cat([get(f + "w1.weight"), get(f + "w3.weight")], 0).contiguous()
            out[p + "mlp.down"] = get(f + "w2.weight")
            continue
        out[p + "moe.router"] = get(f + "gate.weight")
        if cfg.moe_expert_bias:
            out[p + "moe.expert_bias"] = get(f + "expert_bias")
        stacked = has(f + "experts.gate_up_proj")
        gu, dn = (get(f + "experts.gate_up_proj"), get(f + "experts.down_proj")) if stacked else (None, None)
        for e in range(cfg.num_experts):
            if stacked:
                out[p + f"moe.experts.{e}.gate_up"], out[p + f"moe.experts.{e}.down"] = gu[e].contiguous(), dn[e].contiguous()
            else:
                x = f + f"experts.{e}."
                out[p + f"moe.experts.{e}.gate_up"] = torch.cat([get(x + "w1.weight"), get(x + "w3.weight")], 0).contiguous()
                out[p + f"moe.experts.{e}.down"] = get(x + "w2.weight")
    return out


def _export_lfm2(cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    hf: Dict[str, torch.Tensor] = {prefix + "embed_tokens.weight": w["text.embed_tokens"].float(),
                                   prefix + "embedding_norm.weight": _norm_out(cfg, w["text.final_norm"])}
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", prefix + f"layers.{i}."
        hf[s + "operator_norm.weight"] = _norm_out(cfg, w[p + "input_layernorm"])
        hf[s + "ffn_norm.weight"] = _norm_out(cfg, w[p + "post_attention_layernorm"])
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            for mine, theirs in (("qg", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "out_proj")):
                hf[a + theirs + ".weight"] = w[p + "attn." + mine].float()
            hf[a + "q_layernorm.weight"] = _norm_out(cfg, w[p + "attn.q_norm"])
            hf[a + "k_layernorm.weight"] = _norm_out(cfg, w[p + "attn.k_norm"])
        else:
            c = s + "conv."
            hf[c + "in_proj.weight"], hf[c + "out_proj.weight"] = w[p + "conv.in_proj"].float(), w[p + "conv.out_proj"].float()
            hf[c + "conv.weight"] = w[p + "conv.weight"].float().reshape(cfg.hidden_size, 1, -1)
        f = s + "feed_forward."
        if not cfg.layer_is_moe(i):
            gu = w[p + "mlp.gate_up"].float()
            hf[f + "w1.weight"], hf[f + "w3.weight"] = gu[:gu.shape[0] // 2].contiguous(), gu[gu.shape[0] // 2:].contiguous()
            hf[f + "w2.weight"] = w[p + "mlp.down"].float()
            continue
        hf[f + "gate.weight"] = w[p + "moe.router"].float()
        if cfg.moe_expert_bias:
            hf[f + "expert_bias"] = w[p + "moe.expert_bias"].float()
        hf[f + "experts.gate_up_proj"] = torch.stack([w[p + f"moe.experts.{e}.gate_up"].float() for e in range(cfg.num_experts)])
        hf[f + "experts.down_proj"] = torch.stack([w[p + f"moe.experts.{e}.down"].float() for e in range(cfg.num_experts)])
    return hf


def export_hf_weights(cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str = "model.", packed_gdn: bool = True) -> Dict[str, torch.Tensor]:
    """The inverse of ``import_hf_weights`` (mtp.* tensors are not part of the HF layout and are dropped)."""
    if cfg.arch == "lfm2_moe":
        return _export_lfm2(cfg, w, prefix)
    hf: Dict[str, torch.Tensor] = {}
    hf[prefix + "embed_tokens.weight"] = w["text.embed_tokens"].float() / cfg.embed_scale
    hf[prefix + "norm.weight"] = _norm_out(cfg, w["text.final_norm"])
    if not cfg.tie_word_embeddings:
        hf["lm_head.weight"] = w["lm_head"].float()
    for i in range(cfg.num_hidden_layers):
        p, s = f"text.layers.{i}.", prefix + f"layers.{i}."
        for mine, theirs in _layer_norm_names(cfg):
            hf[s + theirs + ".weight"] = _norm_out(cfg, w[p + mine])
        if cfg.is_attention_layer(i):
            a = s + "self_attn."
            hf[a + "q_proj.weight"], hf[a + "k_proj.weight"] = w[p + "attn.qg"].float(), w[p + "attn.k"].float()
            hf[a + "v_proj.weight"], hf[a + "o_proj.weight"] = w[p + "attn.v"].float(), w[p + "attn.o"].float()
            if cfg.qk_norm:
                hf[a + "q_norm.weight"], hf[a + "k_norm.weight"] = _norm_out(cfg, w[p + "attn.q_norm"]), _norm_out(cfg, w[p + "attn.k_norm"])
        else:
            g = s + "linear_attn."
            if packed_gdn:
                hf[g + "in_proj_qkvz.weight"], hf[g + "in_proj_ba.weight"] = _pack_qkvz(
                    cfg, w[p + "gdn.in_proj_qkv"].float(), w[p + "gdn.in_proj_z"].float(), w[p + "gdn.in_proj_a"].float(), w[p + "gdn.in_proj_b"].float())
            else:
                for n in ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b"):
                    hf[g + n + ".weight"] = w[p + "gdn." + n].float()
            hf[g + "conv1d.weight"] = w[p + "gdn.conv1d_weight"].float().reshape(cfg.conv_dim, 1, -1)
            hf[g + "A_log"], hf[g + "dt_bias"] = w[p + "gdn.A_log"].float(), w[p + "gdn.dt_bias"].float()
            hf[g + "norm.weight"], hf[g + "out_proj.weight"] = w[p + "gdn.norm_weight"].float(), w[p + "gdn.out_proj"].float()
        m = s + "mlp."

        def split(name: str, base: str):
            gu = w[p + name + ".gate_up"].float()
            hf[base + "gate_proj.weight"], hf[base + "up_proj.weight"] = gu[:gu.shape[0] // 2].contiguous(), gu[gu.shape[0] // 2:].contiguous()
            hf[base + "down_proj.weight"] = w[p + name + ".down"].float()

        if cfg.is_moe:
            hf[m + "gate.weight"] = w[p + "moe.router"].float()
            if cfg.shared_expert_intermediate_size:
                hf[m + "shared_expert_gate.weight"] = w[p + "moe.shared_gate"].float()
                split("moe.shared", m + "shared_expert.")
            for e in range(cfg.num_experts):
                split(f"moe.experts.{e}", m + f"experts.{e}.")
        else:
            split("mlp", m)
    return hf


# ---- vision tower -------------------------------------------------------------------------------------------------
_VISION_RENAMES = (("attn.qkv.", "qkv."), ("attn.proj.", "proj."), ("mlp.linear_fc1.", "fc1."), ("mlp.linear_fc2.", "fc2."),
                   ("mlp.fc1.", "fc1."), ("mlp.fc2.", "fc2."), ("merger.linear_fc1.", "merger.fc1."), ("merger.linear_fc2.", "merger.fc2."),
                   ("merger.ln_q.", "merger.norm."), ("patch_embed.proj.", "patch_embed."), ("pos_embed.weight", "pos_embed"))


def import_hf_vision(raw: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The vision tower's tensors of a Hugging Face checkpoint under this engine's names (without the ``vision.``
    prefix the container adds): ``[model.]visual.*`` -> patch_embed / pos_embed / blocks.i.{norm1,qkv,proj,norm2,fc1,fc2} /
    merger.{norm,fc1,fc2}.  The patch embedding's convolution kernel [hidden, C, t, p, p] becomes a [hidden, C*t*p*p]
    matrix (patches are flattened in the same order by the preprocessor).
    (reference: src/convert/ keeps the tower in bf16 with --vision on; docs/vision.md lists the tensors.)"""
    out: Dict[str, torch.Tensor] = {}
    for k, v in raw.items():
        for pre in ("model.visual.", "visual.", "model.vision_tower.", "vision_tower."):
            if k.startswith(pre):
                name = k[len(pre):]
                break
        else:
            continue
        for a, b in _VISION_RENAMES:
            name = name.replace(a, b)
        if name == "patch_embed.weight" and v.dim() > 2:
            v = v.reshape(v.shape[0], -1)
        out[name] = v
    return out
