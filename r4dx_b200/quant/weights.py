"""Model weight sets: quantizing fp32 weights, synthetic quantized weights, container save/load.

A weight set is a dict name -> TrellisWeight | W4Weight | torch.Tensor.  Body linears use the
trellis layout (mixed 4/5 bit = ~4.5 bpw by default), the LM head w4a16 (group 64), gates /
norms / conv stay bf16 or fp32 -- the same split the reference container uses
(reference: docs/container-format.md:50-83, 599-605).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional, Tuple

import torch

from ..config import ModelConfig
from . import trellis, w4a16
from .container import Container, write_container
from .trellis import TrellisWeight
from .w4a16 import W4Weight, W8Weight

F32_NAMES = ("A_log", "dt_bias", "k_descale", "v_descale", "expert_bias")


def default_kb_rule(name: str) -> int:
    """Mixed 4/5-bit plan (~4.5 bpw): 5 bits on even layers, 4 bits on odd layers."""
    parts = name.split(".")
    if "layers" in parts:
        layer = int(parts[parts.index("layers") + 1])
        return 5 if layer % 2 == 0 else 4
    return 4


def moe_kb_rule(name: str) -> int:
    """Mixed 3/4-bit plan (~3.3 bpw) for the expert-heavy MoE variant: experts mostly 3 bits."""
    parts = name.split(".")
    if ".experts." in name and "layers" in parts:
        layer = int(parts[parts.index("layers") + 1])
        return 4 if layer % 3 == 0 else 3      # one width per layer, so a layer's experts share one launch
    return 4


def is_quantized_linear(name: str) -> bool:
    leaf = name.split(".")[-1]
    if ".hc." in name or name.startswith("text.hc_final."):
        return False                  # the stream gates of the qwen4_exp family stay bf16 (their "down" is not an MLP's)
    return leaf in ("qg", "k", "v", "o", "in_proj_qkv", "in_proj_z", "in_proj", "out_proj", "gate_up", "down", "fc")


def quantize_weight_set(cfg: ModelConfig, w: Dict[str, torch.Tensor], layout: str = "trellis",
                        kb_rule: Callable[[str], int] = default_kb_rule, head_group: int = 64,
                        seed: int = 0, encoder: str = "cpu", hessians: Optional[Dict[str, torch.Tensor]] = None,
                        imatrix: Optional[Dict[str, torch.Tensor]] = None, search: bool = False,
                        group_rule: Optional[Callable[[str], Optional[int]]] = None, w8_group: Optional[int] = None,
                        ldlq_damp: float = 0.01) -> Dict[str, object]:
    """fp32 weights -> quantized set.  layout: trellis | w4a16 | bf16.  ``encoder``: where the Viterbi search of the
    trellis layout runs - "cpu" (threads) or "cuda" (one CTA per tile, ~25x the throughput of 32 host threads); the
    result lives on the CPU either way.  ``hessians``: name -> [K, K] input second moments; linears that have one are
    quantized with error compensation (block LDLQ for the trellis layout, GPTQ for w4a16) on the host.  ``search`` /
    ``imatrix`` (name -> [K] input second moments): the w4a16 layout picks each group's range by a clipping search, weighted
    by the channel importances where given."""
    out: Dict[str, object] = {}
    hessians = hessians or {}
    imatrix = imatrix or {}
    default_group = head_group

    def group_of(name: str) -> int:
        """w4a16 group size of ``name``: the first matching rule of ``group_rule`` (32, 64 or 128), else ``head_group``."""
        g_ = group_rule(name) if group_rule is not None else None
        return int(g_) if g_ else default_group

    for i, (name, t) in enumerate(w.items()):
        leaf = name.split(".")[-1]
        head_group = group_of(name)
        if name == "lm_head":
            out[name] = w4a16.quantize(t, head_group) if layout != "bf16" else t.to(torch.bfloat16)
        elif is_quantized_linear(name) and layout == "trellis" and t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0:
            if name in hessians:
                out[name], _, _ = trellis.quantize_ldlq(t, hessians[name], kb_rule(name), seed=seed * 100003 + i, damp=ldlq_damp)
            elif encoder == "cuda":
                tw, _ = trellis.quantize_cuda(t, kb_rule(name), seed=seed * 100003 + i)
                out[name] = TrellisWeight(tw.words.cpu(), tw.suh.cpu(), tw.svh.cpu(), tw.N, tw.K, tw.kb)
            else:
                out[name], _ = trellis.quantize(t, kb_rule(name), seed=seed * 100003 + i)
        elif is_quantized_linear(name) and layout == "w8a16" and t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0:
            out[name] = w4a16.quantize_w8(t, w8_group or default_group)          # symmetric int8, fp16 group scales, round to nearest
        elif is_quantized_linear(name) and layout == "w4a16":
            if name in hessians:
                from .calibrate import gptq_w4a16
                out[name] = gptq_w4a16(t, hessians[name], head_group)
            elif search or name in imatrix:
                from .calibrate import search_w4a16
                out[name] = search_w4a16(t, imatrix.get(name), head_group)
            else:
                out[name] = w4a16.quantize(t, head_group)
        elif leaf in F32_NAMES or name.startswith("rotation."):
            out[name] = t.float()
        else:
            out[name] = t.to(torch.bfloat16)
    return out


def dequantize_weight_set(q: Dict[str, object]) -> Dict[str, torch.Tensor]:
    """Effective fp32 weights of a quantized set: what the CPU oracle must use to match the GPU."""
    out = {}
    for name, t in q.items():
        if isinstance(t, TrellisWeight):
            out[name] = trellis.reconstruct(t)
        elif isinstance(t, W8Weight):
            out[name] = w4a16.dequantize_w8(W8Weight(t.wq.cpu(), t.ws.cpu(), t.N, t.K, t.group))
        elif isinstance(t, W4Weight):
            out[name] = w4a16.dequantize(t)
        else:
            out[name] = t.float().cpu()
    return out


def linear_shapes(cfg: ModelConfig, with_mtp: bool = False) -> Iterable[Tuple[str, int, int]]:
    """(name, N, K) of every quantizable linear of the (rank-local) config."""
    H = cfg.hidden_size
    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        if cfg.is_attention_layer(i):
            yield p + "attn.qg", cfg.q_proj_dim, H
            yield p + "attn.k", cfg.kv_dim, H
            yield p + "attn.v", cfg.kv_dim, H
            yield p + "attn.o", H, cfg.q_dim
        elif cfg.is_conv_layer(i):
            yield p + "conv.in_proj", 3 * H, H
            yield p + "conv.out_proj", H, H
        else:
            yield p + "gdn.in_proj_qkv", cfg.conv_dim, H
            yield p + "gdn.in_proj_z", cfg.value_dim, H
            yield p + "gdn.out_proj", H, cfg.value_dim
        if not cfg.layer_is_moe(i):
            yield p + "mlp.gate_up", 2 * cfg.intermediate_size, H
            yield p + "mlp.down", H, cfg.intermediate_size
        elif cfg.shared_expert_intermediate_size:
            yield p + "moe.shared.gate_up", 2 * cfg.shared_expert_intermediate_size, H
            yield p + "moe.shared.down", H, cfg.shared_expert_intermediate_size


def synthetic_weight_set(cfg: ModelConfig, device="cuda", seed: int = 0, sigma: float = 0.02,
                         kb_rule: Callable[[str], int] = default_kb_rule, head_group: int = 64,
                         with_mtp: bool = False, expert_range=None) -> Dict[str, object]:
    """Random-init weights created directly in the quantized domain (dense hybrid or MoE hybrid;
    ``expert_range`` = (first, count) of the routed experts this rank holds under expert parallelism).

    Body linears get random trellis code bits (decoded values ~ N(0,1)) with svh = +-sigma, the LM
    head random nibbles; everything else is N(0, sigma).  ``cfg`` may be a TP shard view, in which
    case only this rank's slices are created.
    """
    g = torch.Generator(device=device).manual_seed(seed)

    def n(*shape, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * sigma).to(dtype)

    H = cfg.hidden_size
    w: Dict[str, object] = {"text.embed_tokens": (n(cfg.vocab_size, H).float() * cfg.embed_scale).to(torch.bfloat16)}
    for i, (name, N, K) in enumerate(linear_shapes(cfg)):
        w[name] = trellis.random_weight(N, K, kb_rule(name), seed=seed * 7919 + i, sigma=sigma, device=device)
    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        w[p + "input_layernorm"] = n(H)
        w[p + "post_attention_layernorm"] = n(H)
        if cfg.sandwich_norm:
            w[p + "post_attn_out_norm"] = n(H)
            w[p + "post_mlp_out_norm"] = n(H)
        if cfg.is_attention_layer(i):
            if cfg.qk_norm:
                w[p + "attn.q_norm"] = n(cfg.head_dim)
                w[p + "attn.k_norm"] = n(cfg.head_dim)
            w[p + "attn.k_descale"] = torch.full((cfg.num_key_value_heads,), 1.0 / 16, device=device)
            w[p + "attn.v_descale"] = torch.full((cfg.num_key_value_heads,), 1.0 / 16, device=device)
        elif cfg.is_conv_layer(i):
            w[p + "conv.weight"] = (n(H, cfg.short_conv_taps).float() * (0.5 / sigma)).to(torch.bfloat16)
        else:
            Hv = cfg.linear_num_value_heads
            w[p + "gdn.in_proj_a"] = n(Hv, H)
            w[p + "gdn.in_proj_b"] = n(Hv, H)
            w[p + "gdn.conv1d_weight"] = n(cfg.conv_dim, cfg.linear_conv_kernel_dim)
            w[p + "gdn.A_log"] = n(Hv, dtype=torch.float32)
            w[p + "gdn.dt_bias"] = n(Hv, dtype=torch.float32)
            w[p + "gdn.norm_weight"] = (1.0 + n(cfg.linear_value_head_dim).float()).to(torch.bfloat16)
    w["text.final_norm"] = n(H)
    if cfg.is_qwen4_exp:
        # the stream gates are this family's only norms; they, the indexer and the n-gram layer stay bf16
        # (reference: src/model/qwen4exp_container.h:11-25 lists the tensors)
        for k_ in [k_ for k_ in w if k_.endswith("layernorm") or k_ == "text.final_norm"]:
            del w[k_]
        hc, L, C = cfg.hc_count, cfg.hc_lowrank, cfg.hc_count * H

        def gate(p: str, inject: bool = True):
            w[p + "norm"] = n(C)
            w[p + "down"] = n(L, C)
            w[p + "up"] = (n(C, L).float() * 8).to(torch.bfloat16)
            if inject:
                w[p + "inject"] = n(hc, C)

        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            gate(p + "hc.attn.")
            gate(p + "hc.mlp.")
            if cfg.is_attention_layer(i) and cfg.indexer_heads:
                w[p + "attn.indexer.qk"] = (n((cfg.indexer_heads + 1) * cfg.indexer_dim, H).float() * 4).to(torch.bfloat16)
                w[p + "attn.indexer.q_norm"] = n(cfg.indexer_dim)
                w[p + "attn.indexer.k_norm"] = n(cfg.indexer_dim)
            if i in cfg.ple_layers:
                w[p + "ple.key_proj"] = (n(C, cfg.ple_embed_dim).float() * 10).to(torch.bfloat16)
                w[p + "ple.value_proj"] = (n(H, cfg.ple_embed_dim).float() * 10).to(torch.bfloat16)
                for name in ("norm_key", "norm_query", "norm_conv"):
                    w[p + "ple." + name] = n(C)
                w[p + "ple.conv1d"] = (n(C, cfg.ple_conv_kernel).float() * 10).to(torch.bfloat16)
        gate("text.hc_final.", inject=False)
    w["lm_head"] = w4a16.random_weight(cfg.vocab_shard_size, H, head_group, seed=seed + 17, sigma=sigma, device=device)
    if with_mtp and cfg.mtp_num_hidden_layers:
        # the next-token-prediction head: fc over [embedding | hidden], one gated attention layer, one MLP, its own norm
        p = "mtp."
        inner = cfg.intermediate_size if cfg.intermediate_size else cfg.moe_intermediate_size
        shapes = [("fc", H, 2 * H), ("attn.qg", cfg.q_proj_dim, H), ("attn.k", cfg.kv_dim, H), ("attn.v", cfg.kv_dim, H),
                  ("attn.o", H, cfg.q_dim), ("mlp.gate_up", 2 * inner, H), ("mlp.down", H, inner)]
        for j, (name, N, K) in enumerate(shapes):
            w[p + name] = trellis.random_weight(N, K, kb_rule(p + name), seed=seed * 7919 + 100003 + j, sigma=sigma, device=device)
        for name in ("pre_fc_norm_embedding", "pre_fc_norm_hidden", "input_layernorm", "post_attention_layernorm", "norm"):
            w[p + name] = n(H)
        if cfg.qk_norm:
            w[p + "attn.q_norm"] = n(cfg.head_dim)
            w[p + "attn.k_norm"] = n(cfg.head_dim)
        w[p + "attn.k_descale"] = torch.full((cfg.num_key_value_heads,), 1.0 / 16, device=device)
        w[p + "attn.v_descale"] = torch.full((cfg.num_key_value_heads,), 1.0 / 16, device=device)
    if cfg.is_moe:
        e_begin, e_count = expert_range if expert_range is not None else (0, cfg.num_experts)
        for i in range(cfg.num_dense_layers, cfg.num_hidden_layers):
            p = f"text.layers.{i}.moe."
            w[p + "router"] = n(cfg.num_experts, H)
            if cfg.moe_expert_bias:
                w[p + "expert_bias"] = n(cfg.num_experts, dtype=torch.float32)
            if cfg.shared_expert_intermediate_size:
                w[p + "shared_gate"] = n(1, H)
            kb = kb_rule(p + "experts.0.gate_up")
            for j in range(e_count):
                e = e_begin + j
                w[p + f"experts.{e}.gate_up"] = trellis.random_weight(2 * cfg.moe_intermediate_size, H, kb, seed=seed * 31 + i * 1009 + e,
                                                                     sigma=sigma, device=device)
                w[p + f"experts.{e}.down"] = trellis.random_weight(H, cfg.moe_intermediate_size, kb, seed=seed * 37 + i * 1013 + e,
                                                                  sigma=sigma, device=device)
    return w


# ---- container -------------------------------------------------------------------------------------
def save_weight_set(path: str, cfg: ModelConfig, q: Dict[str, object], extra_meta: Optional[Dict[str, str]] = None) -> None:
    tensors = []
    quant = {}
    for name, t in q.items():
        if isinstance(t, TrellisWeight):
            quant[name] = {"layout": "trellis", "kb": t.kb, "N": t.N, "K": t.K}
            tensors += [(name + ".trellis.words", t.words), (name + ".trellis.suh", t.suh), (name + ".trellis.svh", t.svh)]
        elif isinstance(t, W8Weight):
            quant[name] = {"layout": "w8a16", "group": t.group, "N": t.N, "K": t.K}
            tensors += [(name + ".w8a16.wq", t.wq), (name + ".w8a16.ws", t.ws)]
        elif isinstance(t, W4Weight):
            quant[name] = {"layout": "w4a16", "group": t.group, "N": t.N, "K": t.K}
            tensors += [(name + ".w4a16.wq", t.wq), (name + ".w4a16.wsz", t.wsz)]
        else:
            tensors.append((name, t))
    meta = {"model_config": cfg.to_json(), "quant": json.dumps(quant), "format": "r4dxb-1",
            "arch": cfg.arch}
    meta.update(extra_meta or {})
    write_container(path, tensors, meta)


def load_weight_set(path: str, device="cpu", names: Optional[Callable[[str], bool]] = None) -> Tuple[ModelConfig, Dict[str, object]]:
    ct = Container(path)
    cfg = ct.model_config()
    quant = ct.quant_info()
    out: Dict[str, object] = {}
    on_cpu = str(device) == "cpu"

    class _Get:
        """Copies out of the read-only mapping (the mapping dies with the Container object)."""
        @staticmethod
        def tensor(n):
            t = Container.tensor(ct, n)
            return t.clone() if on_cpu else t.to(device)
    ct_get = _Get()
    for name, qi in quant.items():
        if names and not names(name):
            continue
        if qi["layout"] == "trellis":
            out[name] = TrellisWeight(ct_get.tensor(name + ".trellis.words"), ct_get.tensor(name + ".trellis.suh"),
                                      ct_get.tensor(name + ".trellis.svh"), qi["N"], qi["K"], qi["kb"])
        elif qi["layout"] == "w8a16":
            out[name] = W8Weight(ct_get.tensor(name + ".w8a16.wq"), ct_get.tensor(name + ".w8a16.ws"), qi["N"], qi["K"], qi["group"])
        else:
            out[name] = W4Weight(ct_get.tensor(name + ".w4a16.wq"), ct_get.tensor(name + ".w4a16.wsz"),
                                 qi["N"], qi["K"], qi["group"])
    for name in ct.names:
        if ".trellis." in name or ".w4a16." in name or ".w8a16." in name:
            continue
        if names and not names(name):
            continue
        out[name] = ct_get.tensor(name)
    ct.close()
    return cfg, out


# ---- pre-encoded trellis tensors ---------------------------------------------------------------------------------
def export_trellis_dir(q: Dict[str, object], d: str, rel_err: Optional[Dict[str, float]] = None) -> None:
    """Writes every trellis tensor of ``q`` as <name>.trellis.{words,suh,svh} into ``d``/trellis.safetensors plus a
    manifest (shape, bit width and, when given, the encoder's relative squared error per tensor): the input of
    ``convert --trellis-from``."""
    from safetensors.torch import save_file
    os.makedirs(d, exist_ok=True)
    tensors, manifest = {}, {"format": "r4dxb-trellis-1", "tensors": {}}
    for name, t in q.items():
        if isinstance(t, TrellisWeight):
            tensors[name + ".trellis.words"] = t.words.cpu().contiguous()
            tensors[name + ".trellis.suh"] = t.suh.cpu().contiguous()
            tensors[name + ".trellis.svh"] = t.svh.cpu().contiguous()
            manifest["tensors"][name] = {"N": t.N, "K": t.K, "kb": t.kb}
            if rel_err and name in rel_err:
                manifest["tensors"][name]["rel_err"] = float(rel_err[name])
    save_file(tensors, os.path.join(d, "trellis.safetensors"))
    with open(os.path.join(d, "trellis_manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)


def import_trellis_dir(d: str, w: Dict[str, torch.Tensor], verify: bool = True) -> Tuple[Dict[str, TrellisWeight], Dict[str, float]]:
    """Trellis tensors written by ``export_trellis_dir`` (or any tool that writes the same names in this engine's tile
    order), checked against the fp32 checkpoint ``w``: shape and bit width must fit, and with ``verify`` every tensor is
    reconstructed on the CPU and its relative squared error must stay within the encoder's range for its bit width
    (6 * 4^-kb) and, where the manifest records the encoder's own error, within 2 % + 1e-4 of that record.
    Returns (name -> weight, name -> measured error).  (reference: src/convert/trellis_import.hpp does the same gate for its
    imported tensors: reconstruct from the file's bytes, compare with the recorded error.)"""
    from safetensors import safe_open
    man = json.load(open(os.path.join(d, "trellis_manifest.json")))
    if man.get("format") != "r4dxb-trellis-1":
        raise ValueError(f"unknown trellis manifest format {man.get('format')!r}")
    raw = {}
    for f in sorted(os.listdir(d)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(d, f), "pt") as sf:
                for k in sf.keys():
                    raw[k] = sf.get_tensor(k)
    out, errs = {}, {}
    for name, rec in man["tensors"].items():
        if name not in w:
            raise ValueError(f"{name}: not a tensor of this checkpoint")
        N, K_, kb = int(rec["N"]), int(rec["K"]), int(rec["kb"])
        if tuple(w[name].shape) != (N, K_):
            raise ValueError(f"{name}: manifest shape {(N, K_)} != checkpoint shape {tuple(w[name].shape)}")
        if kb not in (3, 4, 5):
            raise ValueError(f"{name}: bit width {kb} is not 3, 4 or 5")
        try:
            words, suh, svh = raw[name + ".trellis.words"], raw[name + ".trellis.suh"], raw[name + ".trellis.svh"]
        except KeyError as e:
            raise ValueError(f"{name}: missing {e.args[0]}")
        if words.numel() != trellis.packed_words(N, K_, kb) or suh.numel() != K_ or svh.numel() != N:
            raise ValueError(f"{name}: tensor sizes do not match N={N}, K={K_}, kb={kb}")
        tw = TrellisWeight(words.to(torch.int32).contiguous(), suh.to(torch.float16).contiguous(), svh.to(torch.float16).contiguous(), N, K_, kb)
        if verify:
            ref = w[name].float()
            rel = float(((trellis.reconstruct(tw) - ref) ** 2).sum() / (ref ** 2).sum().clamp_min(1e-30))
            errs[name] = rel
            if rel > 6.0 * 4.0 ** (-kb):
                raise ValueError(f"{name}: reconstruction error {rel:.4f} is outside the range of a {kb}-bit encoding of this tensor")
            rec_err = rec.get("rel_err")
            if rec_err is not None and abs(rel - rec_err) > 0.02 * rec_err + 1e-4:
                raise ValueError(f"{name}: reconstruction error {rel:.5f} differs from the recorded {rec_err:.5f}")
        out[name] = tw
    return out, errs
