"""fp32 CPU reference model of the Qwen-style hybrid decoder (dense and MoE variants).

This is the numerics oracle for the GPU engine and the timed CPU baseline.  It keeps explicit
per-sequence state (KV rows per attention layer, recurrent + conv state per Gated DeltaNet layer)
so that prefill-then-decode can be compared against a single full forward.

Layer math (reference: docs/architecture.md:29-137):
  x += mixer(rmsnorm(x));  x += mlp(rmsnorm(x));  logits = lm_head(rmsnorm(x))
with the zero-centred ``(1 + w)`` RMSNorm, per-head-interleaved q|gate rows in ``attn.qg``,
partial NeoX rope, sigmoid output gate, and the gated delta rule with causal conv1d + SiLU,
L2-normalised q/k and a gated RMSNorm on the output.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig
from ..ops import reference as R


def linear_names(cfg: ModelConfig) -> List[str]:
    """Names of every quantizable linear (weights stored [out, in])."""
    names = []
    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        if cfg.is_attention_layer(i):
            names += [p + "attn.qg", p + "attn.k", p + "attn.v", p + "attn.o"]
        elif cfg.is_conv_layer(i):
            names += [p + "conv.in_proj", p + "conv.out_proj"]
        else:
            names += [p + "gdn.in_proj_qkv", p + "gdn.in_proj_z", p + "gdn.out_proj"]
        if cfg.layer_is_moe(i):
            if cfg.shared_expert_intermediate_size:
                names += [p + "moe.shared.gate_up", p + "moe.shared.down"]
            for e in range(cfg.num_experts):
                names += [p + f"moe.experts.{e}.gate_up", p + f"moe.experts.{e}.down"]
        else:
            names += [p + "mlp.gate_up", p + "mlp.down"]
    names.append("lm_head")
    return names


def init_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, with_mtp: bool = False) -> Dict[str, torch.Tensor]:
    """Random-init weights, every tensor N(0, std) from one seeded generator, fp32."""
    g = torch.Generator().manual_seed(seed)

    def n(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    H = cfg.hidden_size
    # (the stored table already carries the family's embedding scale; a tied head keeps its own unscaled copy)
    w: Dict[str, torch.Tensor] = {"text.embed_tokens": n(cfg.vocab_size, H) * cfg.embed_scale}

    def attn_block(p: str):
        w[p + "attn.qg"] = n(cfg.q_proj_dim, H)
        w[p + "attn.k"] = n(cfg.kv_dim, H)
        w[p + "attn.v"] = n(cfg.kv_dim, H)
        w[p + "attn.o"] = n(H, cfg.q_dim)
        if cfg.qk_norm:
            w[p + "attn.q_norm"] = n(cfg.head_dim)
            w[p + "attn.k_norm"] = n(cfg.head_dim)
        w[p + "attn.k_descale"] = torch.ones(cfg.num_key_value_heads)
        w[p + "attn.v_descale"] = torch.ones(cfg.num_key_value_heads)

    def mlp_block(p: str, inter: int, name: str = "mlp"):
        w[p + f"{name}.gate_up"] = n(2 * inter, H)
        w[p + f"{name}.down"] = n(H, inter)

    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        w[p + "input_layernorm"] = n(H)
        w[p + "post_attention_layernorm"] = n(H)
        if cfg.sandwich_norm:
            w[p + "post_attn_out_norm"] = n(H)
            w[p + "post_mlp_out_norm"] = n(H)
        if cfg.is_attention_layer(i):
            attn_block(p)
        elif cfg.is_conv_layer(i):
            w[p + "conv.in_proj"] = n(3 * H, H)
            w[p + "conv.weight"] = n(H, cfg.short_conv_taps) * (0.5 / std)
            w[p + "conv.out_proj"] = n(H, H)
        else:
            w[p + "gdn.in_proj_qkv"] = n(cfg.conv_dim, H)
            w[p + "gdn.in_proj_z"] = n(cfg.value_dim, H)
            w[p + "gdn.in_proj_a"] = n(cfg.linear_num_value_heads, H)
            w[p + "gdn.in_proj_b"] = n(cfg.linear_num_value_heads, H)
            w[p + "gdn.conv1d_weight"] = n(cfg.conv_dim, cfg.linear_conv_kernel_dim)
            w[p + "gdn.A_log"] = n(cfg.linear_num_value_heads)
            w[p + "gdn.dt_bias"] = n(cfg.linear_num_value_heads)
            w[p + "gdn.norm_weight"] = 1.0 + n(cfg.linear_value_head_dim)
            w[p + "gdn.out_proj"] = n(H, cfg.value_dim)
        if cfg.layer_is_moe(i):
            w[p + "moe.router"] = n(cfg.num_experts, H)
            if cfg.moe_expert_bias:
                w[p + "moe.expert_bias"] = n(cfg.num_experts)
            if cfg.shared_expert_intermediate_size:
                w[p + "moe.shared_gate"] = n(1, H)
                mlp_block(p, cfg.shared_expert_intermediate_size, "moe.shared")
            for e in range(cfg.num_experts):
                mlp_block(p, cfg.moe_intermediate_size, f"moe.experts.{e}")
        else:
            mlp_block(p, cfg.intermediate_size)
    w["text.final_norm"] = n(H)
    w["lm_head"] = n(cfg.vocab_size, H)
    if with_mtp and cfg.mtp_num_hidden_layers:
        p = "mtp."
        w[p + "fc"] = n(H, 2 * H)
        w[p + "pre_fc_norm_embedding"] = n(H)
        w[p + "pre_fc_norm_hidden"] = n(H)
        w[p + "input_layernorm"] = n(H)
        w[p + "post_attention_layernorm"] = n(H)
        attn_block(p)
        mlp_block(p, cfg.intermediate_size if cfg.intermediate_size else cfg.moe_intermediate_size)
        w[p + "norm"] = n(H)
    return w


@dataclass
class OracleState:
    pos: int = 0
    k: Dict[int, torch.Tensor] = field(default_factory=dict)      # layer -> [S, Hkv, D]
    v: Dict[int, torch.Tensor] = field(default_factory=dict)
    gdn: Dict[int, torch.Tensor] = field(default_factory=dict)    # layer -> [H, V, K]
    conv: Dict[int, torch.Tensor] = field(default_factory=dict)   # layer -> [W-1, C]

    def clone(self) -> "OracleState":
        c = OracleState(self.pos)
        for name in ("k", "v", "gdn", "conv"):
            setattr(c, name, {i: t.clone() for i, t in getattr(self, name).items()})
        return c


class OracleModel:
    """fp32 forward over explicit state. ``fp8_kv=True`` rounds K/V through e4m3 like the cache."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], fp8_kv: bool = False,
                 chunked_gdn: bool = False, act_dtype: Optional[torch.dtype] = None):
        cfg.validate()
        self.cfg = cfg
        self.w = {k: v.float() for k, v in weights.items()}
        self.fp8_kv = fp8_kv
        self.chunked_gdn = chunked_gdn
        self.act_dtype = act_dtype     # when set (bf16) activations are rounded at the points the GPU path rounds them

    def _r(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.act_dtype is None else x.to(self.act_dtype).float()

    # calibration taps: ``on_linear(name, input_rows)`` sees the input of every quantizable linear; ``on_kv(layer, k, v)``
    # sees the keys (after norm and rope) and values an attention layer is about to cache
    on_linear = None
    on_kv = None

    def _mm(self, x: torch.Tensor, name: str) -> torch.Tensor:
        if self.on_linear is not None:
            self.on_linear(name, x)
        return x @ self.w[name].T

    # ---- blocks ------------------------------------------------------------------------
    # absolute [start, end) image blocks of the current call: rows inside one see their whole block on sliding-window layers
    image_blocks = None

    def attention(self, p: str, li, x: torch.Tensor, st: OracleState, store: bool = True) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        T = x.shape[0]
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        qg = self._r(self._mm(x, p + "attn.qg")).view(T, Hq, cfg.q_proj_dim // Hq)
        q, gate = qg[..., :D], (qg[..., D:] if cfg.attn_output_gate else None)
        k = self._r(self._mm(x, p + "attn.k")).view(T, Hkv, D)
        v = self._r(self._mm(x, p + "attn.v")).view(T, Hkv, D)
        if cfg.qk_norm:
            q = R.rmsnorm_1pw(q, w[p + "attn.q_norm"], cfg.rms_norm_eps)
            k = R.rmsnorm_1pw(k, w[p + "attn.k_norm"], cfg.rms_norm_eps)
        pos = torch.arange(st.pos, st.pos + T)
        theta = cfg.layer_theta(li) if isinstance(li, int) else cfg.rope_theta
        window = cfg.layer_window(li) if isinstance(li, int) else 0
        q = self._r(R.rope_partial_neox(q, pos, cfg.rotary_dim, theta))
        k = R.rope_partial_neox(k, pos, cfg.rotary_dim, theta)
        if self.on_kv is not None:
            self.on_kv(li, k, v)
        if self.fp8_kv:
            k = R.fp8_e4m3_roundtrip(k, w[p + "attn.k_descale"][None, :, None])
            v = R.fp8_e4m3_roundtrip(v, w[p + "attn.v_descale"][None, :, None])
        K = torch.cat([st.k[li], k], 0) if li in st.k else k
        V = torch.cat([st.v[li], v], 0) if li in st.v else v
        if store:
            st.k[li], st.v[li] = K, V
        limit = None
        if self.image_blocks and window > 0:
            from .gemma_vision import key_limit_ext
            limit = key_limit_ext(st.pos, T, self.image_blocks)
        o = R.causal_gqa_attention(q, K, V, st.pos, window, limit)
        o = self._r(o * torch.sigmoid(gate)) if gate is not None else self._r(o)
        return self._r(self._mm(o.reshape(T, Hq * D), p + "attn.o"))

    def gdn(self, p: str, li, x: torch.Tensor, st: OracleState) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        T = x.shape[0]
        Hk, H = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        Kd, Vd = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        mixed = self._r(self._mm(x, p + "gdn.in_proj_qkv"))
        z = self._r(self._mm(x, p + "gdn.in_proj_z")).view(T, H, Vd)
        a = x @ w[p + "gdn.in_proj_a"].T
        b = x @ w[p + "gdn.in_proj_b"].T
        mixed, st.conv[li] = R.causal_conv1d_silu(mixed, w[p + "gdn.conv1d_weight"], st.conv.get(li))
        q = R.l2norm(mixed[:, :cfg.key_dim].view(T, Hk, Kd))
        k = R.l2norm(mixed[:, cfg.key_dim:2 * cfg.key_dim].view(T, Hk, Kd))
        v = mixed[:, 2 * cfg.key_dim:].view(T, H, Vd)
        g, beta = R.gdn_gates(a, b, w[p + "gdn.A_log"], w[p + "gdn.dt_bias"])
        fn = R.gdn_chunked if (self.chunked_gdn and T > 1) else R.gdn_recurrent
        o, st.gdn[li] = fn(q, k, v, g, beta, st.gdn.get(li))
        o = self._r(R.gated_rmsnorm(o, z, w[p + "gdn.norm_weight"], cfg.rms_norm_eps))
        return self._r(self._mm(o.reshape(T, H * Vd), p + "gdn.out_proj"))

    def short_conv(self, p: str, li, x: torch.Tensor, st: OracleState) -> torch.Tensor:
        """Gated short-convolution mixer: in_proj -> B | C | x, y = C * fir(B * x), out_proj
        (reference: src/kernels/include/r4dx/kernels/lfm2_kernels.h:14-34)."""
        w = self.w
        bcx = self._r(self._mm(x, p + "conv.in_proj"))
        wt = w[p + "conv.weight"]
        if self.act_dtype is not None:
            wt = wt.to(self.act_dtype).float()
        y, st.conv[li] = R.short_conv(bcx, wt, st.conv.get(li), round_bf16=self.act_dtype is not None)
        return self._r(self._mm(self._r(y), p + "conv.out_proj"))

    def mlp(self, p: str, x: torch.Tensor, name: str = "mlp") -> torch.Tensor:
        w = self.w
        act = R.gelu_mul if self.cfg.mlp_act == "gelu_tanh" else R.silu_mul
        h = self._r(act(self._r(self._mm(x, p + f"{name}.gate_up"))))
        return self._r(self._mm(h, p + f"{name}.down"))

    def moe(self, p: str, x: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        logits = self._r(x @ w[p + "moe.router"].T)
        if cfg.moe_router == "sigmoid":
            ids, wts = R.moe_route_sigmoid(logits, w.get(p + "moe.expert_bias"), cfg.num_experts_per_tok, cfg.norm_topk_prob,
                                           cfg.routed_scaling_factor)
        else:
            ids, wts = R.moe_route(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            # combine in ascending expert id, fp32 accumulate (deterministic order)
            order = torch.argsort(ids[t])
            acc = torch.zeros(x.shape[1])
            for j in order.tolist():
                e = int(ids[t, j])
                acc = acc + wts[t, j] * self.mlp(p, x[t:t + 1], f"moe.experts.{e}")[0]
            out[t] = acc
        if cfg.shared_expert_intermediate_size:
            sg = torch.sigmoid(x @ w[p + "moe.shared_gate"].T)
            out = out + sg * self.mlp(p, x, "moe.shared")
        return self._r(out)

    # ---- model -------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, st: Optional[OracleState] = None, return_hidden: bool = False,
                capture_layers: Optional[List[int]] = None, embed_overrides=None, image_blocks=None):
        """Feeds ``ids`` (1-D) at positions st.pos.. and returns logits [T, vocab] (fp32).  ``embed_overrides`` =
        (row indices, rows) replaces those rows' input embeddings (image / audio rows); ``image_blocks`` = absolute
        [start, end) runs of image rows, which must lie inside this call (a block is never split over calls)."""
        cfg, w = self.cfg, self.w
        st = st if st is not None else OracleState()
        x = w["text.embed_tokens"][ids.long()]
        if embed_overrides is not None:
            x = x.clone()
            x[embed_overrides[0].long()] = embed_overrides[1].float()
        self.image_blocks = list(image_blocks) if image_blocks else None
        captured = {}
        rot = self._rotation()
        if rot is not None:                      # rows enter the stack: the stack's basis is x Q
            x = self._r(rot[0](x.float()))
        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            if capture_layers and i in capture_layers:
                captured[i] = x.clone() if rot is None else self._r(rot[1](x.float()))     # consumers read un-rotated rows
            h = self._r(R.rmsnorm_1pw(x, w[p + "input_layernorm"], cfg.rms_norm_eps))
            if cfg.is_attention_layer(i):
                a = self.attention(p, i, h, st)
            elif cfg.is_conv_layer(i):
                a = self.short_conv(p, i, h, st)
            else:
                a = self.gdn(p, i, h, st)
            if cfg.sandwich_norm:
                a = self._r(R.rmsnorm_1pw(a, w[p + "post_attn_out_norm"], cfg.rms_norm_eps))
            x = self._r(x + a)
            h = self._r(R.rmsnorm_1pw(x, w[p + "post_attention_layernorm"], cfg.rms_norm_eps))
            m = self.moe(p, h) if cfg.layer_is_moe(i) else self.mlp(p, h)
            if cfg.sandwich_norm:
                m = self._r(R.rmsnorm_1pw(m, w[p + "post_mlp_out_norm"], cfg.rms_norm_eps))
            x = self._r(x + m)
        st.pos += ids.shape[0]
        self.image_blocks = None
        if rot is not None:                      # rows leave the stack
            x = self._r(rot[1](x.float()))
        hn = self._r(R.rmsnorm_1pw(x, w["text.final_norm"], cfg.rms_norm_eps))
        logits = self._mm(hn, "lm_head")
        if return_hidden:
            return logits, x, st, captured
        return logits, st

    def _rotation(self):
        """(x -> x Q, x -> x Q^T) when the weight set carries a residual rotation, else None."""
        if "rotation.signs" not in self.w:
            return None
        from ..quant import rotation as rot
        signs, mix = self.w["rotation.signs"].float(), self.w["rotation.mix"].float()
        spec = rot.RotationSpec("q2a", 0, signs.numel(), signs.numel() // mix.shape[0])
        return (lambda t: rot.apply_q(t, spec, signs, mix)), (lambda t: rot.apply_qt(t, spec, signs, mix))

    def mtp_step(self, token: torch.Tensor, hidden: torch.Tensor, st: OracleState) -> tuple:
        """One MTP draft step: x = fc([norm_e(embed(t)), norm_h(h)]) -> attention layer -> norm -> lm_head.

        ``st`` is the MTP head's own KV state (layer key "mtp").  (reference: src/model/mtp_head.h:7-60)
        """
        cfg, w = self.cfg, self.w
        e = R.rmsnorm_1pw(w["text.embed_tokens"][token.long()], w["mtp.pre_fc_norm_embedding"], cfg.rms_norm_eps)
        h = R.rmsnorm_1pw(hidden, w["mtp.pre_fc_norm_hidden"], cfg.rms_norm_eps)
        x = self._r(torch.cat([e, h], dim=-1) @ w["mtp.fc"].T)
        hn = self._r(R.rmsnorm_1pw(x, w["mtp.input_layernorm"], cfg.rms_norm_eps))
        x = self._r(x + self.attention("mtp.", "mtp", hn, st))
        hn = self._r(R.rmsnorm_1pw(x, w["mtp.post_attention_layernorm"], cfg.rms_norm_eps))
        x = self._r(x + self.mlp("mtp.", hn))
        st.pos += token.shape[0]
        out = self._r(R.rmsnorm_1pw(x, w["mtp.norm"], cfg.rms_norm_eps))
        return out @ w["lm_head"].T, x, st

    def greedy(self, prompt: torch.Tensor, n: int) -> List[int]:
        logits, st = self.forward(prompt)
        out = []
        tok = int(argmax_lowest(logits[-1]))
        for _ in range(n):
            out.append(tok)
            logits, st = self.forward(torch.tensor([tok]), st)
            tok = int(argmax_lowest(logits[-1]))
        return out


def argmax_lowest(row: torch.Tensor) -> int:
    """Greedy pick with ties to the lowest id (reference: src/kernels/include/r4dx/kernels/kernels.h:297-308)."""
    m = row.max()
    return int(torch.nonzero(row == m)[0, 0])
