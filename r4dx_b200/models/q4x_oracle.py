"""fp32 CPU reference of the qwen4_exp family: a 4-stream gated residual around every mixer and every expert block, one
hashed n-gram embedding layer, Gated DeltaNet mixers with a sigmoid output gate, and attention layers that look at the
top-scoring key blocks only.

    h0 = embedding row repeated over the streams                          [T, hc * H]
    layer i:  (n-gram block first, on the layers that have one)   h += ple(h, ngram rows)
              x, inj = gate(h);  h += broadcast(mixer(x)) * inj     mixer = GDN or sparse attention
              x, inj = gate(h);  h += broadcast(moe(x)) * inj
    logits = lm_head(final_gate(h))                                       no norm before the head

    gate(h):  n = rmsnorm per stream (1 + w);  m = sigmoid(up(silu(down(n) / hc)));  x = mean over streams of m * n;
              inj = 2 * sigmoid(inject(n) / hc)                            [T, hc]

(reference: docs/qwen4exp-plan.md 2.2-2.4; kernel contracts in src/model/qwen4exp/include/r4dx/model/qwen4exp/
hc_kernels.h:20-52, ple_kernels.h:5-46, qsa_kernels.h:12-28.)  The block selection breaks ties towards the most recent
blocks, as the reference does (qwen4exp-plan.md Q23).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import reference as R
from .oracle import OracleModel, OracleState


def init_q4x_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random weights in the container's names (reference: src/model/qwen4exp_container.h:11-25)."""
    from .oracle import init_weights
    w = init_weights(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 101)
    n = lambda *s, sd=std: torch.randn(*s, generator=g, dtype=torch.float32) * sd
    H, hc, C, L = cfg.hidden_size, cfg.hc_count, cfg.hc_count * cfg.hidden_size, cfg.hc_lowrank
    for k in [k for k in w if k.endswith("layernorm") or k == "text.final_norm"]:
        del w[k]                                    # the stream gate's norm is the only norm of a layer

    def hc_block(p: str, inject: bool = True):
        w[p + "norm"] = n(C)
        w[p + "down"] = n(L, C)
        w[p + "up"] = n(C, L, sd=0.3)
        if inject:
            w[p + "inject"] = n(hc, C, sd=0.05)

    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        hc_block(p + "hc.attn.")
        hc_block(p + "hc.mlp.")
        if cfg.is_attention_layer(i) and cfg.indexer_heads:
            w[p + "attn.indexer.qk"] = n((cfg.indexer_heads + 1) * cfg.indexer_dim, H, sd=0.08)
            w[p + "attn.indexer.q_norm"] = n(cfg.indexer_dim)
            w[p + "attn.indexer.k_norm"] = n(cfg.indexer_dim)
        if i in cfg.ple_layers:
            w[p + "ple.key_proj"] = n(C, cfg.ple_embed_dim, sd=0.5)
            w[p + "ple.value_proj"] = n(H, cfg.ple_embed_dim, sd=0.5)
            for name in ("norm_key", "norm_query", "norm_conv"):
                w[p + "ple." + name] = n(C)
            w[p + "ple.conv1d"] = n(C, cfg.ple_conv_kernel, sd=0.4)
    hc_block("text.hc_final.", inject=False)
    return w


def grouped_rmsnorm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    T, C = x.shape
    xg = x.float().view(T, groups, C // groups)
    y = xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)
    return y.view(T, C) * (1.0 + w.float())


def select_blocks(scores: torch.Tensor, topk: int) -> torch.Tensor:
    """Indices (ascending) of the ``topk`` best blocks by (score descending, index descending)."""
    nb = scores.numel()
    order = sorted(range(nb), key=lambda b: (-float(scores[b]), -b))[:topk]
    return torch.tensor(sorted(order), dtype=torch.long)


class Q4xState(OracleState):
    def __init__(self):
        super().__init__()
        self.tokens: List[int] = []                 # every token fed (the n-gram history and nothing else reads it)
        self.ple_hist: Dict[int, torch.Tensor] = {}  # layer -> normalised gated values of every position [S, C]
        self.idx_k: Dict[int, torch.Tensor] = {}     # layer -> raw indexer keys of every position [S, index_dim]
        self.selected: Dict[int, list] = {}          # layer -> per row of the last call: selected token list or None (dense)

    def clone(self) -> "Q4xState":
        c = Q4xState()
        c.pos = self.pos
        for name in ("k", "v", "gdn", "conv", "ple_hist", "idx_k"):
            setattr(c, name, {i: t.clone() for i, t in getattr(self, name).items()})
        c.tokens = list(self.tokens)
        return c


class Q4xOracle(OracleModel):
    """``ngram_rows(tokens, history) -> [T, ple_embed_dim]`` supplies the table rows (a table object or a test stub)."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], ngram_rows, fp8_kv: bool = False,
                 act_dtype: Optional[torch.dtype] = None):
        super().__init__(cfg, weights, fp8_kv=fp8_kv, act_dtype=act_dtype)
        if not cfg.is_qwen4_exp:
            raise ValueError("not a qwen4_exp configuration")
        self.ngram_rows = ngram_rows

    # ---- stream gate ------------------------------------------------------------------------
    def hc_prep(self, p: str, h: torch.Tensor, inject: bool = True):
        cfg, w = self.cfg, self.w
        hc, H = cfg.hc_count, cfg.hidden_size
        n = self._r(grouped_rmsnorm(h, w[p + "norm"], hc, cfg.rms_norm_eps))
        mid = self._r(F.silu(self._r(self._r(n @ w[p + "down"].T) / hc)))
        m = self._r(torch.sigmoid(self._r(mid @ w[p + "up"].T)))
        x = self._r(self._r(m * n).view(-1, hc, H).mean(1))
        inj = None
        if inject:
            inj = self._r(2.0 * self._r(torch.sigmoid(self._r(self._r(n @ w[p + "inject"].T) / hc))))
        return x, inj

    def hc_inject(self, h: torch.Tensor, out: torch.Tensor, inj: torch.Tensor) -> torch.Tensor:
        hc, H = self.cfg.hc_count, self.cfg.hidden_size
        add = self._r(out[:, None, :] * inj[:, :, None]).reshape(-1, hc * H)
        return self._r(h + add)

    # ---- n-gram embedding layer ----------------------------------------------------------------
    def ple(self, p: str, li: int, h: torch.Tensor, emb: torch.Tensor, st: Q4xState) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        hc, H = cfg.hc_count, cfg.hidden_size
        T = h.shape[0]
        kp = self._r(emb @ w[p + "ple.key_proj"].T)
        val = self._r(emb @ w[p + "ple.value_proj"].T)
        kn = self._r(grouped_rmsnorm(kp, w[p + "ple.norm_key"], hc, cfg.rms_norm_eps)).view(T, hc, H)
        qn = self._r(grouped_rmsnorm(h, w[p + "ple.norm_query"], hc, cfg.rms_norm_eps)).view(T, hc, H)
        gate = self._r(self._r((kn * qn).sum(-1)) / math.sqrt(H))
        gate = self._r(torch.sqrt(gate.abs().clamp_min(1e-6))) * torch.sign(gate)
        gv = self._r(self._r(torch.sigmoid(gate))[:, :, None] * val[:, None, :]).reshape(T, hc * H)
        gvn = self._r(grouped_rmsnorm(gv, w[p + "ple.norm_conv"], hc, cfg.rms_norm_eps))
        hist = torch.cat([st.ple_hist[li], gvn], 0) if li in st.ple_hist else gvn
        st.ple_hist[li] = hist
        S, Kc, dil = hist.shape[0], cfg.ple_conv_kernel, cfg.ple_conv_dilation
        cw = self._r(w[p + "ple.conv1d"])
        conv = torch.zeros(T, hc * H)
        for t in range(T):
            at = S - T + t
            for j in range(Kc):                       # tap j reads the value (Kc - 1 - j) * dilation steps back; before the start: 0
                src = at - (Kc - 1 - j) * dil
                if src >= 0:
                    conv[t] += cw[:, j] * hist[src]
        out = self._r(gv + self._r(F.silu(self._r(conv))))
        return self._r(h + out)

    # ---- sparse attention -----------------------------------------------------------------------
    def indexer_select(self, p: str, li: int, x: torch.Tensor, st: Q4xState) -> list:
        """Per row: None while the row sees at most budget / ratio complete blocks (dense), else the selected tokens."""
        cfg, w = self.cfg, self.w
        T = x.shape[0]
        Hi, Di, ratio, topk = cfg.indexer_heads, cfg.indexer_dim, cfg.indexer_ratio, cfg.indexer_budget // cfg.indexer_ratio
        qk = self._r(x @ w[p + "attn.indexer.qk"].T).view(T, Hi + 1, Di)
        pos = torch.arange(st.pos, st.pos + T)
        q = self._r(R.rmsnorm_1pw(qk[:, :Hi], w[p + "attn.indexer.q_norm"], cfg.rms_norm_eps))
        q = self._r(R.rope_partial_neox(q, pos, cfg.rotary_dim, cfg.rope_theta))
        raw = qk[:, Hi]
        keys = torch.cat([st.idx_k[li], raw], 0) if li in st.idx_k else raw
        st.idx_k[li] = keys
        nb_all = keys.shape[0] // ratio
        bk = None
        if nb_all:
            pooled = self._r(keys[:nb_all * ratio].view(nb_all, ratio, Di).sum(1) * (1.0 / ratio))
            bk = self._r(R.rmsnorm_1pw(pooled[:, None, :], w[p + "attn.indexer.k_norm"], cfg.rms_norm_eps))
            bk = self._r(R.rope_partial_neox(bk, torch.arange(nb_all) * ratio, cfg.rotary_dim, cfg.rope_theta))[:, 0]
        sel = []
        for t in range(T):
            ptok = st.pos + t
            nb = (ptok + 1) // ratio
            if nb <= topk:
                sel.append(None)
                continue
            s = torch.relu(torch.einsum("hd,bd->hb", q[t], bk[:nb])).sum(0) / math.sqrt(Di)
            blocks = select_blocks(s, topk)
            toks = (blocks[:, None] * ratio + torch.arange(ratio)[None, :]).reshape(-1).tolist()
            toks += list(range(nb * ratio, ptok + 1))
            sel.append(toks)
        return sel

    def attention(self, p: str, li, x: torch.Tensor, st: Q4xState, store: bool = True) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        if not cfg.indexer_heads:
            return super().attention(p, li, x, st, store)
        T = x.shape[0]
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        sel = self.indexer_select(p, li, x, st)
        st.selected[li] = sel
        qg = self._r(self._mm(x, p + "attn.qg")).view(T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        k = self._r(self._mm(x, p + "attn.k")).view(T, Hkv, D)
        v = self._r(self._mm(x, p + "attn.v")).view(T, Hkv, D)
        q = R.rmsnorm_1pw(q, w[p + "attn.q_norm"], cfg.rms_norm_eps)
        k = R.rmsnorm_1pw(k, w[p + "attn.k_norm"], cfg.rms_norm_eps)
        pos = torch.arange(st.pos, st.pos + T)
        q = self._r(R.rope_partial_neox(q, pos, cfg.rotary_dim, cfg.rope_theta))
        k = R.rope_partial_neox(k, pos, cfg.rotary_dim, cfg.rope_theta)
        if self.on_kv is not None:
            self.on_kv(li, k, v)
        if self.fp8_kv:
            k = R.fp8_e4m3_roundtrip(k, w[p + "attn.k_descale"][None, :, None])
            v = R.fp8_e4m3_roundtrip(v, w[p + "attn.v_descale"][None, :, None])
        Kc = torch.cat([st.k[li], k], 0) if li in st.k else k
        Vc = torch.cat([st.v[li], v], 0) if li in st.v else v
        st.k[li], st.v[li] = Kc, Vc
        g = Hq // Hkv
        out = torch.zeros(T, Hq, D)
        for t in range(T):
            toks = torch.tensor(sel[t] if sel[t] is not None else list(range(st.pos + t + 1)), dtype=torch.long)
            kk, vv = Kc[toks], Vc[toks]                                   # [S, Hkv, D]
            s = torch.einsum("hgd,shd->hgs", q[t].view(Hkv, g, D), kk) / math.sqrt(D)
            out[t] = torch.einsum("hgs,shd->hgd", torch.softmax(s, -1), vv).reshape(Hq, D)
        o = self._r(self._r(out) * self._r(torch.sigmoid(gate)))
        return self._r(self._mm(o.reshape(T, Hq * D), p + "attn.o"))

    # ---- GDN with the sigmoid gate -----------------------------------------------------------------
    def gdn(self, p: str, li, x: torch.Tensor, st: Q4xState) -> torch.Tensor:
        if self.cfg.gdn_gate_act != "sigmoid":
            return super().gdn(p, li, x, st)
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
        gt, beta = R.gdn_gates(a, b, w[p + "gdn.A_log"], w[p + "gdn.dt_bias"])
        o, st.gdn[li] = R.gdn_recurrent(q, k, v, gt, beta, st.gdn.get(li))
        o = self._r(R.rmsnorm_plain(o, w[p + "gdn.norm_weight"], cfg.rms_norm_eps) * torch.sigmoid(z.float()))
        return self._r(self._mm(o.reshape(T, H * Vd), p + "gdn.out_proj"))

    # ---- model ---------------------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, st: Optional[Q4xState] = None, return_hidden: bool = False, **unused):
        cfg, w = self.cfg, self.w
        st = st if st is not None else Q4xState()
        toks = [int(t) for t in ids.tolist()]
        eos = cfg.eos_token_id
        hist = ([eos, eos] + st.tokens)[-2:]
        emb = self.ngram_rows(toks, hist).float() if cfg.ple_layers else None
        st.tokens += toks
        h = self._r(w["text.embed_tokens"][ids.long()]).repeat(1, cfg.hc_count)
        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            if i in cfg.ple_layers:
                h = self.ple(p, i, h, emb, st)
            x, inj = self.hc_prep(p + "hc.attn.", h)
            a = self.attention(p, i, x, st) if cfg.is_attention_layer(i) else self.gdn(p, i, x, st)
            h = self.hc_inject(h, a, inj)
            x, inj = self.hc_prep(p + "hc.mlp.", h)
            h = self.hc_inject(h, self.moe(p, x), inj)
        st.pos += ids.shape[0]
        x, _ = self.hc_prep("text.hc_final.", h, inject=False)
        logits = self._mm(x, "lm_head")
        if return_hidden:
            return logits, h, st, {}
        return logits, st


def table_rows_fn(table):
    """``ngram_rows`` for the oracle from an opened table (``runtime.ngram.NgramTable``): reference ids, rows read on the host."""
    import numpy as np
    from ..runtime import ngram as NG

    def rows(tokens, history):
        ids = np.asarray(NG.ngram_ids_reference(tokens, table.header, history), dtype=np.int64)
        return table.rows(ids).reshape(len(tokens), -1)
    return rows


def make_oracle(cfg: ModelConfig, weights: Dict[str, torch.Tensor], ngram_table=None, **kw):
    """The CPU oracle of ``cfg``'s family (calibration, KL reports, tests): ``Q4xOracle`` for the 4-stream family (its
    n-gram layer needs the table; without one the layer sees zero rows, which only suits shape checks), ``OracleModel`` else."""
    if not cfg.is_qwen4_exp:
        return OracleModel(cfg, weights, **kw)
    if ngram_table is not None:
        rows = table_rows_fn(ngram_table)
    else:
        rows = lambda tokens, history: torch.zeros(len(tokens), cfg.ple_embed_dim)
    return Q4xOracle(cfg, weights, rows, **kw)
