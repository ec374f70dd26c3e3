"""Device model of the qwen4_exp family: Gated DeltaNet and block-selecting attention mixers and a 512-expert MoE, each
wrapped in a gated 4-stream residual, plus one hashed n-gram embedding layer.

    h0 = embedding row repeated over the streams
    layer: [h += ngram_layer(h, table rows)]   x, inj = gate(h); h += mixer(x) * inj   x, inj = gate(h); h += moe(x) * inj
    logits = lm_head(final_gate(h))

The class reuses the hybrid model's machinery (weights, recurrent and KV state, staging, CUDA graphs, checkpoints, the
weight-streaming and expert kernels) and replaces the layer bodies: the stream gate is the only norm of a layer, so the
mixers' projections run without a norm prologue and write a block output instead of adding to a residual row.

What differs from the reference's runtime (src/model/qwen4exp_stage.cpp, qwen4exp_model.cpp; docs/qwen4exp.md):
  * one GPU holds the model and the n-gram table (51 + 95 GiB of 180 GB), so there is no two-card layer split, no host
    bounce of the residual, and no NVMe read per token: the row ids are hashed on the device from a device-resident token
    history and the rows are gathered by the same kernel;
  * every piece of state this family adds is keyed by position (token history, indexer keys, block keys, a 32-row ring for
    the n-gram layer's conv), so a checkpoint adds one small ring and a rewind repairs nothing;
  * every launch has position-independent geometry (the selection kernels take the context bound, attention splits are
    sized by the selection budget), so the whole step is captured in one CUDA graph, n-gram layer and sparse attention
    included (the reference launches those two outside its graphs).
Prompts run in chunks of ``chunk_rows`` rows on the tensor cores (trellis products, stream-gate products, router and grouped
experts; the recurrence stays token by token unless ``chunked_scan`` is set); speculative windows are refused, as the
reference refuses them for this family.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..ops import kernels as K
from .hybrid import BF, MAX_ROWS, HybridModel


class Qwen4ExpModel(HybridModel):
    def __init__(self, cfg: ModelConfig, weights: Dict[str, object], ngram_table=None, max_ctx: int = 8192 + 1024,
                 device: str = "cuda", attn_splits: Optional[int] = None):
        if not cfg.is_qwen4_exp:
            raise ValueError("not a qwen4_exp configuration")
        if cfg.tp_world != 1:
            raise NotImplementedError("qwen4_exp runs on one GPU: no tensor-parallel sharding of this family")
        super().__init__(cfg, weights, max_ctx=max_ctx, device=device, attn_splits=attn_splits)
        dev, w = self.device, weights
        H, hc, L = cfg.hidden_size, cfg.hc_count, cfg.hc_lowrank
        C, R = hc * H, MAX_ROWS
        e = lambda *s, dtype=BF: torch.zeros(*s, dtype=dtype, device=dev)
        f32 = torch.float32
        # ---- stream gates: [down; inject] as one product per gate ----
        self.hc_w: Dict[str, torch.Tensor] = {}
        for i in range(cfg.num_hidden_layers):
            for kind in ("attn", "mlp"):
                p = f"text.layers.{i}.hc.{kind}."
                self.hc_w[p] = torch.cat([w[p + "down"], w[p + "inject"]], 0).contiguous()
        self.hc_w["text.hc_final."] = w["text.hc_final.down"].contiguous()
        self.hx, self.hn = e(R, C), e(R, C)
        self.hc_dn, self.hc_mid, self.hc_up = e(R * (L + hc), dtype=f32), e(R, L), e(R, C, dtype=f32)
        self.bout = e(R, H)
        self.hc_inj, self.hc_rstd = e(R, hc, dtype=f32), e(R, hc, dtype=f32)
        # ---- n-gram layer ----
        self.ngram = None
        self.host_ngram = False
        self.tok_hist = e(self.max_ctx + 2 * R, dtype=torch.int32)
        self.ple_ring: Dict[int, torch.Tensor] = {i: e(32, C) for i in cfg.ple_layers}
        if cfg.ple_layers:
            if ngram_table is None:
                raise ValueError("this model has an n-gram layer: pass its table (runtime.ngram.NgramTable.open)")
            # table in device memory: ids and rows by one kernel, graph decode.  Otherwise (pinned host memory, file): ids and
            # rows on the host for every call, one host-to-device copy, eager decode.
            self.host_ngram = ngram_table.body is None or ngram_table.body.device.type != "cuda"
            self._host_tokens: list = []
            hd = ngram_table.header
            if hd.heads != cfg.ngram_heads or hd.heads * hd.head_dim != cfg.ple_embed_dim:
                raise ValueError("n-gram table geometry does not match the model's ple_embed_dim")
            if hd.eos_token_id != cfg.eos_token_id:
                raise ValueError("n-gram table was built for another end-of-sequence token")
            self.ngram = ngram_table
            self.ngram_args = K.NgramDeviceArgs(hd)
            self.emb = e(R, cfg.ple_embed_dim)
            self.ple_kp, self.ple_val = e(R, C, dtype=f32), e(R, H, dtype=f32)
            self.ple_gv, self.ple_gvn = e(R, C), e(R, C)
        # ---- block-selecting attention ----
        self.raw_keys: Dict[int, torch.Tensor] = {}
        self.block_keys: Dict[int, torch.Tensor] = {}
        if cfg.indexer_heads:
            Hi, Di, ratio = cfg.indexer_heads, cfg.indexer_dim, cfg.indexer_ratio
            self.topk = cfg.indexer_budget // ratio
            self.nb_bound = (self.max_ctx + 2 * R) // ratio + 1
            for i in range(cfg.num_hidden_layers):
                if cfg.is_attention_layer(i):
                    self.raw_keys[i] = e(self.max_ctx + 2 * R, Di)
                    self.block_keys[i] = e(self.nb_bound + 1, Di)
            self.idx_qk, self.idx_q = e(R, (Hi + 1) * Di, dtype=f32), e(R, Hi, Di)
            self.scores = e(R, self.nb_bound, dtype=f32)
            self.sel_stride = cfg.indexer_budget + ratio - 1
            self.sel_tokens, self.sel_count = e(R, self.sel_stride, dtype=torch.int32), e(R, dtype=torch.int32)
            # a row never attends to more than budget + ratio - 1 tokens (dense rows see at most that many, too)
            self.qsa_splits = max(1, min(32, (self.sel_stride + 127) // 128))
            self.qsa_acc = e(R * cfg.num_attention_heads * self.qsa_splits * cfg.head_dim, dtype=f32)
            self.qsa_ml = e(R * cfg.num_attention_heads * self.qsa_splits * 2, dtype=f32)

    # ---- stream gate ------------------------------------------------------------------------------
    fused_gate = os.environ.get("R4DXB_Q4X_FUSED_GATE", "1") != "0"

    def _gate(self, p: str, T: int, inject: bool = True) -> torch.Tensor:
        """Leaves the block input in ``buf.x[:T]`` and returns the injection logits ([T, hc] fp32, a view).  Two launches
        (statistics + [down; inject] product + silu, then up product + mix; with the other launch merges of that change the
        full geometry's step went from 13.6 to 10.8 ms);
        ``fused_gate = False`` runs the five-kernel chain the fused pair is tested against."""
        cfg, b, w = self.cfg, self.buf, self.w
        hc, L = cfg.hc_count, cfg.hc_lowrank
        if self.fused_gate:
            K.q4x_hc_gate(self.hx[:T], w[p + "norm"], self.hc_w[p], w[p + "up"], self.hc_mid, self.hc_inj, self.hc_rstd, b.x[:T], T,
                          hc, L, hc if inject else 0, cfg.rms_norm_eps)
            return self.hc_inj[:T]
        K.q4x_grouped_rmsnorm(self.hx[:T], w[p + "norm"], hc, cfg.rms_norm_eps, out=self.hn[:T])
        n_out = L + (hc if inject else 0)
        dn = self.hc_dn[:T * n_out].view(T, n_out)
        K.bf16_gemv(self.hc_w[p], self.hn[:T], out=dn)
        K.q4x_hc_mid(dn, self.hc_mid[:T], L, hc)
        K.bf16_gemv(w[p + "up"], self.hc_mid[:T], out=self.hc_up[:T])
        K.q4x_hc_mix(self.hn[:T], self.hc_up[:T], b.x[:T], hc)
        return dn[:, L:]

    def _inject(self, inj: torch.Tensor, T: int) -> None:
        K.q4x_hc_inject(self.hx[:T], self.bout[:T], inj, self.cfg.hc_count)

    # ---- layers -----------------------------------------------------------------------------------
    def _ngram_layer(self, i: int, T: int) -> None:
        cfg, b, w = self.cfg, self.buf, self.w
        p = f"text.layers.{i}.ple."
        hc = cfg.hc_count
        K.bf16_gemv(w[p + "key_proj"], self.emb[:T], out=self.ple_kp[:T])
        K.bf16_gemv(w[p + "value_proj"], self.emb[:T], out=self.ple_val[:T])
        K.q4x_ple_gate_value(self.ple_kp[:T], self.hx[:T], self.ple_val[:T], w[p + "norm_key"], w[p + "norm_query"],
                             self.ple_gv[:T], hc, cfg.rms_norm_eps)
        K.q4x_grouped_rmsnorm(self.ple_gv[:T], w[p + "norm_conv"], hc, cfg.rms_norm_eps, out=self.ple_gvn[:T])
        K.q4x_ple_conv(self.ple_gvn[:T], self.ple_gv[:T], w[p + "conv1d"], self.ple_ring[i], self.hx[:T], b.positions, T,
                       cfg.ple_conv_kernel, cfg.ple_conv_dilation)

    def _gdn_layer(self, i: int, T: int) -> None:
        cfg, b, w = self.cfg, self.buf, self.w
        p = f"text.layers.{i}.gdn."
        Hv, Hk, Dg = cfg.linear_num_value_heads, cfg.linear_num_key_heads, cfg.linear_key_head_dim
        x = b.x[:T]
        grp = self._siblings((p + "in_proj_qkv", p + "in_proj_z"))
        if grp is not None:
            grp(x, (b.mixed[:T], b.z[:T]))
        else:
            self.lin[p + "in_proj_qkv"](x, out=b.mixed[:T])
            self.lin[p + "in_proj_z"](x, out=b.z[:T])
        K.bf16_gemv(self.ab_w[i], x, out=b.ab[:T])
        K.gdn_decode_gate(b.mixed, b.z, b.ab, w[p + "conv1d_weight"], w[p + "A_log"], w[p + "dt_bias"], w[p + "norm_weight"],
                          self.ring[i], self.gdn_state[i], self.log_u[i], self.log_k[i], self.log_eg[i], b.positions, b.n_replay,
                          b.core, T, Hv, Hk, Dg, cfg.rms_norm_eps, 1 if cfg.gdn_gate_act == "sigmoid" else 0)
        core = b.core.view(-1)[:T * cfg.value_dim].view(T, cfg.value_dim)
        self.lin[p + "out_proj"](core, out=self.bout[:T])

    def _attn_layer(self, i: int, T: int) -> None:
        cfg, b, w = self.cfg, self.buf, self.w
        p = f"text.layers.{i}.attn."
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        x = b.x[:T]
        grp = self._siblings((p + "qg", p + "k", p + "v"))
        if grp is not None:
            grp(x, (b.qg[:T], b.k[:T], b.v[:T]))
        else:
            self.lin[p + "qg"](x, out=b.qg[:T])
            self.lin[p + "k"](x, out=b.k[:T])
            self.lin[p + "v"](x, out=b.v[:T])
        K.attn_precore(b.qg, b.k, b.v, w.get(p + "q_norm"), w.get(p + "k_norm"), w[p + "k_descale"], w[p + "v_descale"],
                       b.positions, self.block_table, b.q, self.kv[i], T, Hq, Hkv, D, cfg.rotary_dim, cfg.rope_theta,
                       cfg.rms_norm_eps, q_stride=cfg.q_proj_dim // Hq)
        core = b.core.view(-1)[:T * cfg.q_dim].view(T, cfg.q_dim)
        if not cfg.indexer_heads:
            K.attn_decode(b.q, b.qg, self.kv[i], self.block_table, b.positions, w[p + "k_descale"], w[p + "v_descale"],
                          b.part_acc, b.part_ml, core, T, Hq, Hkv, D, self.attn_splits, cfg.attn_output_gate)
        else:
            Hi, Di, ratio = cfg.indexer_heads, cfg.indexer_dim, cfg.indexer_ratio
            K.bf16_gemv(w[p + "indexer.qk"], x, out=self.idx_qk[:T])
            K.q4x_qsa_index(self.idx_qk[:T], w[p + "indexer.q_norm"], w[p + "indexer.k_norm"], b.positions, self.idx_q,
                            self.raw_keys[i], self.block_keys[i], T, Hi, Di, ratio, cfg.rotary_dim, cfg.rope_theta, cfg.rms_norm_eps)
            K.q4x_qsa_select(self.idx_q, self.block_keys[i], b.positions, self.scores, self.sel_tokens, self.sel_count, T, Hi, Di,
                             ratio, self.topk, self.nb_bound)
            K.q4x_qsa_attn(b.q, b.qg, self.kv[i], self.block_table, b.positions, self.sel_tokens, self.sel_count,
                           w[p + "k_descale"], w[p + "v_descale"], self.qsa_acc, self.qsa_ml, core, T, Hq, Hkv, D,
                           self.sel_stride, self.qsa_splits, gated=cfg.attn_output_gate)
        self.lin[p + "o"](core, out=self.bout[:T])

    def _mlp(self, i: int, T: int) -> None:
        self.moe[i].forward(self.buf.x[:T], self.bout[:T], T, residual=False)

    # ---- forward ------------------------------------------------------------------------------------
    def forward_rows(self, T: int, want_logits: bool = True, skip_embed: bool = False) -> None:
        cfg, b, w = self.cfg, self.buf, self.w
        if skip_embed:
            raise NotImplementedError("embedding overrides for the qwen4_exp family (it is text only)")
        K.q4x_embed_repeat(w["text.embed_tokens"], b.ids[:T], self.hx[:T], cfg.hc_count)
        if self.ngram is not None and not self.host_ngram:
            K.q4x_ngram_gather(b.ids, b.positions, self.tok_hist, self.ngram.body, self.emb, T, self.ngram_args)
        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            if i in self.ple_ring:
                self._ngram_layer(i, T)
            dn = self._gate(p + "hc.attn.", T)
            if cfg.is_attention_layer(i):
                self._attn_layer(i, T)
            else:
                self._gdn_layer(i, T)
            self._inject(dn, T)
            dn = self._gate(p + "hc.mlp.", T)
            self._mlp(i, T)
            self._inject(dn, T)
            if self.probe is not None and not torch.cuda.is_current_stream_capturing():
                self.probe(i, self.hx[:T])
        if want_logits:
            self._gate("text.hc_final.", T, inject=False)
            self.lin["lm_head"](b.x[:T], out=b.logits[:T])
            K.argmax_rows(b.logits[:T], 0, b.next_ids[:T], b.next_vals[:T], b.argmax_scratch)

    def feed(self, ids: torch.Tensor, want_logits: bool = True, accepted: Optional[int] = None) -> None:
        if accepted is not None and accepted != ids.numel():
            raise NotImplementedError("speculative windows (partly accepted rows) for the qwen4_exp family")
        if self.host_ngram:
            # the history is keyed by position, so a rewind (checkpoint restore, reset) needs no repair here either
            toks = [int(t) for t in ids.tolist()]
            del self._host_tokens[self.pos:]
            eos = self.cfg.eos_token_id
            self.ngram.ids.restore(([eos, eos] + self._host_tokens)[-2:])
            self.emb[:len(toks)].copy_(self.ngram.gather_host(toks), non_blocking=False)
            self._host_tokens += toks
        super().feed(ids, want_logits)

    chunk_rows = int(os.environ.get("R4DXB_Q4X_CHUNK", "1024"))       # rows per prefill chunk (0: 8-row passes only)
    # the 64-token chunked recurrence (head width 128) instead of the token-by-token one: it forms each pair decay as
    # exp(G_i - G_j) <= 1, and a test runs it on per-chunk gate sums above 10^4 nats against the exact recurrence
    chunked_scan = os.environ.get("R4DXB_Q4X_CHUNKED_SCAN", "1") == "1"

    def prefill(self, ids: torch.Tensor, chunk: Optional[int] = None, hook=None, embed_overrides=None, image_blocks=None) -> int:
        if embed_overrides is not None or image_blocks or hook is not None:
            raise NotImplementedError("the qwen4_exp family is text only and has no drafter hooks")
        ids = ids.to(torch.int32)
        n = ids.numel()
        step = chunk or self.chunk_rows
        if self.pos + n > self.max_ctx:
            raise ValueError("context overflow")
        if self.host_ngram or step <= 2 * MAX_ROWS or n <= 2 * MAX_ROWS:
            tok = self.prefill_small(ids)
            last = (n - 1) % MAX_ROWS
        else:
            # chunks on the tensor cores, a tail of up to 8 rows through the small-batch path
            self.commit_pending()
            step = min(step, n)
            self._chunk_buffers(step)
            self._q4x_chunk_buffers(step)
            s, last = 0, 0
            while s < n:
                e = min(n, s + step)
                T = e - s
                if T <= MAX_ROWS:
                    self.feed(ids[s:e], want_logits=True)
                    last = T - 1
                else:
                    cb = self._cb
                    cb["ids"][:T].copy_(ids[s:e].to(self.device), non_blocking=True)
                    cb["positions"][:T].copy_(torch.arange(self.pos, self.pos + T, dtype=torch.int32, device=self.device))
                    self.forward_chunk(T, want_logits=(e == n))
                    last = 0
                s = e
            K.check_gemm_status(self.device)
            tok = self._read_token(last)
        if last:                                   # callers read the prompt's last logits row at index 0
            self.buf.logits[0].copy_(self.buf.logits[last])
            self.buf.next_ids[:1].copy_(self.buf.next_ids[last:last + 1])
            self.last_row = 0
        return tok

    def _q4x_chunk_buffers(self, C: int) -> dict:
        qb = getattr(self, "_qb", None)
        if qb is not None and qb["C"] >= C:
            return qb
        cfg, dev = self.cfg, self.device
        H, hc, L = cfg.hidden_size, cfg.hc_count, cfg.hc_lowrank
        Ch = hc * H
        e = lambda *s, dtype=BF: torch.empty(*s, dtype=dtype, device=dev)
        f32 = torch.float32
        qb = dict(C=C, hx=e(C, Ch), hn=e(C, Ch), dn=e(C * (L + hc), dtype=f32), mid=e(C, L), up=e(C, Ch, dtype=f32), bout=e(C, H))
        if self.ngram is not None:
            qb.update(emb=e(C, cfg.ple_embed_dim), kp=e(C, Ch, dtype=f32), val=e(C, H, dtype=f32), gv=e(C, Ch), gvn=e(C, Ch))
        if cfg.indexer_heads:
            Hi, Di = cfg.indexer_heads, cfg.indexer_dim
            qb.update(idx_qk=e(C, (Hi + 1) * Di, dtype=f32), idx_q=e(C, Hi, Di), scores=e(C, self.nb_bound, dtype=f32),
                      sel_tokens=e(C, self.sel_stride, dtype=torch.int32), sel_count=e(C, dtype=torch.int32),
                      acc=e(C * cfg.num_attention_heads * self.qsa_splits * cfg.head_dim, dtype=f32),
                      ml=e(C * cfg.num_attention_heads * self.qsa_splits * 2, dtype=f32))
        self._qb = qb
        return qb

    def _gate_chunk(self, p: str, T: int) -> torch.Tensor:
        """The stream gate for a chunk: the products run on the tensor cores; block input in the chunk's x rows."""
        cfg, w, cb, qb = self.cfg, self.w, self._cb, self._qb
        hc, L = cfg.hc_count, cfg.hc_lowrank
        hn = qb["hn"][:T]
        K.q4x_grouped_rmsnorm(qb["hx"][:T], w[p + "norm"], hc, cfg.rms_norm_eps, out=hn)
        dn = qb["dn"][:T * (L + hc)].view(T, L + hc)
        K.linear_tc(self.hc_w[p], hn, out=dn)
        K.q4x_hc_mid(dn, qb["mid"][:T], L, hc)
        K.linear_tc(w[p + "up"], qb["mid"][:T], out=qb["up"][:T])
        K.q4x_hc_mix(hn, qb["up"][:T], cb["x"][:T], hc)
        return dn[:, L:]

    def forward_chunk(self, T: int, want_logits: bool, skip_embed: bool = False) -> None:
        """T (> 8) rows staged in the chunk buffers at positions self.pos ..: trellis products, stream-gate products, router
        and experts on the tensor cores; the recurrence token by token (or chunked, see ``chunked_scan``); attention over each row's
        selected tokens.  Commits the rows."""
        cfg, w, cb, qb, b = self.cfg, self.w, self._cb, self._qb, self.buf
        H, hc = cfg.hidden_size, cfg.hc_count
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        Hv, Hk, Dg = cfg.linear_num_value_heads, cfg.linear_num_key_heads, cfg.linear_key_head_dim
        x, hx, bout, pos = cb["x"][:T], qb["hx"][:T], qb["bout"][:T], cb["positions"]
        pos0 = self.pos
        K.q4x_embed_repeat(w["text.embed_tokens"], cb["ids"][:T], hx, hc)
        if self.ngram is not None:
            K.q4x_ngram_gather(cb["ids"], pos, self.tok_hist, self.ngram.body, qb["emb"], T, self.ngram_args)
        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            if i in self.ple_ring:
                pp = p + "ple."
                K.linear_tc(w[pp + "key_proj"], qb["emb"][:T], out=qb["kp"][:T])
                K.linear_tc(w[pp + "value_proj"], qb["emb"][:T], out=qb["val"][:T])
                K.q4x_ple_gate_value(qb["kp"][:T], hx, qb["val"][:T], w[pp + "norm_key"], w[pp + "norm_query"], qb["gv"][:T], hc,
                                     cfg.rms_norm_eps)
                K.q4x_grouped_rmsnorm(qb["gv"][:T], w[pp + "norm_conv"], hc, cfg.rms_norm_eps, out=qb["gvn"][:T])
                K.q4x_ple_conv(qb["gvn"][:T], qb["gv"][:T], w[pp + "conv1d"], self.ple_ring[i], hx, pos, T, cfg.ple_conv_kernel,
                               cfg.ple_conv_dilation)
            inj = self._gate_chunk(p + "hc.attn.", T)
            if cfg.is_attention_layer(i):
                pa = p + "attn."
                qg, kk, vv, q = cb["qg"][:T], cb["k"][:T], cb["v"][:T], cb["q"][:T]
                self.lin[pa + "qg"].chunk(x, cb["xh"], qg)
                self.lin[pa + "k"].chunk(x, cb["xh"], kk)
                self.lin[pa + "v"].chunk(x, cb["xh"], vv)
                K.attn_precore(qg, kk, vv, w.get(pa + "q_norm"), w.get(pa + "k_norm"), w[pa + "k_descale"], w[pa + "v_descale"],
                               pos, self.block_table, q, self.kv[i], T, Hq, Hkv, D, cfg.rotary_dim, cfg.rope_theta,
                               cfg.rms_norm_eps, q_stride=cfg.q_proj_dim // Hq)
                core = cb["core"][:T * cfg.q_dim].view(T, cfg.q_dim)
                if cfg.indexer_heads:
                    Hi, Di, ratio = cfg.indexer_heads, cfg.indexer_dim, cfg.indexer_ratio
                    K.linear_tc(w[pa + "indexer.qk"], x, out=qb["idx_qk"][:T])
                    K.q4x_qsa_index(qb["idx_qk"][:T], w[pa + "indexer.q_norm"], w[pa + "indexer.k_norm"], pos, qb["idx_q"],
                                    self.raw_keys[i], self.block_keys[i], T, Hi, Di, ratio, cfg.rotary_dim, cfg.rope_theta,
                                    cfg.rms_norm_eps)
                    K.q4x_qsa_select(qb["idx_q"], self.block_keys[i], pos, qb["scores"], qb["sel_tokens"], qb["sel_count"], T, Hi, Di,
                                     ratio, self.topk, min(self.nb_bound, (pos0 + T) // ratio + 1))
                    K.q4x_qsa_attn(q, qg, self.kv[i], self.block_table, pos, qb["sel_tokens"], qb["sel_count"], w[pa + "k_descale"],
                                   w[pa + "v_descale"], qb["acc"], qb["ml"], core, T, Hq, Hkv, D, self.sel_stride, self.qsa_splits,
                                   gated=cfg.attn_output_gate)
                else:
                    K.attn_prefill(q, qg, self.kv[i], self.block_table, w[pa + "k_descale"], w[pa + "v_descale"], core, T, Hq, Hkv, D,
                                   pos0, cfg.attn_output_gate)
                self.lin[pa + "o"].chunk(core, cb["xh"], bout)
            else:
                pg = p + "gdn."
                mixed, z, ab = cb["mixed"][:T * cfg.conv_dim].view(T, cfg.conv_dim), cb["z"][:T], cb["ab"][:T]
                self.lin[pg + "in_proj_qkv"].chunk(x, cb["xh"], mixed)
                self.lin[pg + "in_proj_z"].chunk(x, cb["xh"], z)
                if self.ab_w[i].shape[0] % 4 == 0:
                    K.linear_tc(self.ab_w[i], x, out=ab)
                else:
                    K.bf16_gemv(self.ab_w[i], x, out=ab)
                core = cb["core"][:T * cfg.value_dim].view(T, cfg.value_dim)
                K.gdn_prefill_gate(mixed, z, ab, w[pg + "conv1d_weight"], w[pg + "A_log"], w[pg + "dt_bias"], w[pg + "norm_weight"],
                                   self.ring[i], self.gdn_state[i], cb["gdn"], core, T, Hv, Hk, Dg, pos0, cfg.rms_norm_eps,
                                   1 if cfg.gdn_gate_act == "sigmoid" else 0, exact_scan=not self.chunked_scan)
                self.lin[pg + "out_proj"].chunk(core, cb["xh"], bout)
            K.q4x_hc_inject(hx, bout, inj, hc)
            inj = self._gate_chunk(p + "hc.mlp.", T)
            bout.zero_()                            # the chunk MoE adds into its output rows: from zero that is the block output
            self._moe_chunk(i, x, bout, T)
            K.q4x_hc_inject(hx, bout, inj, hc)
        if want_logits:
            self.hx[:1].copy_(hx[T - 1:T])
            self._gate("text.hc_final.", 1, inject=False)
            self.lin["lm_head"](b.x[:1], out=b.logits[:1])
            K.argmax_rows(b.logits[:1], 0, b.next_ids[:1], b.next_vals[:1], b.argmax_scratch)
        self.pos += T
        self.pending_rows = 0

    def enable_graphs(self, rows=(1,)) -> None:
        if not self.host_ngram:
            super().enable_graphs(rows)

    def decode_step_graph(self) -> None:
        if not self.host_ngram:
            return super().decode_step_graph()
        tok = int(self.buf.ids[0].item())          # host placement of the table: the ids are hashed on the host, so the step is eager
        self.feed(torch.tensor([tok], dtype=torch.int32))
        self.buf.ids[:1].copy_(self.buf.next_ids[:1])

    def verify_window(self, anchor, drafts):
        raise NotImplementedError("speculative decoding for the qwen4_exp family")

    # ---- state ----------------------------------------------------------------------------------------
    def reset(self) -> None:
        super().reset()
        for t in self.ple_ring.values():
            t.zero_()

    def save_checkpoint(self) -> dict:
        ck = super().save_checkpoint()
        ck["ple_ring"] = {i: t.clone() for i, t in self.ple_ring.items()}
        return ck

    def restore_checkpoint(self, ck: dict) -> None:
        super().restore_checkpoint(ck)
        for i, t in ck["ple_ring"].items():
            self.ple_ring[i].copy_(t)

    def _snapshot(self):
        snap = super()._snapshot()
        snap["ple_ring"] = {i: t.clone() for i, t in self.ple_ring.items()}
        snap["hx"] = self.hx.clone()
        return snap

    def _restore(self, snap) -> None:
        super()._restore(snap)
        for i, t in snap["ple_ring"].items():
            self.ple_ring[i].copy_(t)
        self.hx.copy_(snap["hx"])

    def state_bytes(self) -> int:
        n = super().state_bytes()
        for d in (self.raw_keys, self.block_keys, self.ple_ring):
            n += sum(t.numel() * t.element_size() for t in d.values())
        return n + self.tok_hist.numel() * 4

    def selected_tokens(self, row: int):
        """The token list the latest attention layer call used for ``row`` (None for a row that attended densely)."""
        c = int(self.sel_count[row].item())
        return None if c < 0 else self.sel_tokens[row, :c].tolist()
