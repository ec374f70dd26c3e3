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
Prompts run through the 8-row weight-streaming path (this family has no tensor-core chunk path here); speculative windows
are refused, as the reference refuses them for this family.
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
        (statistics + [down; inject] product + silu, then up product + mix: 95 us -> 12 us per gate on the full geometry);
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

    def prefill(self, ids: torch.Tensor, chunk: Optional[int] = None, hook=None, embed_overrides=None, image_blocks=None) -> int:
        if embed_overrides is not None or image_blocks or hook is not None:
            raise NotImplementedError("the qwen4_exp family is text only and has no drafter hooks")
        tok = self.prefill_small(ids)
        last = (ids.numel() - 1) % MAX_ROWS
        if last:                                   # callers read the prompt's last logits row at index 0, as after a chunked prefill
            self.buf.logits[0].copy_(self.buf.logits[last])
            self.buf.next_ids[:1].copy_(self.buf.next_ids[last:last + 1])
            self.last_row = 0
        return tok

    def enable_graphs(self, rows=(1,)) -> None:
        if not self.host_ngram:
            super().enable_graphs(rows)

    def decode_step_graph(self) -> None:
        if not self.host_ngram:
            return super().decode_step_graph()
        tok = int(self.buf.ids[0].item())          # host placement of the table: the ids are hashed on the host, so the step is eager
        self.feed(torch.tensor([tok], dtype=torch.int32))
        self.buf.ids[:1].copy_(self.buf.next_ids[:1])

    def forward_chunk(self, T: int, want_logits: bool, skip_embed: bool = False) -> None:
        raise NotImplementedError("no tensor-core chunk path for the qwen4_exp family: prompts take prefill_small")

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
