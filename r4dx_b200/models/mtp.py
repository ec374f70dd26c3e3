"""Multi-token-prediction drafter: one extra gated-attention decoder layer that predicts the token after
next from (embedding of the next token, hidden state of the main model), chained k times.

    x = fc([rmsnorm_e(embed(t_{i+1})), rmsnorm_h(h_i)]) -> attention layer + MLP -> norm -> shared lm_head

The head keeps its own KV cache in lock-step with the main model: position i holds the K/V computed from
the TRUE pair (t_{i+1}, h_i).  Draft steps overwrite positions beyond the committed frontier with
speculative values; they are re-primed with true pairs after every verify (position-keyed overwrite, no
rollback needed because the head has no recurrent state)
(reference: src/model/mtp_head.h:7-60, priming src/model/model.cpp:1609-1686, rounds :3440-3516).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config import ModelConfig
from ..ops import kernels as K
from .hybrid import MAX_ROWS, HybridModel, Linear

BF = torch.bfloat16


def mtp_config(cfg: ModelConfig, vocab: int = 0) -> ModelConfig:
    import dataclasses
    c = dataclasses.replace(cfg, num_hidden_layers=1, layer_types=["full_attention"])
    if vocab:
        c.vocab_size = vocab                 # a reduced-vocabulary draft head: the logits buffers shrink with it
    return c


class MtpDrafter:
    kind = "mtp"

    def __init__(self, main: HybridModel, weights: Dict[str, object], use_draft_head: bool = True):
        self.main = main
        cfg = main.cfg
        # a container may carry a smaller head over a subset of the vocabulary for the drafter's own drafts
        # (mtp.draft_head.lm_head [Vd, H] + mtp.draft_head.vocab_ids [Vd]): drafting reads Vd rows instead of the full
        # vocabulary; the verify pass scores the full vocabulary, so what is emitted does not change
        # (reference: src/convert/main.cpp:165-169 "reduced-vocab draft head").  Single-rank models only.
        self.vocab_ids = None
        head_w = weights["lm_head"]
        vocab = 0
        if use_draft_head and "mtp.draft_head.lm_head" in weights and (main.comm is None or main.comm.world == 1):
            head_w = weights["mtp.draft_head.lm_head"]
            self.vocab_ids = weights["mtp.draft_head.vocab_ids"].to(main.device, torch.int32).contiguous()
            vocab = int(self.vocab_ids.numel())
        w: Dict[str, object] = {"text.embed_tokens": weights["text.embed_tokens"], "lm_head": head_w,
                                "text.final_norm": weights["mtp.norm"]}
        for k, v in weights.items():
            if k.startswith("mtp.") and not k.startswith("mtp.draft_head.") and \
                    k not in ("mtp.fc", "mtp.norm", "mtp.pre_fc_norm_embedding", "mtp.pre_fc_norm_hidden"):
                w["text.layers.0." + k[4:]] = v
        self.head = HybridModel(mtp_config(cfg, vocab), w, max_ctx=main.max_ctx, device=str(main.device), comm=main.comm)
        self.fc = Linear(weights["mtp.fc"], "mtp.fc")
        self.norm_e, self.norm_h = weights["mtp.pre_fc_norm_embedding"], weights["mtp.pre_fc_norm_hidden"]
        H = cfg.hidden_size
        dev = main.device
        self.cat = torch.zeros(MAX_ROWS, 2 * H, dtype=BF, device=dev)
        self.emb = torch.zeros(MAX_ROWS, H, dtype=BF, device=dev)
        self.tmp = torch.zeros(MAX_ROWS, H, dtype=BF, device=dev)
        self.ids = torch.zeros(MAX_ROWS, dtype=torch.int32, device=dev)
        self.h_last = torch.zeros(1, H, dtype=BF, device=dev)        # main hidden state of the last committed row
        self.rounds = 0
        self.accepted = 0

    def reset(self) -> None:
        self.head.reset()
        self.h_last.zero_()

    # ---- building the head's input rows ---------------------------------------------------------
    def _inputs(self, tokens: torch.Tensor, hidden: torch.Tensor, out_x: torch.Tensor) -> None:
        """out_x[T, H] = fc([norm_e(embed(tokens)), norm_h(hidden)])"""
        T = tokens.numel()
        eps = self.main.cfg.rms_norm_eps
        if T <= MAX_ROWS:
            self.ids[:T].copy_(tokens)
            K.embed_gather(self.ids[:T], self.head.w["text.embed_tokens"], out=self.emb[:T])
            K.rmsnorm(self.emb[:T], self.norm_e, eps, out=self.tmp[:T])
            self.cat[:T, :self.tmp.shape[1]].copy_(self.tmp[:T])
            K.rmsnorm(hidden.contiguous(), self.norm_h, eps, out=self.tmp[:T])
            self.cat[:T, self.tmp.shape[1]:].copy_(self.tmp[:T])
            self.fc(self.cat[:T], out=out_x)
        else:
            dev = tokens.device
            emb = K.embed_gather(tokens.to(torch.int32), self.head.w["text.embed_tokens"])
            cat = torch.cat([K.rmsnorm(emb, self.norm_e, eps), K.rmsnorm(hidden.contiguous(), self.norm_h, eps)], dim=1).contiguous()
            xh = torch.empty(T * 2 * emb.shape[1], dtype=torch.float16, device=dev)
            self.fc.chunk(cat, xh, out_x)

    def _prime(self, tokens_next: torch.Tensor, hidden: torch.Tensor) -> None:
        """Writes true (t_{i+1}, h_i) pairs at the head's current position (no logits needed)."""
        T = tokens_next.numel()
        if T == 0:
            return
        head = self.head
        if T <= MAX_ROWS:
            head._stage(tokens_next, head.pos)
            self._inputs(tokens_next.to(head.device), hidden, head.buf.x[:T])
            head.buf.n_replay.zero_()
            head.forward_rows(T, want_logits=False, skip_embed=True)
            head.pos += T
        else:
            cb = head._chunk_buffers(T)
            cb["positions"][:T].copy_(torch.arange(head.pos, head.pos + T, dtype=torch.int32, device=head.device))
            self._inputs(tokens_next.to(head.device), hidden, cb["x"][:T])
            head.forward_chunk(T, want_logits=False, skip_embed=True)

    # ---- hooks called by the text model -------------------------------------------------------------
    def prefill_hook(self, ids: torch.Tensor):
        """Returns the per-chunk hook for HybridModel.prefill: primes rows whose next token is known."""
        ids_dev = ids.to(self.main.device)
        n = ids.numel()

        def hook(start: int, T: int, hidden: torch.Tensor) -> None:
            # row i of the chunk is position start + i; its next token is ids[start + i + 1] if it exists
            last = min(start + T, n - 1)
            m = last - start
            if m > 0:
                self._prime(ids_dev[start + 1:start + 1 + m], hidden[:m])
            if start + T == n:
                self.h_last.copy_(hidden[T - 1:T])
        return hook

    def after_prefill(self, ids: torch.Tensor, tok: int) -> None:
        pass          # priming happened chunk by chunk through prefill_hook

    def draft(self, anchor: int, k: int) -> List[int]:
        """k chained steps from (anchor, h_last); leaves the head positioned after the one true pair."""
        head = self.head
        k = min(k, MAX_ROWS - 1)
        start = head.pos
        tok = torch.tensor([anchor], dtype=torch.int32, device=head.device)
        hidden = self.h_last
        out: List[int] = []
        for _ in range(k):
            head._stage(tok, head.pos)
            self._inputs(tok, hidden, head.buf.x[:1])
            head.buf.n_replay.zero_()
            head.forward_rows(1, want_logits=True, skip_embed=True)
            head.pos += 1
            tok = head.buf.next_ids[:1].clone()
            if self.vocab_ids is not None:
                tok = self.vocab_ids[tok.long()]            # index in the reduced head -> token id
            hidden = head.buf.x[:1].clone()
            out.append(tok)
        head.pos = start + 1               # only the first pair (anchor, h_last) was a true pair
        self.rounds += 1
        return [int(t.item()) for t in out] if out else []

    def after_verify(self, anchor: int, drafts: List[int], emitted: List[int]) -> None:
        """Main committed rows 0..a (a = accepted drafts): re-prime positions with true pairs, keep h of row a."""
        a = len(emitted) - 1
        self.accepted += a
        hidden = self.main.buf.x
        if a > 0:
            toks = torch.tensor(drafts[:a], dtype=torch.int32, device=self.main.device)
            self._prime(toks, hidden[:a])
        self.h_last.copy_(hidden[a:a + 1])

    def acceptance(self) -> float:
        return self.accepted / max(1, self.rounds)
