"""Block-diffusion drafter: a small bidirectional model that proposes up to ``block - 1`` tokens per round from
the target's intermediate residuals; the target verifies them losslessly in one window.

Context injection (after every prefill chunk and every verified window): the residuals entering the target's
``target_layers`` are concatenated, projected and normalised, ``g = rmsnorm(fc(features))``, and every drafter
layer stores ``K = rope(k_norm(W_k g))``, ``V = W_v g`` at ring slot ``position % window``.
Draft round: the block ``[anchor, <mask> x (block-1)]`` at positions ``n .. n+block-1`` runs through the layers
{rmsnorm; dynamic grouped conv; q/k/v; q/k norm; rope; bidirectional attention over ring and block; W_o; conv;
residual; rmsnorm; conv; SwiGLU; conv; residual}, then the final norm and the TARGET's lm_head; per row the top
candidates and a rank-R gate go to the host in one copy, where the selector walk (C++) picks a chain
(reference: docs/dflash2.md:26-40, 117-186; src/model/dflash_draft.h:20-45; round src/model/model.cpp:3551-3653).
Big linears are w4a16 and run on the weight-streaming kernel; the block's K/V are never stored.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import native
from ..native import c_f32, c_i64, c_int, c_ptr, register_cuda_sig, register_host_sig
from ..ops import kernels as K
from ..quant import w4a16

BF = torch.bfloat16
register_cuda_sig("r4dxb_dflash_conv", c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_ptr])
register_cuda_sig("r4dxb_dflash_norm_rope", c_int, [c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_f32, c_f32, c_ptr])
register_cuda_sig("r4dxb_dflash_attention", c_int, [c_ptr] * 6 + [c_int] * 7 + [c_ptr])
register_host_sig("r4dxb_dflash_select", c_int, [c_ptr] * 5 + [c_int, c_int, c_int, c_i64, ctypes.c_int32, c_f32, c_int, c_ptr])


@dataclass
class DflashConfig:
    layers: int = 5
    hidden: int = 5120                      # equals the target's hidden size: the target's lm_head reads the output
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 13824
    window: int = 2048
    block: int = 8
    rank: int = 256
    target_layers: Tuple[int, ...] = (6, 20, 34, 48, 62)
    mask_token_id: int = 0
    rope_theta: float = 1.0e6
    eps: float = 1e-6
    cands: int = 16
    p_min: float = 0.0
    n_min: int = 0
    group: int = 64                         # w4a16 group size of the drafter's linears


def tiny_dflash_config(hidden: int = 256, target_layers=(1, 3)) -> DflashConfig:
    return DflashConfig(layers=2, hidden=hidden, heads=4, kv_heads=2, head_dim=64, intermediate=512, window=48, block=8,
                        rank=16, target_layers=tuple(target_layers), mask_token_id=3)


_BIG = ("fc", "wq", "wk", "wv", "wo", "gate_up", "down")


def init_dflash_weights(c: DflashConfig, vocab: int, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    n = lambda *s, sc=0.05: torch.randn(*s, generator=g) * sc
    H, G = c.hidden, c.hidden // 16
    w = {"fc": n(H, len(c.target_layers) * H, sc=0.02), "inject_norm": 1 + n(H), "out_norm": 1 + n(H), "mask_embed": n(H, sc=0.5),
         "selector_hidden": n(c.rank, H), "succ": n(vocab, c.rank, sc=0.3), "pred": n(vocab, c.rank, sc=0.3)}
    for i in range(c.layers):
        p = f"layers.{i}."
        w.update({p + "in_norm": 1 + n(H), p + "post_norm": 1 + n(H), p + "q_norm": 1 + n(c.head_dim), p + "k_norm": 1 + n(c.head_dim),
                  p + "wq": n(c.heads * c.head_dim, H), p + "wk": n(c.kv_heads * c.head_dim, H), p + "wv": n(c.kv_heads * c.head_dim, H),
                  p + "wo": n(H, c.heads * c.head_dim), p + "gate_up": n(2 * c.intermediate, H), p + "down": n(H, c.intermediate)})
        for j in range(4):
            w[p + f"conv{j}.base"] = torch.cat([1 + n(1, H), n(1, H)], 0)      # per channel: [tap, H]
            w[p + f"conv{j}.dyn"] = n(2 * G, H, sc=0.02)
    return w


def synthetic_dflash_weights(c: DflashConfig, vocab: int, device="cuda", seed: int = 0) -> Dict[str, object]:
    """A random drafter created directly in the device layouts (random w4a16 nibbles for the large linears): the same
    bytes and kernels per round as a converted drafter, without a minutes-long host quantization.  Benchmarks only."""
    g = torch.Generator(device=device).manual_seed(seed)
    n = lambda *s, sc=0.05: (torch.randn(*s, generator=g, device=device) * sc)
    H, G = c.hidden, c.hidden // 16
    big = lambda N, K_, i: w4a16.random_weight(N, K_, c.group, seed=seed * 1000 + i, sigma=0.02, device=device)
    gc = torch.Generator().manual_seed(seed)
    q: Dict[str, object] = {"fc": big(H, len(c.target_layers) * H, 0), "inject_norm": (1 + n(H)).to(BF), "out_norm": (1 + n(H)).to(BF),
                            "mask_embed": n(H, sc=0.5).to(BF), "selector_hidden": n(c.rank, H).to(BF),
                            "succ": (torch.randn(vocab, c.rank, generator=gc) * 0.3).contiguous(),
                            "pred": (torch.randn(vocab, c.rank, generator=gc) * 0.3).contiguous()}
    for i in range(c.layers):
        p = f"layers.{i}."
        q.update({p + "in_norm": (1 + n(H)).to(BF), p + "post_norm": (1 + n(H)).to(BF), p + "q_norm": (1 + n(c.head_dim)).to(BF),
                  p + "k_norm": (1 + n(c.head_dim)).to(BF),
                  p + "wq": big(c.heads * c.head_dim, H, 10 * i + 1), p + "wk": big(c.kv_heads * c.head_dim, H, 10 * i + 2),
                  p + "wv": big(c.kv_heads * c.head_dim, H, 10 * i + 3), p + "wo": big(H, c.heads * c.head_dim, 10 * i + 4),
                  p + "gate_up": big(2 * c.intermediate, H, 10 * i + 5), p + "down": big(H, c.intermediate, 10 * i + 6)})
        for j in range(4):
            q[p + f"conv{j}.base"] = torch.cat([1 + n(1, H), n(1, H)], 0).to(BF)
            q[p + f"conv{j}.dyn"] = n(2 * G, H, sc=0.02).to(BF)
    return q


def quantize_dflash_weights(c: DflashConfig, w: Dict[str, torch.Tensor]):
    """(device-format dict, fp32 dict holding exactly the values the device will use)."""
    q, dq = {}, {}
    for k, v in w.items():
        if k.split(".")[-1] in _BIG:
            q[k] = w4a16.quantize(v, c.group)
            dq[k] = w4a16.dequantize(q[k])
        elif k in ("succ", "pred"):
            q[k] = dq[k] = v.float().contiguous()
        else:
            q[k] = v.to(BF)
            dq[k] = q[k].float()
    return q, dq


# ---------------------------------------------------------------- fp32 restatement ----------------------------
def _r(t):
    return t.to(BF).float()


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope_full(x, pos, theta):
    D = x.shape[-1]
    half = D // 2
    inv = theta ** (-(torch.arange(half).float() * 2.0 / D))
    ang = pos.float()[:, None] * inv
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    return torch.cat([x[..., :half] * c - x[..., half:] * s, x[..., half:] * c + x[..., :half] * s], -1)


def _conv_ref(h, base, dyn_w):
    """Two-tap causal conv over the block's rows: a per-channel base kernel [2, H] plus a per-row dynamic part shared by
    groups of 16 channels (dyn_w [2G, H], G = H / 16)."""
    G = dyn_w.shape[0] // 2
    dyn = _r(h @ dyn_w.T)                                   # [T, 2G]
    a0 = base[0] + dyn[:, :G].repeat_interleave(16, -1)
    a1 = base[1] + dyn[:, G:].repeat_interleave(16, -1)
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return _r(a0 * h + a1 * prev)


class DflashOracle:
    """CPU restatement with bf16 rounding at the device path's rounding points."""

    def __init__(self, c: DflashConfig, w: Dict[str, torch.Tensor], embed: torch.Tensor, lm_head: torch.Tensor):
        self.c, self.w, self.embed, self.lm_head = c, w, embed.float(), lm_head.float()
        self.ring_k = [dict() for _ in range(c.layers)]
        self.ring_v = [dict() for _ in range(c.layers)]

    def inject(self, feats: torch.Tensor, pos0: int) -> None:
        """feats fp32 [T, F * H] (bf16-representable)."""
        c, w = self.c, self.w
        g = _r(_rms(_r(feats @ w["fc"].T), w["inject_norm"], c.eps))
        pos = torch.arange(pos0, pos0 + feats.shape[0])
        for i in range(c.layers):
            p = f"layers.{i}."
            k = _r(g @ w[p + "wk"].T).view(-1, c.kv_heads, c.head_dim)
            k = _r(_rope_full(_rms(k, w[p + "k_norm"], c.eps), pos, c.rope_theta))
            v = _r(g @ w[p + "wv"].T).view(-1, c.kv_heads, c.head_dim)
            for j, pp in enumerate(pos.tolist()):
                self.ring_k[i][pp], self.ring_v[i][pp] = k[j], v[j]

    def draft_logits(self, anchor: int, n: int, valid_from: int = 0):
        c, w = self.c, self.w
        B = c.block
        x = torch.stack([self.embed[anchor]] + [w["mask_embed"]] * (B - 1))
        pos = torch.arange(n, n + B)
        lo = max(valid_from, n - c.window)
        for i in range(c.layers):
            p = f"layers.{i}."
            h = _r(_rms(x, w[p + "in_norm"], c.eps))
            h = _conv_ref(h, w[p + "conv0.base"], w[p + "conv0.dyn"])
            q = _r(h @ w[p + "wq"].T).view(B, c.heads, c.head_dim)
            k = _r(h @ w[p + "wk"].T).view(B, c.kv_heads, c.head_dim)
            v = _r(h @ w[p + "wv"].T).view(B, c.kv_heads, c.head_dim)
            q = _r(_rope_full(_rms(q, w[p + "q_norm"], c.eps), pos, c.rope_theta))
            k = _r(_rope_full(_rms(k, w[p + "k_norm"], c.eps), pos, c.rope_theta))
            ks = [self.ring_k[i][pp] for pp in range(lo, n)] + list(k)
            vs = [self.ring_v[i][pp] for pp in range(lo, n)] + list(v)
            Kt, Vt = torch.stack(ks), torch.stack(vs)                     # [S, Hkv, D]
            rep = c.heads // c.kv_heads
            att = torch.einsum("qhd,khd->hqk", q, Kt.repeat_interleave(rep, 1)) / math.sqrt(c.head_dim)
            o = _r(torch.einsum("hqk,khd->qhd", att.softmax(-1), Vt.repeat_interleave(rep, 1))).reshape(B, -1)
            a = _conv_ref(_r(o @ w[p + "wo"].T), w[p + "conv1.base"], w[p + "conv1.dyn"])
            x = _r(x + a)
            h = _conv_ref(_r(_rms(x, w[p + "post_norm"], c.eps)), w[p + "conv2.base"], w[p + "conv2.dyn"])
            gu = _r(h @ w[p + "gate_up"].T)
            I = c.intermediate
            m = _r(F.silu(gu[:, :I]) * gu[:, I:])
            d = _conv_ref(_r(m @ w[p + "down"].T), w[p + "conv3.base"], w[p + "conv3.dyn"])
            x = _r(x + d)
        xo = _r(_rms(x, w["out_norm"], c.eps))
        return xo @ self.lm_head.T, xo


def save_dflash(path: str, c: DflashConfig, w: Dict[str, torch.Tensor]) -> None:
    """fp32/bf16 source weights + config in one torch file (quantized at load)."""
    import dataclasses
    torch.save({"config": dataclasses.asdict(c), "weights": w}, path)


def load_dflash(path: str):
    d = torch.load(path, map_location="cpu", weights_only=False)
    cfgd = dict(d["config"])
    cfgd["target_layers"] = tuple(cfgd["target_layers"])
    c = DflashConfig(**cfgd)
    q, _ = quantize_dflash_weights(c, d["weights"])
    return c, q


def select_chain(c: DflashConfig, cand: torch.Tensor, unary: torch.Tensor, gate: torch.Tensor, succ: torch.Tensor,
                 pred: torch.Tensor, anchor: int) -> List[int]:
    """Host selector walk (C++): cand int32 [B, cands], unary / gate fp32, codebooks fp32 [vocab, rank]."""
    cand, unary, gate = cand.contiguous(), unary.contiguous(), gate.contiguous()
    out = torch.zeros(cand.shape[0], dtype=torch.int32)
    n = native.host().r4dxb_dflash_select(cand.data_ptr(), unary.data_ptr(), gate.data_ptr(), succ.data_ptr(), pred.data_ptr(),
                                          cand.shape[0], cand.shape[1], gate.shape[1], succ.shape[0], int(anchor),
                                          c.p_min, c.n_min, out.data_ptr())
    return out[:max(n, 0)].tolist()


# ---------------------------------------------------------------- device drafter ------------------------------
class DflashDrafter:
    kind = "dflash"

    def __init__(self, main, c: DflashConfig, qweights: Dict[str, object]):
        self.main, self.c = main, c
        dev = main.device
        self.w = {k: (v.to(dev) if k not in ("succ", "pred") else v) for k, v in qweights.items()}
        self.succ, self.pred = qweights["succ"], qweights["pred"]
        z = lambda *s: torch.zeros(*s, dtype=BF, device=dev)
        self.ring_k = [z(c.window, c.kv_heads, c.head_dim) for _ in range(c.layers)]
        self.ring_v = [z(c.window, c.kv_heads, c.head_dim) for _ in range(c.layers)]
        self.valid_from, self.frontier = 0, 0
        self.rounds, self.proposed, self.accepted = 0, 0, 0
        main.enable_capture(c.target_layers, 8)
        self._L = native.cuda()

    def reset(self) -> None:
        self.valid_from, self.frontier = 0, 0

    def _lin(self, name: str, x: torch.Tensor) -> torch.Tensor:
        """w4a16 product: the weight-streaming kernel up to 8 rows, the tensor-core kernel above."""
        w = self.w[name]
        T = x.shape[0]
        tmax = 1 if T == 1 else (2 if T == 2 else (4 if T <= 4 else 8))       # rows the streaming kernel stages in shared memory
        if T > 8 or tmax * w.K * 2 > 200 * 1024:
            return K.linear_tc(w, x)
        out = torch.empty(T, w.N, dtype=BF, device=x.device)
        K.w4a16_gemv(w, x.contiguous(), out_f32=False, out=out)
        return out

    def _norm_rope(self, x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, heads: int) -> None:
        c = self.c
        rc = self._L.r4dxb_dflash_norm_rope(x.data_ptr(), w.data_ptr(), pos.data_ptr(), x.shape[0], heads, c.head_dim,
                                            c.rope_theta, c.eps, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc

    def _conv(self, h: torch.Tensor, name: str) -> torch.Tensor:
        dyn = K.linear_tc(self.w[name + ".dyn"], h)       # [T, 2G]
        out = torch.empty_like(h)
        rc = self._L.r4dxb_dflash_conv(h.data_ptr(), self.w[name + ".base"].data_ptr(), dyn.data_ptr(), out.data_ptr(),
                                       h.shape[0], h.shape[1], torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
        return out

    def inject(self, feats: torch.Tensor, pos0: int, T: int) -> None:
        """feats: captured residuals bf16 [F, >=T, H] of target rows at positions pos0 .. pos0+T-1."""
        c = self.c
        if pos0 != self.frontier:
            raise RuntimeError(f"drafter frontier {self.frontier} != injected position {pos0}")
        cat = feats[:, :T].permute(1, 0, 2).reshape(T, -1).contiguous()
        g = K.rmsnorm(self._lin("fc", cat), self.w["inject_norm"], c.eps, zero_centered=False)
        pos = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=g.device)
        slots = (pos.long() % c.window)
        for i in range(c.layers):
            p = f"layers.{i}."
            k = self._lin(p + "wk", g)
            self._norm_rope(k, self.w[p + "k_norm"], pos, c.kv_heads)
            v = self._lin(p + "wv", g)
            # a chunk longer than the window keeps its last `window` rows
            keep = slice(max(0, T - c.window), T)
            self.ring_k[i][slots[keep]] = k.view(T, c.kv_heads, c.head_dim)[keep]
            self.ring_v[i][slots[keep]] = v.view(T, c.kv_heads, c.head_dim)[keep]
        self.frontier = pos0 + T

    def draft_rows(self, anchor: int):
        """Runs the block; returns (logits fp32 [B, V], final hidden bf16 [B, H])."""
        c, w, main = self.c, self.w, self.main
        B, n = c.block, self.frontier
        dev = main.device
        x = torch.cat([main.w["text.embed_tokens"][anchor:anchor + 1], w["mask_embed"].view(1, -1).expand(B - 1, -1)], 0).contiguous()
        pos = torch.arange(n, n + B, dtype=torch.int32, device=dev)
        lo = max(self.valid_from, n - c.window)
        st = torch.cuda.current_stream().cuda_stream
        for i in range(c.layers):
            p = f"layers.{i}."
            h = self._conv(K.rmsnorm(x, w[p + "in_norm"], c.eps, zero_centered=False), p + "conv0")
            q, k, v = self._lin(p + "wq", h), self._lin(p + "wk", h), self._lin(p + "wv", h)
            self._norm_rope(q, w[p + "q_norm"], pos, c.heads)
            self._norm_rope(k, w[p + "k_norm"], pos, c.kv_heads)
            o = torch.empty(B, c.heads * c.head_dim, dtype=BF, device=dev)
            rc = self._L.r4dxb_dflash_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), self.ring_k[i].data_ptr(),
                                                self.ring_v[i].data_ptr(), o.data_ptr(), B, c.heads, c.kv_heads, c.head_dim,
                                                c.window, lo, n, st)
            assert rc == 0, rc
            x = K.residual_add(x, self._conv(self._lin(p + "wo", o), p + "conv1"))
            h = self._conv(K.rmsnorm(x, w[p + "post_norm"], c.eps, zero_centered=False), p + "conv2")
            m = K.silu_mul(self._lin(p + "gate_up", h))
            x = K.residual_add(x, self._conv(self._lin(p + "down", m), p + "conv3"))
        xo = K.rmsnorm(x, w["out_norm"], c.eps, zero_centered=False)
        logits = torch.empty(B, main.cfg.vocab_shard_size, dtype=torch.float32, device=dev)
        main.lin["lm_head"](xo, out=logits)
        return logits, xo

    # ---- drafter protocol used by runtime.text_model.LocalTextModel --------------------------------------
    def prefill_hook(self, ids: torch.Tensor):
        state = {"s": self.frontier}

        def hook(start: int, T: int, _hidden: torch.Tensor) -> None:
            self.inject(self.main.captured, state["s"], T)
            state["s"] += T

        return hook

    def after_prefill(self, ids: torch.Tensor, tok: int) -> None:
        pass

    def after_verify(self, anchor: int, drafts: List[int], emitted: List[int]) -> None:
        self.accepted += len(emitted) - 1
        self.inject(self.main.captured, self.frontier, len(emitted))

    def acceptance(self) -> float:
        return self.accepted / max(1, self.rounds)

    def draft(self, anchor: int, k: int = 7) -> List[int]:
        c = self.c
        logits, xo = self.draft_rows(anchor)
        vals, ids, _ = K.topk_lse(logits, 64)
        gate = K.linear_tc(self.w["selector_hidden"], xo, out_f32=True)
        packed = torch.cat([vals[:, :c.cands].reshape(-1), ids[:, :c.cands].reshape(-1).float(), gate.reshape(-1)]).cpu()   # one copy
        nb = c.block * c.cands
        unary, cand, g = packed[:nb].view(c.block, c.cands), packed[nb:2 * nb].view(c.block, c.cands).to(torch.int32), packed[2 * nb:].view(c.block, -1)
        self.rounds += 1
        out = select_chain(c, cand, unary, g.contiguous(), self.succ, self.pred, anchor)
        out = out[:min(k, 7)]
        self.proposed += len(out)
        return out

    # ---- speculative generation on top of the target's verify window -------------------------------------
    def generate(self, prompt: torch.Tensor, n_tokens: int) -> List[int]:
        main = self.main
        main.reset()
        self.reset()
        tok = main.prefill(prompt, hook=self.prefill_hook(prompt))
        out = [tok]
        while len(out) < n_tokens:
            drafts = self.draft(out[-1])
            emitted = main.verify_window(out[-1], drafts)
            self.after_verify(out[-1], drafts, emitted)
            out += emitted
        return out[:n_tokens]
