"""Plain PyTorch fp32 reference of every op the CUDA kernels implement.

These functions are the numerics oracle for the kernel tests and the building blocks of the CPU
reference model.  They restate the math documented by the reference engine
(reference: docs/architecture.md:29-137, src/kernels/include/r4dx/kernels/kernels.h:42-49,199-270,
tests/kernels/test_gdn_chunk_scan.cpp:1-46) without sharing any code with it.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------
# norms / elementwise
# ---------------------------------------------------------------------------------------------
def rmsnorm_1pw(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Zero-centred RMSNorm: x * rsqrt(mean(x^2) + eps) * (1 + w), fp32 accumulate."""
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return xf * r * (1.0 + w.float())


def rmsnorm_plain(x: torch.Tensor, w: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = xf * r
    return y if w is None else y * w.float()


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return xf / torch.sqrt(xf.pow(2).sum(-1, keepdim=True) + eps)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """SwiGLU on fused rows [gate | up]."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return F.silu(g) * u


def gelu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """GeGLU on fused rows [gate | up] (tanh approximation)."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return F.gelu(g, approximate="tanh") * u


def softplus_linear_above_20(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """rms(o) * w * silu(z), per (token, head) row of width V."""
    return rmsnorm_plain(o, w, eps) * F.silu(z.float())


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x.float(), approximate="tanh")


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x.float())


# ---------------------------------------------------------------------------------------------
# rope
# ---------------------------------------------------------------------------------------------
def rope_partial_neox(x: torch.Tensor, positions: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """NeoX rope on the first ``rotary_dim`` dims of each head; pairs (i, i + rotary_dim/2).

    x: [T, H, D]; positions: [T] (int).  Remaining dims pass through.
    """
    xf = x.float()
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim)
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    cos = ang.cos().float()[:, None, :]
    sin = ang.sin().float()[:, None, :]
    a = xf[..., :half]
    b = xf[..., half:rotary_dim]
    out = xf.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = b * cos + a * sin
    return out


# ---------------------------------------------------------------------------------------------
# fp8 e4m3 round trip (paged KV cache precision)
# ---------------------------------------------------------------------------------------------
def fp8_e4m3_roundtrip(x: torch.Tensor, descale: float | torch.Tensor = 1.0) -> torch.Tensor:
    """fp8(x / descale) * descale with saturation to +-448."""
    y = (x.float() / descale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    return y * descale


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos0: int, window: int = 0,
                         key_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [T, Hq, D]; k, v: [S, Hkv, D] holding positions 0..S-1; query row t sits at q_pos0 + t.

    q head h reads KV head h // (Hq / Hkv).  ``key_limit`` [T] (absolute position, -1 = none) lets a row also see keys
    AFTER its own position up to that limit - the bidirectional mask inside an image block; the window still applies from
    below.  Returns [T, Hq, D] fp32.
    """
    T, Hq, D = q.shape
    S, Hkv, _ = k.shape
    g = Hq // Hkv
    qf = q.float().view(T, Hkv, g, D)
    kf = k.float()
    vf = v.float()
    scores = torch.einsum("thgd,shd->hgts", qf, kf) / math.sqrt(D)
    pos_q = q_pos0 + torch.arange(T)
    upper = pos_q if key_limit is None else torch.maximum(pos_q, key_limit.to(pos_q.dtype))
    mask = torch.arange(S)[None, :] > upper[:, None]
    if window > 0:          # sliding window: a row sees its last ``window`` keys only
        mask = mask | (torch.arange(S)[None, :] <= pos_q[:, None] - window)
    scores = scores.masked_fill(mask[None, None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    out = torch.einsum("hgts,shd->thgd", p, vf)
    return out.reshape(T, Hq, D)


def noncausal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Dense non-causal multi-head attention (vision tower / drafter block). q,k,v: [T|S, H, D]."""
    D = q.shape[-1]
    Hq, Hkv = q.shape[1], k.shape[1]
    g = Hq // Hkv
    qf = q.float().view(q.shape[0], Hkv, g, D)
    s = torch.einsum("thgd,shd->hgts", qf, k.float()) / math.sqrt(D)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hgts,shd->thgd", p, v.float()).reshape(q.shape[0], Hq, D)


# ---------------------------------------------------------------------------------------------
# Gated DeltaNet
# ---------------------------------------------------------------------------------------------
def causal_conv1d_silu(x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal conv (no bias) + SiLU.

    x: [T, C]; w: [C, W]; state: [W-1, C] previous inputs (oldest first) or None (zeros).
    Returns (y [T, C], new_state [W-1, C]).
    """
    T, C = x.shape
    W = w.shape[1]
    xf = x.float()
    if state is None:
        state = torch.zeros(W - 1, C, dtype=torch.float32)
    full = torch.cat([state.float(), xf], dim=0)            # [W-1+T, C]
    y = torch.zeros(T, C, dtype=torch.float32)
    for j in range(W):
        y += full[j:j + T] * w.float()[:, j][None, :]
    new_state = full[-(W - 1):].clone()
    return F.silu(y), new_state


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """g = -exp(A_log) * softplus(a + dt_bias); beta = sigmoid(b).  a, b: [T, H]."""
    g = -torch.exp(A_log.float()) * softplus_linear_above_20(a.float() + dt_bias.float())
    beta = torch.sigmoid(b.float())
    return g, beta


def gdn_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                  state: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token-recurrent gated delta rule.

    q, k: [T, Hk, K] (already L2-normalised); v: [T, H, V]; g, beta: [T, H]; state: [H, V, K] fp32.
    Per token and v head: S *= e^g; u = beta (v - S k); S += u k^T; o = S q / sqrt(K).
    """
    T, Hk, K = q.shape
    H, V = v.shape[1], v.shape[2]
    rep = H // Hk
    S = torch.zeros(H, V, K, dtype=torch.float32) if state is None else state.float().clone()
    qf = q.float().repeat_interleave(rep, dim=1)
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float()
    out = torch.zeros(T, H, V, dtype=torch.float32)
    scale = 1.0 / math.sqrt(K)
    for t in range(T):
        S = S * torch.exp(g[t].float())[:, None, None]
        Sk = torch.einsum("hvk,hk->hv", S, kf[t])
        u = beta[t].float()[:, None] * (vf[t] - Sk)
        S = S + torch.einsum("hv,hk->hvk", u, kf[t])
        out[t] = torch.einsum("hvk,hk->hv", S, qf[t]) * scale
    return out, S


def gdn_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                state: Optional[torch.Tensor], chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunked (WY) form of ``gdn_recurrent``; same arguments and results up to rounding.

    Within a chunk with cumulative gate c_i = sum_{j<=i} g_j:
      A = (I + strict_lower(diag(beta) K K^T exp(c_i - c_j)))^-1
      U = A diag(beta) (V - exp(c) * (K S0^T))         (rows: tokens)
      O = exp(c) * (Q S0^T) + tril(Q K^T exp(c_i - c_j)) U, scaled by 1/sqrt(K)
      S1 = exp(c_last) S0 + sum_i exp(c_last - c_i) u_i k_i^T
    """
    T, Hk, K = q.shape
    H, V = v.shape[1], v.shape[2]
    rep = H // Hk
    S = torch.zeros(H, V, K, dtype=torch.float32) if state is None else state.float().clone()
    qf = q.float().repeat_interleave(rep, dim=1).transpose(0, 1)     # [H, T, K]
    kf = k.float().repeat_interleave(rep, dim=1).transpose(0, 1)
    vf = v.float().transpose(0, 1)                                     # [H, T, V]
    gf = g.float().transpose(0, 1)                                     # [H, T]
    bf = beta.float().transpose(0, 1)
    out = torch.zeros(H, T, V, dtype=torch.float32)
    scale = 1.0 / math.sqrt(K)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        L = e - s
        Q, Kc, Vc = qf[:, s:e], kf[:, s:e], vf[:, s:e]
        c = gf[:, s:e].cumsum(-1)                                       # [H, L]
        decay = torch.exp(c[:, :, None] - c[:, None, :])               # [H, L, L]  e^{c_i - c_j}
        lower = torch.tril(torch.ones(L, L), diagonal=-1)
        M = (bf[:, s:e, None] * torch.einsum("hik,hjk->hij", Kc, Kc) * decay) * lower
        A = torch.linalg.inv(torch.eye(L)[None] + M)
        KS = torch.einsum("hik,hvk->hiv", Kc, S) * torch.exp(c)[:, :, None]
        U = torch.einsum("hij,hjv->hiv", A, bf[:, s:e, None] * (Vc - KS))
        QS = torch.einsum("hik,hvk->hiv", Q, S) * torch.exp(c)[:, :, None]
        QK = torch.einsum("hik,hjk->hij", Q, Kc) * decay * torch.tril(torch.ones(L, L))
        out[:, s:e] = (QS + torch.einsum("hij,hjv->hiv", QK, U)) * scale
        w_last = torch.exp(c[:, -1:, None] - c[:, :, None])            # [H, L, 1]
        S = S * torch.exp(c[:, -1])[:, None, None] + torch.einsum("hiv,hik->hvk", U * w_last, Kc)
    return out.transpose(0, 1).contiguous(), S


# ---------------------------------------------------------------------------------------------
# Hadamard
# ---------------------------------------------------------------------------------------------
def fwht(x: torch.Tensor, block: int = 128, normalize: bool = True) -> torch.Tensor:
    """Sylvester-ordered fast Walsh-Hadamard transform on each ``block`` of the last dim."""
    shp = x.shape
    y = x.float().reshape(-1, shp[-1] // block, block).clone()
    h = 1
    while h < block:
        y = y.view(y.shape[0], y.shape[1], block // (2 * h), 2, h)
        a = y[..., 0, :] + y[..., 1, :]
        b = y[..., 0, :] - y[..., 1, :]
        y = torch.stack([a, b], dim=-2).reshape(y.shape[0], y.shape[1], block)
        h *= 2
    if normalize:
        y = y / math.sqrt(block)
    return y.reshape(shp)


# ---------------------------------------------------------------------------------------------
# MoE
# ---------------------------------------------------------------------------------------------
def moe_route_sigmoid(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, renorm: bool = True,
                      scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sigmoid router: experts ranked by sigmoid(logit) + bias (ties to the lower id); weights are the unbiased sigmoids of
    the selected experts / (their sum + 1e-6), times ``scale``, rounded through bf16
    (reference: src/kernels/include/r4dx/kernels/lfm2_kernels.h:38-50)."""
    s = torch.sigmoid(logits.float())
    sel = s + bias.float() if bias is not None else s
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[..., :top_k]
    w = torch.gather(s, -1, order)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-6)
    return order, (w * scale).to(torch.bfloat16).float()


def short_conv(bcx: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor], round_bf16: bool = False):
    """Gated short convolution over [T, 3H] rows B | C | x: y = C * causal_fir(B * x) with taps ``weight`` [H, L].
    ``state`` holds the previous L - 1 rows of B * x ([L-1, H], zeros at the start).  Returns (y [T, H], new state).
    (reference: src/kernels/include/r4dx/kernels/lfm2_kernels.h:14-34)"""
    T, H3 = bcx.shape
    H, L = weight.shape
    B, C, x = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    bx = B * x
    if round_bf16:
        bx = bx.to(torch.bfloat16).float()
    prev = state if state is not None else torch.zeros(L - 1, H)
    full = torch.cat([prev, bx], 0)                       # [L-1+T, H]
    y = torch.zeros(T, H)
    for j in range(L):
        y = y + full[j:j + T] * weight[:, j][None, :]
    return C * y, full[full.shape[0] - (L - 1):].clone()


def moe_route(logits: torch.Tensor, top_k: int, renorm: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax over router logits, top-k with ties to the lower expert id.

    Returns (ids [T, k] int64 in selection order, weights [T, k] fp32, rounded through bf16).
    (reference: src/model/qwen4exp/include/r4dx/model/qwen4exp/moe_kernels.h:18-32)
    """
    p = torch.softmax(logits.float(), dim=-1)
    # stable sort keeps the lower id first among equal probabilities
    order = torch.sort(p, dim=-1, descending=True, stable=True).indices[..., :top_k]
    w = torch.gather(p, -1, order)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return order, w.to(torch.bfloat16).float()
