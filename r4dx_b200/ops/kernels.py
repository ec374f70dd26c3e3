"""Python face of the sm_100a kernel library: tensor checks + ctypes calls on the current stream.

Every function requires CUDA tensors and the in-tree ``libr4dxb_cuda.so``; there is no eager
fallback (a missing library raises).  Reference numerics for each op live in ``ops/reference.py``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from .. import native
from ..native import c_f32, c_i64, c_int, c_ptr, register_cuda_sig
from ..quant.trellis import TrellisWeight
from ..quant.w4a16 import W4Weight, W8Weight

_I = c_int
_P = c_ptr
_F = c_f32

register_cuda_sig("r4dxb_launch_count", ctypes.c_ulonglong, [])
register_cuda_sig("r4dxb_launch_count_reset", None, [])
register_cuda_sig("r4dxb_embed_gather_bf16", _I, [_P, _P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_rmsnorm_bf16", _I, [_P, _P, _P, _I, _I, _F, _I, _P])
register_cuda_sig("r4dxb_add_rmsnorm_bf16", _I, [_P, _P, _P, _P, _I, _I, _F, _I, _P])
register_cuda_sig("r4dxb_layernorm_bf16", _I, [_P, _P, _P, _P, _I, _I, _F, _P])
register_cuda_sig("r4dxb_silu_mul_bf16", _I, [_P, _P, _I, _I, _P])
register_cuda_sig("r4dxb_residual_add_bf16", _I, [_P, _P, ctypes.c_longlong, _P])
register_cuda_sig("r4dxb_bias_act_bf16", _I, [_P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemv", _I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemv_ex", _I, [_P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_w4a16_gemv", _I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_bf16_gemv", _I, [_P, _P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_bf16_gemv_norm", _I, [_P, _P, _P, _F, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_argmax_rows", _I, [_P, _I, _I, _I, _I, _P, _P, _P, _P])
register_cuda_sig("r4dxb_gdn_decode", _I, [_P] * 15 + [_I, _I, _I, _I, _F, _P])
register_cuda_sig("r4dxb_attn_precore", _I, [_P] * 11 + [_I, _I, _I, _I, _I, _F, _F, _I, _P])
register_cuda_sig("r4dxb_attn_decode", _I, [_P] * 10 + [_I, _I, _I, _I, _I, _I, _P])


class KernelError(RuntimeError):
    pass


def _lib():
    return native.cuda()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, name: str) -> None:
    if code != 0:
        raise KernelError(f"{name} failed with code {code}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def _req(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def launch_count() -> int:
    return int(_lib().r4dxb_launch_count())


def launch_count_reset() -> None:
    _lib().r4dxb_launch_count_reset()


BF = torch.bfloat16

NORM_ZERO_CENTERED = 1
NORM_NO_WEIGHT = 2


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(ids, torch.int32, "ids"); _req(table, BF, "table")
    T, (V, H) = ids.numel(), table.shape
    out = out if out is not None else torch.empty(T, H, dtype=BF, device=ids.device)
    _check(_lib().r4dxb_embed_gather_bf16(_p(ids), _p(table), _p(out), T, H, V, _stream()), "embed_gather")
    return out


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float = 1e-6, zero_centered: bool = True,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(x, BF, "x")
    H = x.shape[-1]
    T = x.numel() // H
    out = out if out is not None else torch.empty_like(x)
    mode = (NORM_ZERO_CENTERED if zero_centered else 0) | (NORM_NO_WEIGHT if w is None else 0)
    _check(_lib().r4dxb_rmsnorm_bf16(_p(x), _p(w), _p(out), T, H, eps, mode, _stream()), "rmsnorm")
    return out


def add_rmsnorm(res: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
                zero_centered: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res += delta in place (bf16); returns rmsnorm(res)."""
    _req(res, BF, "res"); _req(delta, BF, "delta")
    H = res.shape[-1]
    T = res.numel() // H
    out = out if out is not None else torch.empty_like(res)
    mode = NORM_ZERO_CENTERED if zero_centered else 0
    _check(_lib().r4dxb_add_rmsnorm_bf16(_p(res), _p(delta), _p(w), _p(out), T, H, eps, mode, _stream()), "add_rmsnorm")
    return out


register_cuda_sig("r4dxb_norm_add_bf16", _I, [_P, _P, _P, _I, _I, _F, _P])


def norm_add(res: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """res += rmsnorm(delta) * (1 + w), in place (sandwich-norm residual update)."""
    _req(res, BF, "res"); _req(delta, BF, "delta")
    H = res.shape[-1]
    _check(_lib().r4dxb_norm_add_bf16(_p(res), _p(delta), _p(w), res.numel() // H, H, eps, _stream()), "norm_add")
    return res


def layernorm(x, w, b, eps: float = 1e-6):
    _req(x, BF, "x")
    H = x.shape[-1]
    out = torch.empty_like(x)
    _check(_lib().r4dxb_layernorm_bf16(_p(x), _p(w), _p(b), _p(out), x.numel() // H, H, eps, _stream()), "layernorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(gate_up, BF, "gate_up")
    I = gate_up.shape[-1] // 2
    T = gate_up.numel() // (2 * I)
    out = out if out is not None else torch.empty(*gate_up.shape[:-1], I, dtype=BF, device=gate_up.device)
    _check(_lib().r4dxb_silu_mul_bf16(_p(gate_up), _p(out), T, I, _stream()), "silu_mul")
    return out


def residual_add(res: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _req(res, BF, "res"); _req(delta, BF, "delta")
    _check(_lib().r4dxb_residual_add_bf16(_p(res), _p(delta), res.numel(), _stream()), "residual_add")
    return res


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], act: int = 0) -> torch.Tensor:
    _req(x, BF, "x")
    H = x.shape[-1]
    _check(_lib().r4dxb_bias_act_bf16(_p(x), _p(bias), x.numel() // H, H, act, _stream()), "bias_act")
    return x


def _load_tuning() -> dict:
    """Measured exceptions to the two heuristics below (written by ``utils/tune_gemm.py``); ``R4DXB_TUNING=0`` ignores it."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuning_table.json")
    if os.environ.get("R4DXB_TUNING", "1") == "0" or not os.path.exists(path):
        return {}
    import json
    try:
        t = json.load(open(path))
    except (OSError, ValueError):
        return {}
    out = {("gemv",) + tuple(k.split("x")): v["ksplit"] for k, v in t.get("gemv", {}).items()}
    out.update({("gemm",) + tuple(k.split("x")): v["tn"] for k, v in t.get("gemm", {}).items()})
    return out


TUNING = _load_tuning()


def pick_ksplit(N: int, K: int, target_ctas: int = int(os.environ.get("R4DXB_KSPLIT_TARGET", "296")), rows: int = 1) -> int:
    """Smallest cluster split (1/2/4/8) that gives at least ``target_ctas`` CTAs; every CTA needs at least one 128-wide
    K block, and a block count the split does not divide is dealt out unevenly (17 blocks over 8 CTAs: 2 or 3 each).
    (In isolation the widest split is the fastest on every 27B shape, by up to 5 us; inside a decode step, where
    the RMSNorm prologue is repeated per K slice and neighbouring kernels overlap, it measured slower:
    90.3 vs 92.2 tok/s.)"""
    kblocks = K // 128
    hit = TUNING.get(("gemv", str(N), str(K), "1" if rows == 1 else "n")) if target_ctas == 296 else None
    if hit is not None and kblocks >= hit:
        return hit
    best = 1
    for s in (1, 2, 4, 8):
        if kblocks < s:
            break
        best = s
        if (N // 128) * s >= target_ctas:
            break
    return best


_STATUS = {}


def gemm_status(device) -> torch.Tensor:
    """Device word that a tcgen05 kernel sets when one of its bounded waits runs out."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_gemm_status(device) -> None:
    code = int(gemm_status(device).item())
    if code:
        gemm_status(device).zero_()
        raise KernelError(f"tcgen05 GEMM gave up in a bounded wait (role code {code})")


PRO_NONE, PRO_RMSNORM, PRO_SILU_MUL, PRO_GELU_MUL = 0, 1, 2, 3

register_cuda_sig("r4dxb_trellis_gemv_mma", _I, [_P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _P, _P])

# Which weight-streaming kernel serves T <= 8 rows: "simt" = CUDA-core decode + fp16 FMA (default: the faster one
# on the 27B shapes, 56-62 us vs 66-68 us on gate_up), "mma" = code values written to tensor memory and contracted
# by tcgen05.mma kind::f16 (trellis_gemv_mma.cu).
# "auto" (the default) takes the CUDA-core kernel for one to three rows and the tensor-memory kernel where it measured faster:
# from six rows everywhere (gate_up at 8 rows: 95 against 121 us, down 69 against 97 us) and from four rows on the two large
# MLP products (80 against 83 us, 57 against 67 us).
GEMV_IMPL = os.environ.get("R4DXB_GEMV", "auto")


def set_gemv_impl(name: str) -> None:
    global GEMV_IMPL
    if name not in ("mma", "simt", "auto"):
        raise KernelError(f"unknown weight-streaming kernel {name!r}")
    GEMV_IMPL = name


def use_mma_gemv(T: int, N: int, K: int, ksplit: int) -> bool:
    """Whether a product of T rows goes to the tensor-memory weight-streaming kernel (it needs an even K split of at most
    6144 columns per CTA)."""
    if GEMV_IMPL == "simt" or K // ksplit > 6144 or (K // 128) % ksplit:
        return False
    if GEMV_IMPL == "mma":
        return True
    return T >= 6 or (T >= 4 and N * K >= (1 << 26))


def trellis_gemv(w: TrellisWeight, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, ksplit: Optional[int] = None, prologue: int = PRO_NONE,
                 norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """y[T, N] = trellis linear of act(x) (T <= 8), optionally + residual (may alias out).

    prologue PRO_RMSNORM: x is the residual stream [T, K], act = zero-centred RMSNorm with ``norm_w``;
    PRO_SILU_MUL: x is fused [gate | up] rows [T, 2K].
    """
    _req(x, BF, "x")
    T = x.numel() // (2 * w.K if prologue in (PRO_SILU_MUL, PRO_GELU_MUL) else w.K)
    out = out if out is not None else torch.empty(T, w.N, dtype=BF, device=x.device)
    ks = ksplit or pick_ksplit(w.N, w.K)
    if use_mma_gemv(T, w.N, w.K, ks):
        _check(_lib().r4dxb_trellis_gemv_mma(_p(w.words), _p(w.suh), _p(w.svh), _p(x), _p(out), _p(residual), _p(norm_w), eps,
                                             prologue, T, w.N, w.K, w.kb, ks, _p(gemm_status(x.device)), _stream()),
               "trellis_gemv_mma")
        return out
    _check(_lib().r4dxb_trellis_gemv_ex(_p(w.words), _p(w.suh), _p(w.svh), _p(x), _p(out), _p(residual), _p(norm_w), eps,
                                        prologue, T, w.N, w.K, w.kb, ks, _stream()), "trellis_gemv")
    return out


register_cuda_sig("r4dxb_trellis_gemv_siblings", _I, [_I, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _P])


class SiblingGroup:
    """Trellis weights that read the same rows through the same prologue (q / k / v; the GDN qkv / z pair), served by
    one launch of the weight-streaming kernel.  Holds the pointer tables so a call allocates nothing."""

    def __init__(self, weights: Sequence[TrellisWeight]):
        w0 = weights[0]
        if not (2 <= len(weights) <= 3) or any(w.K != w0.K or w.kb != w0.kb for w in weights):
            raise KernelError("siblings must be 2 or 3 trellis weights of one K and one bit width")
        self.weights = list(weights)
        self.K, self.kb = w0.K, w0.kb
        arr = lambda vals: (ctypes.c_void_p * len(vals))(*vals)
        self._words = arr([w.words.data_ptr() for w in weights])
        self._suh = arr([w.suh.data_ptr() for w in weights])
        self._svh = arr([w.svh.data_ptr() for w in weights])
        self._n = (ctypes.c_int * len(weights))(*[w.N for w in weights])
        self.ksplit = pick_ksplit(sum(w.N for w in weights), w0.K)
        self._outs = {}

    def __call__(self, x: torch.Tensor, outs: Sequence[torch.Tensor], prologue: int = PRO_NONE,
                 norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6) -> None:
        _req(x, BF, "x")
        T = x.numel() // (2 * self.K if prologue in (PRO_SILU_MUL, PRO_GELU_MUL) else self.K)
        key = tuple(o.data_ptr() for o in outs)
        y = self._outs.get(key)
        if y is None:
            y = self._outs[key] = (ctypes.c_void_p * len(outs))(*key)
        _check(_lib().r4dxb_trellis_gemv_siblings(len(self.weights), self._words, self._suh, self._svh, y, self._n, _p(x),
                                                  _p(norm_w), eps, prologue, T, self.K, self.kb, self.ksplit, _stream()),
               "trellis_gemv_siblings")


def w4a16_gemv(w: W4Weight, x: torch.Tensor, out_f32: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(x, BF, "x")
    T = x.numel() // w.K
    if out is None:
        out = torch.empty(T, w.N, dtype=torch.float32 if out_f32 else BF, device=x.device)
    _check(_lib().r4dxb_w4a16_gemv(_p(w.wq), _p(w.wsz), _p(x), _p(out), T, w.N, w.K, w.group, 1 if out_f32 else 0,
                                   _stream()), "w4a16_gemv")
    return out


def bf16_gemv(W: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(W, BF, "W"); _req(x, BF, "x")
    N, K = W.shape
    T = x.numel() // K
    out = out if out is not None else torch.empty(T, N, dtype=torch.float32, device=x.device)
    _check(_lib().r4dxb_bf16_gemv(_p(W), _p(x), _p(out), T, N, K, _stream()), "bf16_gemv")
    return out


def bf16_gemv_norm(W: torch.Tensor, x: torch.Tensor, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] = rmsnorm(x) W^T for T <= 8 rows of the residual stream (fp32 out)."""
    _req(W, BF, "W"); _req(x, BF, "x")
    N, K = W.shape
    T = x.numel() // K
    _check(_lib().r4dxb_bf16_gemv_norm(_p(W), _p(x), _p(norm_w), eps, _p(out), T, N, K, _stream()), "bf16_gemv_norm")
    return out


def argmax_rows(logits: torch.Tensor, id_offset: int = 0, out_ids: Optional[torch.Tensor] = None,
                out_vals: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None):
    T, V = logits.shape
    is_f32 = logits.dtype == torch.float32
    if not is_f32:
        _req(logits, BF, "logits")
    dev = logits.device
    out_ids = out_ids if out_ids is not None else torch.empty(T, dtype=torch.int32, device=dev)
    out_vals = out_vals if out_vals is not None else torch.empty(T, dtype=torch.float32, device=dev)
    scratch = scratch if scratch is not None else torch.empty(2 * T * 256, dtype=torch.float32, device=dev)
    _check(_lib().r4dxb_argmax_rows(_p(logits), 1 if is_f32 else 0, T, V, id_offset, _p(out_ids), _p(out_vals),
                                    _p(scratch), _stream()), "argmax_rows")
    return out_ids, out_vals


register_cuda_sig("r4dxb_gdn_decode_ab", _I, [_P] * 6 + [_I, _F] + [_P] * 12 + [_I, _I, _I, _I, _F, _P])


def gdn_decode(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, log_u, log_k, log_eg, positions,
               n_replay, out, T: int, H: int, Hk: int, D: int, eps: float = 1e-6, ab_w=None, x=None, in_norm_w=None,
               in_eps: float = 1e-6) -> torch.Tensor:
    """With ``ab_w`` ([2H, K] bf16) the a / b projections of the residual rows ``x`` (input RMSNorm ``in_norm_w``) are
    computed inside the kernel and ``ab`` is not read."""
    if ab_w is not None:
        _check(_lib().r4dxb_gdn_decode_ab(_p(mixed), _p(z), _p(ab), _p(ab_w), _p(x), _p(in_norm_w), ab_w.shape[1], in_eps,
                                          _p(conv_w), _p(A_log), _p(dt_bias), _p(norm_w), _p(ring), _p(state), _p(log_u),
                                          _p(log_k), _p(log_eg), _p(positions), _p(n_replay), _p(out), T, H, Hk, D, eps,
                                          _stream()), "gdn_decode_ab")
        return out
    _check(_lib().r4dxb_gdn_decode(_p(mixed), _p(z), _p(ab), _p(conv_w), _p(A_log), _p(dt_bias), _p(norm_w), _p(ring),
                                   _p(state), _p(log_u), _p(log_k), _p(log_eg), _p(positions), _p(n_replay), _p(out),
                                   T, H, Hk, D, eps, _stream()), "gdn_decode")
    return out


def attn_precore(qg, k, v, q_norm, k_norm, k_descale, v_descale, positions, block_table, q_out, cache, T: int,
                 Hq: int, Hkv: int, D: int, rotary_dim: int, theta: float, eps: float = 1e-6, q_stride: int = 0):
    """q_norm / k_norm None: no per-head normalisation; q_stride 0: qg rows are q|gate pairs (2D per head)."""
    _check(_lib().r4dxb_attn_precore(_p(qg), _p(k), _p(v), _p(q_norm), _p(k_norm), _p(k_descale), _p(v_descale),
                                     _p(positions), _p(block_table), _p(q_out), _p(cache), T, Hq, Hkv, D, rotary_dim,
                                     theta, eps, q_stride, _stream()), "attn_precore")
    return q_out


def attn_decode(q, qg, cache, block_table, positions, k_descale, v_descale, part_acc, part_ml, out, T: int, Hq: int,
                Hkv: int, D: int, splits: int, gated: bool = True, window: int = 0):
    """``window`` > 0: every row sees only its last ``window`` keys (sliding-window layers)."""
    _check(_lib().r4dxb_attn_decode(_p(q), _p(qg), _p(cache), _p(block_table), _p(positions), _p(k_descale),
                                    _p(v_descale), _p(part_acc), _p(part_ml), _p(out), T, Hq, Hkv, D, splits,
                                    (1 if gated else 0) | (window << 1), _stream()), "attn_decode")
    return out


register_cuda_sig("r4dxb_trellis_input", _I, [_P, _P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemm", _I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P])

def trellis_input(x: torch.Tensor, suh: torch.Tensor, out: Optional[torch.Tensor] = None, fused_silu_mul: bool = False,
                  gelu: bool = False) -> torch.Tensor:
    """fp16 H128(suh * x) rows; with ``fused_silu_mul`` x is act(gate) * up of fused [T, 2K] rows (SiLU, or tanh-GELU with ``gelu``)."""
    _req(x, BF, "x")
    K_ = suh.numel()
    T = x.numel() // (2 * K_ if fused_silu_mul else K_)
    out = out if out is not None else torch.empty(T, K_, dtype=torch.float16, device=x.device)
    mode = (2 if gelu else 1) if fused_silu_mul else 0
    _check(_lib().r4dxb_trellis_input(_p(x), _p(suh), _p(out), T, K_, mode, _stream()), "trellis_input")
    return out


_TILE_COST = {128: 0.60, 256: 0.62, 512: 1.0}   # relative time of one CTA's K loop (decode-bound below 512 columns)


def pick_token_tile(T: int, N: int = 0, K: int = 0) -> int:
    """Token-tile width of the tensor-core GEMM: the smallest tile that covers T below 512 rows; above,
    the width whose CTA count wastes the fewest of the 148 SMs' waves (one CTA per SM)."""
    for tn in (16, 32, 64, 128):
        if T <= tn:
            return tn
    hit = TUNING.get(("gemm", str(N), str(K), str(T))) if K else None
    if hit is not None:
        return hit
    if T < 512:
        return 256 if T > 192 else 128      # measured at 256 rows: one 256-row tile per CTA is 1.6-1.7x faster than two 128-row CTAs
    if N <= 0:
        return 512 if T >= 1024 else 256
    best, best_cost = 256, None
    for tn, c in _TILE_COST.items():
        ctas = (N // 128) * ((T + tn - 1) // tn)
        cost = ((ctas + 147) // 148) * c
        if best_cost is None or cost < best_cost - 1e-9 or (abs(cost - best_cost) < 1e-9 and tn > best):
            best, best_cost = tn, cost
    return best


def trellis_gemm(w: TrellisWeight, xh: torch.Tensor, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, tn: Optional[int] = None) -> torch.Tensor:
    """y[T, N] from input-transformed xh[T, K] on the tcgen05 path."""
    _req(xh, torch.float16, "xh")
    T = xh.numel() // w.K
    out = out if out is not None else torch.empty(T, w.N, dtype=BF, device=xh.device)
    tn = tn or pick_token_tile(T, w.N, w.K)
    _check(_lib().r4dxb_trellis_gemm(_p(w.words), _p(w.svh), _p(xh), _p(out), _p(residual), T, w.N, w.K, w.kb, tn,
                                     _p(gemm_status(xh.device)), _stream()), "trellis_gemm")
    return out


register_cuda_sig("r4dxb_quantize_rows_e4m3", _I, [_P, _P, _P, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemm_f8", _I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P])

# Opt-in 8-bit prefill products (R4DXB_PREFILL_F8=1): e4m3 activations (one scale per row) times e4m3 code values.  Half the
# activation bytes per product and the 8-bit tensor-core rate; the rounding of both operands to three mantissa bits shows
# in the logits (see the KL figures in the design notes), so the 16-bit path stays the default.
PREFILL_F8 = os.environ.get("R4DXB_PREFILL_F8", "0") == "1"


def set_prefill_f8(on: bool) -> None:
    global PREFILL_F8
    PREFILL_F8 = bool(on)


def quantize_rows_e4m3(xh: torch.Tensor, xq: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None):
    """fp16 rows [T, K] -> (e4m3 bytes [T, K], fp32 scale [T]) with xh ~= scale * e4m3."""
    _req(xh, torch.float16, "xh")
    T, K_ = xh.shape
    xq = xq if xq is not None else torch.empty(T, K_, dtype=torch.uint8, device=xh.device)
    scale = scale if scale is not None else torch.empty(T, dtype=torch.float32, device=xh.device)
    _check(_lib().r4dxb_quantize_rows_e4m3(_p(xh), _p(xq), _p(scale), T, K_, _stream()), "quantize_rows_e4m3")
    return xq, scale


def trellis_gemm_f8(w: TrellisWeight, xq: torch.Tensor, x_scale: torch.Tensor, residual: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None, tn: Optional[int] = None) -> torch.Tensor:
    """y[T, N] from e4m3 transformed activations (``quantize_rows_e4m3``) on the 8-bit tcgen05 path."""
    T = xq.numel() // w.K
    out = out if out is not None else torch.empty(T, w.N, dtype=BF, device=xq.device)
    # 512-column tiles as soon as there are that many rows: below, the decode warps and not the operand bytes set the pace
    tn = tn or (512 if T > 256 else (256 if T > 128 else 128))
    _check(_lib().r4dxb_trellis_gemm_f8(_p(w.words), _p(w.svh), _p(xq), _p(x_scale), _p(out), _p(residual), T, w.N, w.K, w.kb, tn,
                                        _p(gemm_status(xq.device)), _stream()), "trellis_gemm_f8")
    return out


def dense_gemm_hadamard(W: torch.Tensor, svh: torch.Tensor, xh: torch.Tensor, tn: Optional[int] = None) -> torch.Tensor:
    """Same kernel with a dense fp16 A operand: y = svh * H128(xh W^T) over 128-row blocks of N."""
    _req(W, torch.float16, "W"); _req(xh, torch.float16, "xh")
    N, K_ = W.shape
    T = xh.numel() // K_
    out = torch.empty(T, N, dtype=BF, device=xh.device)
    tn = tn or pick_token_tile(T, N)
    _check(_lib().r4dxb_trellis_gemm(_p(W), _p(svh), _p(xh), _p(out), None, T, N, K_, 0, tn,
                                     _p(gemm_status(xh.device)), _stream()), "dense_gemm")
    return out


register_cuda_sig("r4dxb_linear_tc", _I, [_P, _P, _I, _I, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P])


def linear_tc(W, x: torch.Tensor, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
              out_f32: bool = False, out: Optional[torch.Tensor] = None, tn: Optional[int] = None,
              act: int = 0) -> torch.Tensor:
    """y[T, N] = act(x W^T + bias) + residual on the tcgen05 kernel for any number of rows.

    ``W``: a dense bf16 / fp16 [N, K] matrix (x must have the same dtype; N % 4 == 0, K % 8 == 0), a ``W4Weight`` or a
    ``W8Weight`` (x bf16 or fp16; bf16 rows are narrowed to fp16 first: the group scales already make the weights fp16;
    N and K multiples of 128).  ``act``: 0 none, 1 tanh-GELU, 2 erf-GELU.
    """
    dev = x.device
    if isinstance(W, W8Weight):
        N, K_ = W.N, W.K
        xk = x if x.dtype == torch.float16 else x.to(torch.float16)
        kind, group, is_bf, wp, szp = 2, W.group, 0, W.wq, W.ws
    elif isinstance(W, W4Weight):
        N, K_ = W.N, W.K
        xk = x if x.dtype == torch.float16 else x.to(torch.float16)
        kind, group, is_bf, wp, szp = 1, W.group, 0, W.wq, W.wsz
    else:
        N, K_ = W.shape
        if W.dtype not in (BF, torch.float16) or x.dtype != W.dtype:
            raise KernelError("linear_tc: W and x must both be bf16 or both fp16")
        xk, kind, group, is_bf, wp, szp = x, 0, 0, int(W.dtype == BF), W, None
    if (kind >= 1 and (N % 128 or K_ % 128)) or N % 4 or K_ % 8:
        raise KernelError(f"linear_tc: unsupported shape N={N}, K={K_}")
    xk = xk.reshape(-1, K_)
    if not xk.is_contiguous():
        xk = xk.contiguous()
    T = xk.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if out_f32 else BF, device=dev)
    else:
        if out.dtype not in (torch.float32, BF) or out.numel() != T * N or not out.is_contiguous():
            raise KernelError("linear_tc: out must be a contiguous fp32 or bf16 [T, N] tensor")
        out_f32 = out.dtype == torch.float32
    if bias is not None:
        _req(bias, BF, "bias")
    if residual is not None:
        _req(residual, BF, "residual")
    tn = tn or pick_token_tile(T, N)
    _check(_lib().r4dxb_linear_tc(_p(wp), _p(szp), kind, group, is_bf, _p(xk), _p(out), (1 if out_f32 else 0) | (act << 8),
                                  _p(bias), _p(residual), T, N, K_, tn, _p(gemm_status(dev)), _stream()), "linear_tc")
    return out


register_cuda_sig("r4dxb_gdn_prefill", _I, [_P] * 16 + [_I, _I, _I, _I, _I, _F, _P, _P])
register_cuda_sig("r4dxb_gdn_chunk_ws_floats", ctypes.c_longlong, [_I, _I])
register_cuda_sig("r4dxb_attn_prefill", _I, [_P] * 7 + [_I, _I, _I, _I, _I, _I, _P])


register_cuda_sig("r4dxb_gdn_prefill_gate", _I, [_P] * 16 + [_I, _I, _I, _I, _I, _F, _P, _I, _P])


def gdn_prefill_gate(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, scratch: dict, out, T: int, H: int, Hk: int,
                     D: int, pos0: int, eps: float, gate_act: int, exact_scan: bool = True):
    """``gdn_prefill`` with the norm's output gate chosen by the caller (1 = sigmoid).  ``exact_scan`` keeps the recurrence
    token by token.  The chunked kernel forms every pair decay directly as exp(G_i - G_j) <= 1 (it never splits it around
    the chunk's midpoint, the construction that broke the reference's scan on gates of A = exp(A_log) up to ~158 per step;
    docs/qwen4exp.md "The GDN chunk-scan defect"), so it is not exposed to that defect; a GPU test runs it on per-chunk gate
    sums above 10^4 nats against the exact recurrence."""
    _check(_lib().r4dxb_gdn_prefill_gate(_p(mixed), _p(z), _p(ab), _p(conv_w), _p(A_log), _p(dt_bias), _p(norm_w), _p(ring),
                                         _p(state), _p(scratch["q"]), _p(scratch["k"]), _p(scratch["v"]), _p(scratch["eg"]),
                                         _p(scratch["beta"]), _p(scratch["o"]), _p(out), T, H, Hk, D, pos0, eps,
                                         None if exact_scan else _p(scratch.get("ws")), gate_act, _stream()), "gdn_prefill_gate")
    return out


def gdn_prefill(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, scratch: dict, out, T: int, H: int, Hk: int,
                D: int, pos0: int, eps: float = 1e-6):
    """scratch: dict with fp32 tensors q, k [T,Hk,D]; v, o [T,H,D]; eg, beta [T,H]; optional "ws" (see
    gdn_chunk_ws_floats) switches D = 128 chunks of >= 128 tokens to the chunked tensor-core recurrence."""
    _check(_lib().r4dxb_gdn_prefill(_p(mixed), _p(z), _p(ab), _p(conv_w), _p(A_log), _p(dt_bias), _p(norm_w), _p(ring),
                                    _p(state), _p(scratch["q"]), _p(scratch["k"]), _p(scratch["v"]), _p(scratch["eg"]),
                                    _p(scratch["beta"]), _p(scratch["o"]), _p(out), T, H, Hk, D, pos0, eps,
                                    _p(scratch.get("ws")), _stream()),
           "gdn_prefill")
    return out


register_cuda_sig("r4dxb_w8a16_gemv", _I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_rotate_rows", _I, [_P, _P, ctypes.c_longlong, _I, _I, _P])


def w8a16_gemv(w, x: torch.Tensor, out: Optional[torch.Tensor] = None, out_f32: bool = False) -> torch.Tensor:
    """y[T, N] for a quant.w4a16.W8Weight on the device (T <= 8)."""
    _req(x, BF, "x")
    T = x.numel() // w.K
    out = out if out is not None else torch.empty(T, w.N, dtype=torch.float32 if out_f32 else BF, device=x.device)
    _check(_lib().r4dxb_w8a16_gemv(_p(w.wq), _p(w.ws), _p(x), _p(out), T, w.N, w.K, w.group,
                                   1 if out.dtype == torch.float32 else 0, _stream()), "w8a16_gemv")
    return out


def rotate_rows(x: torch.Tensor, signs: Optional[torch.Tensor] = None, mode: int = 0) -> torch.Tensor:
    """In-place 128-block Hadamard rotation of bf16 rows; mode 1 applies ``signs`` before, mode 2 after."""
    _req(x, BF, "x")
    H = x.shape[-1]
    _check(_lib().r4dxb_rotate_rows(_p(x), _p(signs), x.numel() // H, H, mode, _stream()), "rotate_rows")
    return x


def gdn_chunk_ws_floats(T: int, H: int) -> int:
    return int(_lib().r4dxb_gdn_chunk_ws_floats(T, H))


register_cuda_sig("r4dxb_attn_prefill_tc", _I, [_P] * 7 + [_I, _I, _I, _I, _I, _I, _P, _P])

# Prefill attention kernel: "tc" = tcgen05 with S, P and O in tensor memory (head dimensions 128 / 256, default),
# "mma" = the warp-level mma.sync kernel (every head dimension; kill switch / A-B runs).
ATTN_PREFILL_IMPL = os.environ.get("R4DXB_ATTN_PREFILL", "tc")


def set_attn_prefill_impl(name: str) -> None:
    global ATTN_PREFILL_IMPL
    if name not in ("tc", "mma"):
        raise KernelError(f"unknown prefill attention kernel {name!r}")
    ATTN_PREFILL_IMPL = name


register_cuda_sig("r4dxb_attn_prefill_ex", _I, [_P] * 7 + [_I, _I, _I, _I, _I, _I, _P, _P])


def attn_prefill(q, qg, cache, block_table, k_descale, v_descale, out, T: int, Hq: int, Hkv: int, D: int, pos0: int,
                 gated: bool = True, window: int = 0, key_limit: Optional[torch.Tensor] = None):
    """``key_limit`` ([T] int32, -1 = none): row t also sees keys up to that absolute position (rows of an image block
    attend to their whole block); such calls take the mma.sync kernel, which carries the per-row limit."""
    if key_limit is not None:
        _check(_lib().r4dxb_attn_prefill_ex(_p(q), _p(qg), _p(cache), _p(block_table), _p(k_descale), _p(v_descale), _p(out),
                                            T, Hq, Hkv, D, pos0, (1 if gated else 0) | (window << 1), _p(key_limit), _stream()),
               "attn_prefill_ex")
        return out
    if ATTN_PREFILL_IMPL == "tc" and D in (128, 256):
        _check(_lib().r4dxb_attn_prefill_tc(_p(q), _p(qg), _p(cache), _p(block_table), _p(k_descale), _p(v_descale), _p(out),
                                            T, Hq, Hkv, D, pos0, (1 if gated else 0) | (window << 1),
                                            _p(gemm_status(out.device)), _stream()), "attn_prefill_tc")
        return out
    _check(_lib().r4dxb_attn_prefill(_p(q), _p(qg), _p(cache), _p(block_table), _p(k_descale), _p(v_descale), _p(out),
                                     T, Hq, Hkv, D, pos0, (1 if gated else 0) | (window << 1), _stream()), "attn_prefill")
    return out


register_cuda_sig("r4dxb_spec_accept", _I, [_P, _P, _I, _P, _P, _P])


def spec_accept(next_ids: torch.Tensor, draft: torch.Tensor, T: int, out: torch.Tensor, n_replay: Optional[torch.Tensor]) -> torch.Tensor:
    """out[0] = rows to commit, out[1..] = emitted tokens for a T-row speculative window."""
    _check(_lib().r4dxb_spec_accept(_p(next_ids), _p(draft), T, _p(out), _p(n_replay), _stream()), "spec_accept")
    return out


register_cuda_sig("r4dxb_moe_router", _I, [_P, _I, _I, _I, _I, _P, _P, _P])
register_cuda_sig("r4dxb_moe_plan", _I, [_P, _I, _I, _I, _I, _P, _P, _P])
register_cuda_sig("r4dxb_moe_combine", _I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemv_grouped", _I, [_P] * 7 + [_I] * 9 + [_P])


def moe_router(logits: torch.Tensor, k: int, renorm: bool, ids: torch.Tensor, weights: torch.Tensor):
    T, E = logits.shape
    _check(_lib().r4dxb_moe_router(_p(logits), T, E, k, 1 if renorm else 0, _p(ids), _p(weights), _stream()), "moe_router")
    return ids, weights


register_cuda_sig("r4dxb_moe_router_sigmoid", _I, [_P, _P, _I, _I, _I, _I, _F, _P, _P, _P])
register_cuda_sig("r4dxb_short_conv", _I, [_P, _P, _P, _P, _P, _I, _I, _I, _P])


def moe_router_sigmoid(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, renorm: bool, scale: float,
                       ids: torch.Tensor, weights: torch.Tensor):
    """Sigmoid router: experts are selected by sigmoid(logit) + bias, weighted by the unbiased sigmoids."""
    T, E = logits.shape
    _check(_lib().r4dxb_moe_router_sigmoid(_p(logits), _p(bias), T, E, k, 1 if renorm else 0, float(scale), _p(ids), _p(weights),
                                           _stream()), "moe_router_sigmoid")
    return ids, weights


def short_conv(bcx: torch.Tensor, w: torch.Tensor, ring: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, T: int):
    """out[T, H] = C * causal_fir(B * x) over the thirds of bcx [T, 3H]; ``ring`` [32, H] carries the rows before the call."""
    H, L = w.shape
    assert bcx.shape[1] == 3 * H and ring.shape == (32, H) and w.dtype == torch.bfloat16 and bcx.is_contiguous()
    _check(_lib().r4dxb_short_conv(_p(bcx), _p(w), _p(ring), _p(positions), _p(out), T, H, L, _stream()), "short_conv")
    return out


register_cuda_sig("r4dxb_moe_route_plan", _I, [_P, _P, _I, _I, _I, _I, _I, _F, _P, _P, _I, _I, _P, _P, _P])


def moe_route_plan(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, renorm: bool, sigmoid: bool, scale: float,
                   ids: torch.Tensor, weights: torch.Tensor, e_begin: int, e_count: int, offsets: torch.Tensor, perm: torch.Tensor):
    """Router + routing plan of T <= 8 rows in one launch (the results of ``moe_router`` / ``moe_router_sigmoid`` + ``moe_plan``)."""
    _req(logits, torch.float32, "logits")
    T, E = logits.shape
    _check(_lib().r4dxb_moe_route_plan(_p(logits), _p(bias), T, E, k, 1 if renorm else 0, 1 if sigmoid else 0, scale, _p(ids),
                                       _p(weights), e_begin, e_count, _p(offsets), _p(perm), _stream()), "moe_route_plan")


def moe_plan(ids: torch.Tensor, npairs: int, E: int, e_begin: int, e_count: int, offsets: torch.Tensor, perm: torch.Tensor):
    _check(_lib().r4dxb_moe_plan(_p(ids), npairs, E, e_begin, e_count, _p(offsets), _p(perm), _stream()), "moe_plan")
    return offsets, perm


def moe_combine(y_pairs, ids, weights, shared, shared_gate, residual, out, T: int, H: int, k: int):
    _check(_lib().r4dxb_moe_combine(_p(y_pairs), _p(ids), _p(weights), _p(shared), _p(shared_gate), _p(residual), _p(out),
                                    T, H, k, _stream()), "moe_combine")
    return out


register_cuda_sig("r4dxb_trellis_gemv_grouped_pairs", _I, [_P] * 8 + [_I] * 11 + [_P])


def trellis_gemv_grouped_pairs(words, suh, svh, x, y, offsets, perm, pair_ids, pairs: int, e_begin: int, in_div: int, n_pass: int,
                               tmax: int, prologue: int, experts: int, N: int, Kd: int, kb: int, ksplit: int):
    """The grouped expert product launched over the call's routed pairs only (``pair_ids`` = the router's expert ids,
    [pairs] int32): the CTAs of the first pair of each expert's list run that expert, so a decode step launches
    10 experts' CTAs instead of 512 experts' (most of which returned at once)."""
    for p_ in range(n_pass):
        _check(_lib().r4dxb_trellis_gemv_grouped_pairs(_p(words), _p(suh), _p(svh), _p(x), _p(y), _p(offsets), _p(perm), _p(pair_ids),
                                                       pairs, e_begin, in_div, p_, tmax, prologue, experts, N, Kd, kb, ksplit,
                                                       _stream()), "trellis_gemv_grouped_pairs")
    return y


def trellis_gemv_grouped(words, suh, svh, x, y, offsets, perm, in_div: int, n_pass: int, tmax: int, prologue: int,
                         experts: int, N: int, Kd: int, kb: int, ksplit: int):
    """Every local expert times its planned rows; ``n_pass`` launches cover up to n_pass * tmax rows per expert."""
    for p_ in range(n_pass):
        _check(_lib().r4dxb_trellis_gemv_grouped(_p(words), _p(suh), _p(svh), _p(x), _p(y), _p(offsets), _p(perm), in_div, p_,
                                                 tmax, prologue, experts, N, Kd, kb, ksplit, _stream()), "trellis_gemv_grouped")
    return y


register_cuda_sig("r4dxb_rotate_residual", _I, [_P, _P, _P, ctypes.c_longlong, _I, _I, _I, _P])


def rotate_residual(x: torch.Tensor, signs: torch.Tensor, mix: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """In place on bf16 rows [T, H]: x <- x Q (or x Q^T), the residual-stream rotation of ``quant/rotation.py``."""
    _req(x, BF, "x")
    H = x.shape[-1]
    B = H // mix.shape[0]
    _check(_lib().r4dxb_rotate_residual(_p(x), _p(signs), _p(mix), x.numel() // H, H, B, 1 if inverse else 0, _stream()),
           "rotate_residual")
    return x


register_cuda_sig("r4dxb_moe_tiles", _I, [_P, _I, _I, _P, _P, _I, _P])
register_cuda_sig("r4dxb_trellis_input_grouped", _I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_trellis_gemm_grouped", _I, [_P] * 8 + [_I] * 7 + [_P, _P])


def moe_tiles(offsets: torch.Tensor, E: int, tn: int, tiles: torch.Tensor, ntiles: torch.Tensor):
    """Token tiles of a routing plan: (local expert, first sorted row) pairs, ``tn`` rows of one expert each."""
    _check(_lib().r4dxb_moe_tiles(_p(offsets), E, tn, _p(tiles), _p(ntiles), tiles.numel() // 2, _stream()), "moe_tiles")


def trellis_input_grouped(x: torch.Tensor, suh: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, perm: torch.Tensor,
                          P: int, xdiv: int, mode: int = 0):
    """out[p] = fp16 H128(suh[e(p)] * act(x[perm[p] // xdiv])) for the planned pairs in expert order."""
    E, K_ = suh.shape
    _check(_lib().r4dxb_trellis_input_grouped(_p(x), _p(suh), _p(out), _p(offsets), _p(perm), E, P, K_, xdiv, mode, _stream()),
           "trellis_input_grouped")
    return out


def trellis_gemm_grouped(words, svh, xh, y, offsets, perm, tiles, ntiles, P: int, E: int, N: int, Kd: int, kb: int, tn: int):
    """y[perm[p]] = expert e(p)'s trellis linear of the transformed row xh[p]; one launch for every expert."""
    # grid height: no plan of P pairs over E experts has more than P / tn + E tiles (CTAs past the plan's count leave at once)
    bound = min(tiles.numel() // 2, P // tn + E)
    _check(_lib().r4dxb_trellis_gemm_grouped(_p(words), _p(svh), _p(xh), _p(y), _p(offsets), _p(perm), _p(tiles), _p(ntiles),
                                             bound, P, E, N, Kd, kb, tn, _p(gemm_status(xh.device)), _stream()),
           "trellis_gemm_grouped")
    return y


register_cuda_sig("r4dxb_topk_lse", _I, [_P, _I, _I, _I, _F, _I, _P, _P, _P, _P, _P])
register_cuda_sig("r4dxb_repetition_penalty", _I, [_P, _I, _P, _I, _F, _P])


def topk_lse(logits: torch.Tensor, k: int = 64, temperature: float = 1.0, id_offset: int = 0):
    """(values [T,k], ids [T,k] in canonical order, lse [T]) of fp32 logits rows."""
    _req(logits, torch.float32, "logits")
    T, V = logits.shape
    dev = logits.device
    vals = torch.empty(T, k, dtype=torch.float32, device=dev)
    ids = torch.empty(T, k, dtype=torch.int32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    scratch = torch.empty(T * 128 * (2 * k + 2), dtype=torch.float32, device=dev)
    _check(_lib().r4dxb_topk_lse(_p(logits), T, V, k, temperature, id_offset, _p(vals), _p(ids), _p(lse), _p(scratch), _stream()),
           "topk_lse")
    return vals, ids, lse


def repetition_penalty(logits_row: torch.Tensor, seen: torch.Tensor, penalty: float) -> torch.Tensor:
    _req(logits_row, torch.float32, "logits"); _req(seen, torch.int32, "seen")
    _check(_lib().r4dxb_repetition_penalty(_p(logits_row), logits_row.numel(), _p(seen), seen.numel(), penalty, _stream()),
           "repetition_penalty")
    return logits_row


# ---- qwen4_exp family: gated multi-stream residual, n-gram embedding layer, block-selecting attention ----------------
_LL = ctypes.c_longlong
register_cuda_sig("r4dxb_gdn_decode_gate", _I, [_P] * 15 + [_I, _I, _I, _I, _F, _I, _P])
register_cuda_sig("r4dxb_q4x_grouped_rmsnorm", _I, [_P, _P, _P, _I, _I, _I, _F, _P])
register_cuda_sig("r4dxb_q4x_hc_mid", _I, [_P, _P, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_q4x_hc_mix", _I, [_P, _P, _P, _I, _I, _I, _P])
register_cuda_sig("r4dxb_q4x_hc_inject", _I, [_P, _P, _P, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_q4x_embed_repeat", _I, [_P, _P, _P, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_q4x_ngram_gather", _I, [_P, _P, _P, _P, _P, _I, _I, _I, _LL, _P, _P, _P, _LL, _P])
register_cuda_sig("r4dxb_q4x_ple_gate_value", _I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P])
register_cuda_sig("r4dxb_q4x_ple_conv", _I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P])
register_cuda_sig("r4dxb_q4x_qsa_index", _I, [_P] * 7 + [_I, _I, _I, _I, _I, _F, _F, _P])
register_cuda_sig("r4dxb_q4x_qsa_select", _I, [_P] * 6 + [_I] * 8 + [_P])
register_cuda_sig("r4dxb_q4x_qsa_attn", _I, [_P] * 12 + [_I] * 8 + [_P])


def gdn_decode_gate(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, log_u, log_k, log_eg, positions, n_replay, out,
                    T: int, H: int, Hk: int, D: int, eps: float, gate_act: int):
    """One GDN step for T <= 8 rows with the norm's output gate chosen by the caller (0 silu, 1 sigmoid)."""
    _check(_lib().r4dxb_gdn_decode_gate(_p(mixed), _p(z), _p(ab), _p(conv_w), _p(A_log), _p(dt_bias), _p(norm_w), _p(ring), _p(state),
                                        _p(log_u), _p(log_k), _p(log_eg), _p(positions), _p(n_replay), _p(out), T, H, Hk, D, eps,
                                        gate_act, _stream()), "gdn_decode_gate")
    return out


def q4x_grouped_rmsnorm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _req(x, BF, "x"); _req(w, BF, "w")
    rows, C = x.shape
    out = out if out is not None else torch.empty_like(x)
    _check(_lib().r4dxb_q4x_grouped_rmsnorm(_p(x), _p(w), _p(out), rows, groups, C // groups, eps, _stream()), "q4x_grouped_rmsnorm")
    return out


def q4x_hc_mid(down: torch.Tensor, mid: torch.Tensor, lowrank: int, hc: int) -> torch.Tensor:
    _req(down, torch.float32, "down"); _req(mid, BF, "mid")
    rows, stride = down.shape
    _check(_lib().r4dxb_q4x_hc_mid(_p(down), _p(mid), rows, lowrank, stride, hc, _stream()), "q4x_hc_mid")
    return mid


def q4x_hc_mix(n: torch.Tensor, up: torch.Tensor, x: torch.Tensor, hc: int) -> torch.Tensor:
    _req(n, BF, "n"); _req(up, torch.float32, "up"); _req(x, BF, "x")
    rows, H = x.shape
    _check(_lib().r4dxb_q4x_hc_mix(_p(n), _p(up), _p(x), rows, hc, H, _stream()), "q4x_hc_mix")
    return x


def q4x_hc_inject(h: torch.Tensor, block_out: torch.Tensor, inject: torch.Tensor, hc: int) -> torch.Tensor:
    """``inject``: the hc inject columns of the gate's fp32 product (a column slice of a wider row is fine)."""
    _req(h, BF, "h"); _req(block_out, BF, "block_out")
    rows, H = block_out.shape
    if inject.dtype != torch.float32 or inject.stride(1) != 1:
        raise ValueError("inject: fp32 with unit column stride")
    _check(_lib().r4dxb_q4x_hc_inject(_p(h), _p(block_out), inject.data_ptr(), rows, hc, H, inject.stride(0), _stream()), "q4x_hc_inject")
    return h


def q4x_embed_repeat(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, hc: int) -> torch.Tensor:
    _req(table, BF, "table"); _req(ids, torch.int32, "ids"); _req(out, BF, "out")
    rows = ids.numel()
    _check(_lib().r4dxb_q4x_embed_repeat(_p(table), _p(ids), _p(out), rows, table.shape[0], table.shape[1], hc, _stream()), "q4x_embed_repeat")
    return out


class NgramDeviceArgs:
    """Host arrays of the hash parameters, built once per table (ctypes reads them at every launch)."""

    def __init__(self, header):
        self.heads, self.head_dim, self.rows, self.eos = header.heads, header.head_dim, header.rows, header.eos_token_id
        self.mult = (ctypes.c_longlong * 3)(*header.multipliers)
        self.primes = (ctypes.c_ulonglong * 16)(*header.head_primes)
        self.offsets = (ctypes.c_ulonglong * 16)(*header.head_offsets)


def q4x_ngram_gather(ids: torch.Tensor, positions: torch.Tensor, hist: torch.Tensor, table: torch.Tensor, emb: torch.Tensor, T: int,
                     args: NgramDeviceArgs) -> torch.Tensor:
    _req(ids, torch.int32, "ids"); _req(hist, torch.int32, "hist"); _req(table, BF, "table"); _req(emb, BF, "emb")
    _check(_lib().r4dxb_q4x_ngram_gather(_p(ids), _p(positions), _p(hist), _p(table), _p(emb), T, args.heads, args.head_dim, args.rows,
                                         ctypes.addressof(args.mult), ctypes.addressof(args.primes), ctypes.addressof(args.offsets),
                                         args.eos, _stream()), "q4x_ngram_gather")
    return emb


def q4x_ple_gate_value(key_proj, h, value, norm_key, norm_query, gated_value, hc: int, eps: float):
    _req(key_proj, torch.float32, "key_proj"); _req(value, torch.float32, "value"); _req(h, BF, "h")
    rows, H = value.shape
    _check(_lib().r4dxb_q4x_ple_gate_value(_p(key_proj), _p(h), _p(value), _p(norm_key), _p(norm_query), _p(gated_value), rows, hc, H,
                                           eps, _stream()), "q4x_ple_gate_value")
    return gated_value


def q4x_ple_conv(gvn, gated_value, conv_w, ring, h, positions, rows: int, kernel: int, dilation: int):
    _req(gvn, BF, "gvn"); _req(ring, BF, "ring"); _req(conv_w, BF, "conv_w")
    C = gvn.shape[1]
    assert ring.shape == (32, C) and conv_w.shape == (C, kernel)
    _check(_lib().r4dxb_q4x_ple_conv(_p(gvn), _p(gated_value), _p(conv_w), _p(ring), _p(h), _p(positions), rows, C, kernel, dilation,
                                     _stream()), "q4x_ple_conv")
    return h


def q4x_qsa_index(qk, q_norm, k_norm, positions, idx_q, raw_keys, block_keys, T: int, Hi: int, Di: int, ratio: int, rotary_dim: int,
                  theta: float, eps: float):
    _req(qk, torch.float32, "qk"); _req(idx_q, BF, "idx_q"); _req(raw_keys, BF, "raw_keys"); _req(block_keys, BF, "block_keys")
    _check(_lib().r4dxb_q4x_qsa_index(_p(qk), _p(q_norm), _p(k_norm), _p(positions), _p(idx_q), _p(raw_keys), _p(block_keys), T, Hi, Di,
                                      ratio, rotary_dim, theta, eps, _stream()), "q4x_qsa_index")


def q4x_qsa_select(idx_q, block_keys, positions, scores, sel_tokens, sel_count, T: int, Hi: int, Di: int, ratio: int, topk: int,
                   nb_max: int):
    _req(scores, torch.float32, "scores"); _req(sel_tokens, torch.int32, "sel_tokens"); _req(sel_count, torch.int32, "sel_count")
    _check(_lib().r4dxb_q4x_qsa_select(_p(idx_q), _p(block_keys), _p(positions), _p(scores), _p(sel_tokens), _p(sel_count), T, Hi, Di,
                                       ratio, topk, nb_max, scores.shape[1], sel_tokens.shape[1], _stream()), "q4x_qsa_select")


def q4x_qsa_attn(q, qg, cache, block_table, positions, sel_tokens, sel_count, k_descale, v_descale, part_acc, part_ml, out, T: int,
                 Hq: int, Hkv: int, D: int, max_tokens: int, nsplit: int, gated: bool = True):
    need = T * Hq * nsplit
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise ValueError("q4x_qsa_attn: partial buffers too small for this split count")
    _check(_lib().r4dxb_q4x_qsa_attn(_p(q), _p(qg), _p(cache), _p(block_table), _p(positions), _p(sel_tokens), _p(sel_count),
                                     _p(k_descale), _p(v_descale), _p(part_acc), _p(part_ml), _p(out), T, Hq, Hkv, D,
                                     sel_tokens.shape[1], max_tokens, nsplit, 1 if gated else 0, _stream()), "q4x_qsa_attn")
    return out


register_cuda_sig("r4dxb_q4x_hc_gate", _I, [_P] * 8 + [_I, _I, _I, _I, _I, _F, _P])


def q4x_hc_gate(h, norm_w, w_down_inject, w_up, mid, injv, rstd, x, T: int, hc: int, lowrank: int, n_inject: int, eps: float):
    """The stream gate of T <= 8 rows in two launches; ``x`` [T, H] receives the block input, ``injv`` [T, n_inject] the raw
    injection logits (the same numbers the five-kernel chain produces)."""
    _req(h, BF, "h"); _req(w_down_inject, BF, "w_down_inject"); _req(w_up, BF, "w_up"); _req(x, BF, "x")
    H = x.shape[1]
    assert w_down_inject.shape == (lowrank + n_inject, hc * H) and w_up.shape == (hc * H, lowrank)
    _check(_lib().r4dxb_q4x_hc_gate(_p(h), _p(norm_w), _p(w_down_inject), _p(w_up), _p(mid), _p(injv), _p(rstd), _p(x), T, hc, H,
                                    lowrank, n_inject, eps, _stream()), "q4x_hc_gate")
    return x
