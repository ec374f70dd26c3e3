"""Request-level sampling: parameters, the canonical full-row sampler, the exact summary sampler.

The math lives in C++ (``native/src/host/sampler.cpp``); this module owns the per-request RNG and the
choice between the cheap summary path (top-K + log-sum-exp from the device) and the full-row fallback.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from .. import native
from ..native import c_f32, c_f64, c_i64, c_int, c_ptr, c_u64, register_host_sig

register_host_sig("r4dxb_rng_new", c_ptr, [c_u64])
register_host_sig("r4dxb_rng_free", None, [c_ptr])
register_host_sig("r4dxb_rng_next", c_f64, [c_ptr])
register_host_sig("r4dxb_sample_canonical", ctypes.c_int32, [c_ptr, c_i64, c_f32, c_int, c_f32, c_f32, c_f64])
register_host_sig("r4dxb_sample_from_summary", ctypes.c_int32, [c_ptr, c_ptr, c_int, c_f64, c_f32, c_int, c_f32, c_f32, c_f64])
register_host_sig("r4dxb_repetition_penalty", None, [c_ptr, c_i64, c_ptr, c_i64, c_f32])


@dataclass
class SampleParams:
    temperature: float = 1.0      # <= 0: greedy
    top_k: int = 0                # 0: off
    top_p: float = 1.0            # 1: off
    min_p: float = 0.0            # 0: off
    seed: int = 0
    repetition_penalty: float = 1.0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


class Rng:
    """64-bit Mersenne twister; one draw in [0, 1) per emitted token."""

    def __init__(self, seed: int):
        self._L = native.host()
        self._h = self._L.r4dxb_rng_new(seed & (2**64 - 1))

    def next(self) -> float:
        return float(self._L.r4dxb_rng_next(self._h))

    def __del__(self):
        try:
            self._L.r4dxb_rng_free(self._h)
        except Exception:
            pass


def sample_canonical(logits: torch.Tensor, p: SampleParams, u: float) -> int:
    lg = logits.detach().to(torch.float32).cpu().contiguous()
    return int(native.host().r4dxb_sample_canonical(lg.data_ptr(), lg.numel(), p.temperature, p.top_k, p.top_p, p.min_p, u))


def sample_from_summary(top_logits: torch.Tensor, top_ids: torch.Tensor, lse: float, p: SampleParams, u: float) -> int:
    """Exact token or -1 when the summary cannot prove it (caller then uses the full row)."""
    tl = top_logits.detach().to(torch.float32).cpu().contiguous()
    ti = top_ids.detach().to(torch.int32).cpu().contiguous()
    return int(native.host().r4dxb_sample_from_summary(tl.data_ptr(), ti.data_ptr(), tl.numel(), lse, p.temperature,
                                                       p.top_k, p.top_p, p.min_p, u))


def apply_repetition_penalty(logits: torch.Tensor, seen: Sequence[int], penalty: float) -> torch.Tensor:
    """In place on a CPU fp32 row."""
    if penalty == 1.0 or not len(seen):
        return logits
    ids = torch.tensor(list(seen), dtype=torch.int32)
    native.host().r4dxb_repetition_penalty(logits.data_ptr(), logits.numel(), ids.data_ptr(), ids.numel(), penalty)
    return logits


def row_summary(logits: torch.Tensor, temperature: float, k: int = 64):
    """Host twin of the device summary kernel: top-k raw logits in canonical order + lse of the scaled row."""
    lg = logits.detach().to(torch.float32).cpu()
    order = sorted(range(lg.numel()), key=lambda i: (-float(lg[i]), i))[:k] if lg.numel() <= 4096 else None
    if order is None:
        vals, idx = torch.topk(lg, k)
        pairs = sorted(zip(vals.tolist(), idx.tolist()), key=lambda t: (-t[0], t[1]))
        order = [i for _, i in pairs]
    ids = torch.tensor(order, dtype=torch.int32)
    tl = lg[ids.long()]
    lse = float(torch.logsumexp(lg.double() / temperature, 0)) if temperature > 0 else 0.0
    return tl, ids, lse
