"""Per-op device timing of a decode step or a prefill (the `--profile` / `--profile-prefill` flags).

Every kernel-family call made through ``ops.kernels`` is bracketed by a CUDA event pair while the
profile is active; one synchronise at the end turns the pairs into a table.  Names prefixed ``gemm:``
are the weight-streaming linears (reference: src/model/profile_span.h:1-50, model_types.h:84-118).
"""
from __future__ import annotations

import contextlib
from collections import defaultdict
from typing import Dict, List

import torch

from ..ops import kernels as K

_GEMM = {"trellis_gemv", "trellis_gemm", "w4a16_gemv", "bf16_gemv", "bf16_gemv_norm", "trellis_input"}
_OPS = ["embed_gather", "rmsnorm", "add_rmsnorm", "silu_mul", "residual_add", "trellis_gemv", "trellis_gemm", "trellis_input",
        "w4a16_gemv", "bf16_gemv", "bf16_gemv_norm", "argmax_rows", "gdn_decode", "gdn_prefill", "attn_precore", "attn_decode",
        "attn_prefill", "spec_accept"]


class SpanAccumulator:
    def __init__(self):
        self.spans: List = []

    def record(self, name: str, fn, *a, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **kw)
        e1.record()
        self.spans.append((name, e0, e1))
        return out

    def table(self) -> Dict[str, Dict[str, float]]:
        torch.cuda.synchronize()
        agg = defaultdict(lambda: {"calls": 0, "ms": 0.0})
        for name, e0, e1 in self.spans:
            agg[name]["calls"] += 1
            agg[name]["ms"] += e0.elapsed_time(e1)
        return dict(agg)


@contextlib.contextmanager
def profiled(acc: SpanAccumulator):
    saved = {}
    for name in _OPS:
        fn = getattr(K, name)
        saved[name] = fn
        label = ("gemm:" if name in _GEMM else "") + name
        setattr(K, name, (lambda f, l: (lambda *a, **kw: acc.record(l, f, *a, **kw)))(fn, label))
    try:
        yield acc
    finally:
        for name, fn in saved.items():
            setattr(K, name, fn)


def _format(table: Dict[str, Dict[str, float]], title: str) -> str:
    total = sum(v["ms"] for v in table.values())
    lines = [f"{title}: {total:.3f} ms in {sum(v['calls'] for v in table.values())} calls"]
    for name, v in sorted(table.items(), key=lambda kv: -kv[1]["ms"]):
        lines.append(f"  {name:28s} {v['calls']:5d} calls {v['ms']:9.3f} ms {100 * v['ms'] / max(total, 1e-9):5.1f}%")
    gemm = sum(v["ms"] for k, v in table.items() if k.startswith("gemm:"))
    lines.append(f"  weight-streaming linears: {gemm:.3f} ms ({100 * gemm / max(total, 1e-9):.1f}%)")
    return "\n".join(lines)


def profile_decode_step(model, prompt_ids) -> str:
    model.reset()
    tok = model.prefill(torch.as_tensor(list(prompt_ids), dtype=torch.int32))
    model.decode_step_greedy(tok)                       # warm
    acc = SpanAccumulator()
    with profiled(acc):
        model.decode_step_greedy(tok)
    return _format(acc.table(), "decode step")


def profile_prefill(model, prompt_ids) -> str:
    model.reset()
    ids = torch.as_tensor(list(prompt_ids), dtype=torch.int32)
    model.prefill(ids)
    model.reset()
    acc = SpanAccumulator()
    with profiled(acc):
        model.prefill(ids)
    return _format(acc.table(), f"prefill of {ids.numel()} tokens")
