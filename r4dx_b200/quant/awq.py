"""compressed-tensors ``pack-quantized`` (AWQ-style int4, group-wise, asymmetric) checkpoints as plain weights.

Every quantized linear ``<b>`` of such a checkpoint is four tensors

    <b>.weight_packed      int32 [N, K / 8]          8 unsigned nibbles per word along K (nibble j of word c = column 8 c + j)
    <b>.weight_scale       bf16  [N, K / G]
    <b>.weight_zero_point  int32 [ceil(N / 8), K / G]  8 unsigned nibbles per word along N (nibble n % 8 of row n / 8)
    <b>.weight_shape       int64 [2] = (N, K)

and  W[n, k] = bf16( (q[n, k] - zp[n, k / G]) * scale[n, k / G] ): the product of a 4-bit integer and a bf16 scale is exact
in fp32, so the one rounding is the cast.  ``AwqView`` makes each quad appear as one bf16 tensor ``<b>.weight``, dequantized
when it is read, so the importers and the converter see an ordinary checkpoint.
(reference: src/convert/awq_source.hpp:1-30 states the layout and the rounding; docs/qwen4exp-plan.md 2.5.)
"""
from __future__ import annotations

import json
from typing import Dict, Iterator, Mapping, Optional

import torch

SUFFIXES = ("weight_packed", "weight_scale", "weight_zero_point", "weight_shape")


def pack_scheme(config_text: str) -> Optional[int]:
    """The group size when config.json announces a pack-quantized int4 checkpoint, None when it announces no such format;
    anything but int4 / group strategy / asymmetric static weights raises."""
    d = json.loads(config_text)
    q = d.get("quantization_config")
    if not q or q.get("format") != "pack-quantized":
        return None
    groups = q.get("config_groups") or {}
    if not groups:
        raise ValueError("pack-quantized checkpoint without config_groups")
    size = None
    for name, g in groups.items():
        wq = g.get("weights") or {}
        if wq.get("num_bits") != 4 or wq.get("strategy") != "group" or wq.get("symmetric", False) or wq.get("dynamic", False):
            raise ValueError(f"quantization group {name}: only int4, group strategy, asymmetric, static weights are read")
        if g.get("input_activations"):
            raise ValueError(f"quantization group {name}: activation quantization is not supported")
        if wq.get("actorder") not in (None, "static", False):
            raise ValueError(f"quantization group {name}: activation reordering is not supported")
        gs = int(wq.get("group_size", 128))
        if size is not None and gs != size:
            raise ValueError("quantization groups with different group sizes")
        size = gs
    return size


def _nibbles(words: torch.Tensor) -> torch.Tensor:
    """int32 [..., W] -> uint8-valued int32 [..., W * 8], nibble j of a word at position 8 w + j."""
    shifts = torch.arange(0, 32, 4, dtype=torch.int32)
    return ((words.to(torch.int32).unsqueeze(-1) >> shifts) & 0xF).reshape(*words.shape[:-1], words.shape[-1] * 8)


def dequantize(packed: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, N: int, K: int, group: int = 128) -> torch.Tensor:
    if K % group or group % 8 or packed.shape != (N, K // 8) or scale.shape != (N, K // group) \
            or zero_point.shape != ((N + 7) // 8, K // group):
        raise ValueError("pack-quantized tensor shapes do not fit (N, K, group)")
    q = _nibbles(packed)                                                            # [N, K]
    zp = _nibbles(zero_point.t().contiguous()).t()[:N]                              # [N, K / G]
    w = (q.view(N, K // group, group) - zp.unsqueeze(-1)).float() * scale.float().unsqueeze(-1)
    return w.view(N, K).to(torch.bfloat16)


def quantize(w: torch.Tensor, group: int = 128) -> Dict[str, torch.Tensor]:
    """Min/max asymmetric int4 per group, in the checkpoint's tensor layout (tests and tools)."""
    N, K = w.shape
    g = w.float().view(N, K // group, group)
    lo, hi = g.amin(-1), g.amax(-1)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(torch.bfloat16)
    zp = torch.round(-lo / scale.float()).clamp(0, 15).to(torch.int32)
    q = torch.round(g / scale.float().unsqueeze(-1) + zp.unsqueeze(-1)).clamp(0, 15).to(torch.int32).view(N, K)
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    pack = lambda t: (t.to(torch.int64).view(*t.shape[:-1], -1, 8) << shifts).sum(-1)
    to_i32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    zpad = torch.zeros((N + 7) // 8 * 8, K // group, dtype=torch.int32)
    zpad[:N] = zp
    return {"weight_packed": to_i32(pack(q)), "weight_scale": scale, "weight_zero_point": to_i32(pack(zpad.t().contiguous())).t().contiguous(),
            "weight_shape": torch.tensor([N, K], dtype=torch.int64)}


class AwqView(Mapping):
    """A tensor mapping in which every pack-quantized quad reads as ``<b>.weight`` (bf16 [N, K]); the four component
    names are hidden, everything else passes through."""

    def __init__(self, raw: Mapping, group: int = 128):
        self.raw, self.group = raw, group
        self.bases = {k[:-len("weight_packed")] for k in raw.keys() if k.endswith(".weight_packed")}
        for b in self.bases:
            for sfx in SUFFIXES:
                if b + sfx not in raw:
                    raise ValueError(f"pack-quantized linear {b}: tensor {sfx} is missing")
        self._hidden = {b + sfx for b in self.bases for sfx in SUFFIXES}

    def __getitem__(self, name: str) -> torch.Tensor:
        if name.endswith(".weight") and name[:-len("weight")] in self.bases:
            b = name[:-len("weight")]
            N, K = (int(v) for v in self.raw[b + "weight_shape"].tolist())
            return dequantize(self.raw[b + "weight_packed"], self.raw[b + "weight_scale"], self.raw[b + "weight_zero_point"], N, K, self.group)
        if name in self._hidden:
            raise KeyError(name)
        return self.raw[name]

    def __iter__(self) -> Iterator[str]:
        for k in self.raw.keys():
            if k not in self._hidden:
                yield k
        for b in sorted(self.bases):
            yield b + "weight"

    def __len__(self) -> int:
        return sum(1 for _ in self)

    def __contains__(self, name) -> bool:
        if isinstance(name, str) and name.endswith(".weight") and name[:-len("weight")] in self.bases:
            return True
        return name in self.raw and name not in self._hidden
