"""w4a16 / w8a16 group-quantized weights (C++ packers; layout in native/src/host/w4a16.cpp)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import native


@dataclass
class W4Weight:
    wq: torch.Tensor    # int32 [N, K/8]
    wsz: torch.Tensor   # int32 [N, K/group]: fp16 scale | fp16 -(1024 + zero)
    N: int
    K: int
    group: int

    def to(self, device) -> "W4Weight":
        return W4Weight(self.wq.to(device), self.wsz.to(device), self.N, self.K, self.group)

    @property
    def nbytes(self) -> int:
        return self.wq.numel() * 4 + self.wsz.numel() * 4


def quantize(W: torch.Tensor, group: int = 64) -> W4Weight:
    L = native.host()
    W = W.detach().to(torch.float32).contiguous().cpu()
    N, K = W.shape
    wq = torch.zeros(N, K // 8, dtype=torch.int32)
    wsz = torch.zeros(N, K // group, dtype=torch.int32)
    if L.r4dxb_w4a16_quantize(W.data_ptr(), N, K, group, wq.data_ptr(), wsz.data_ptr()) != 0:
        raise ValueError("w4a16 quantize rejected the arguments")
    return W4Weight(wq, wsz, N, K, group)


def dequantize(w: W4Weight) -> torch.Tensor:
    L = native.host()
    out = torch.empty(w.N, w.K, dtype=torch.float32)
    wq, wsz = w.wq.cpu().contiguous(), w.wsz.cpu().contiguous()
    if L.r4dxb_w4a16_dequantize(wq.data_ptr(), wsz.data_ptr(), w.N, w.K, w.group, out.data_ptr()) != 0:
        raise ValueError("w4a16 dequantize rejected the arguments")
    return out


def random_weight(N: int, K: int, group: int = 64, seed: int = 0, sigma: float = 0.02, device="cpu") -> W4Weight:
    """Synthetic weight: random nibbles, zero = 8, scale = sigma / 2.3 (unit-ish variance in nibble steps)."""
    import numpy as np
    g = torch.Generator(device=device if str(device).startswith("cuda") else "cpu").manual_seed(seed)
    wq = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=device, generator=g)
    scale = np.float16(sigma / 2.3).view(np.uint16).item()
    nz = np.float16(-(1024.0 + 8.0)).view(np.uint16).item()
    val = (nz << 16) | scale
    if val >= 2**31:
        val -= 2**32
    wsz = torch.full((N, K // group), val, dtype=torch.int32, device=device)
    return W4Weight(wq, wsz, N, K, group)


@dataclass
class W8Weight:
    wq: torch.Tensor    # uint8 [N, K] offset binary
    ws: torch.Tensor    # fp16 [N, K/group]
    N: int
    K: int
    group: int

    def to(self, device) -> "W8Weight":
        return W8Weight(self.wq.to(device), self.ws.to(device), self.N, self.K, self.group)

    @property
    def nbytes(self) -> int:
        return self.wq.numel() + self.ws.numel() * 2


def quantize_w8(W: torch.Tensor, group: int = 64) -> W8Weight:
    L = native.host()
    W = W.detach().to(torch.float32).contiguous().cpu()
    N, K = W.shape
    wq = torch.zeros(N, K, dtype=torch.uint8)
    ws = torch.zeros(N, K // group, dtype=torch.float16)
    if L.r4dxb_w8a16_quantize(W.data_ptr(), N, K, group, wq.data_ptr(), ws.data_ptr()) != 0:
        raise ValueError("w8a16 quantize rejected the arguments")
    return W8Weight(wq, ws, N, K, group)


def dequantize_w8(w: W8Weight) -> torch.Tensor:
    L = native.host()
    out = torch.empty(w.N, w.K, dtype=torch.float32)
    if L.r4dxb_w8a16_dequantize(w.wq.data_ptr(), w.ws.data_ptr(), w.N, w.K, w.group, out.data_ptr()) != 0:
        raise ValueError("w8a16 dequantize rejected the arguments")
    return out
