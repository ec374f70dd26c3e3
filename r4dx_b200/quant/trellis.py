"""Trellis-coded weights: Python face of the C++ quantizer / decoder.

Format and bit-exact decode definition: ``native/include/r4dxb_trellis.h``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from .. import native


@dataclass
class TrellisWeight:
    """One quantized linear. ``words`` int32 [packed], ``suh`` fp16 [K], ``svh`` fp16 [N]."""
    words: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor
    N: int
    K: int
    kb: int

    def to(self, device) -> "TrellisWeight":
        return TrellisWeight(self.words.to(device), self.suh.to(device), self.svh.to(device), self.N, self.K, self.kb)

    @property
    def nbytes(self) -> int:
        return self.words.numel() * 4 + self.suh.numel() * 2 + self.svh.numel() * 2


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


def packed_words(N: int, K: int, kb: int) -> int:
    return (N // 16) * (K // 16) * 8 * kb


def quantize(W: torch.Tensor, kb: int, seed: int = 0, threads: int | None = None) -> tuple[TrellisWeight, float]:
    """Viterbi-quantizes W [N, K] (any float dtype, CPU). Returns (weight, relative squared error)."""
    L = native.host()
    W = W.detach().to(torch.float32).contiguous().cpu()
    N, K = W.shape
    if N % 128 or K % 128:
        raise ValueError(f"trellis needs N and K multiples of 128, got {N}x{K}")
    words = torch.empty(packed_words(N, K, kb), dtype=torch.int32)
    suh = torch.empty(K, dtype=torch.float16)
    svh = torch.empty(N, dtype=torch.float16)
    threads = threads or min(32, os.cpu_count() or 1)
    err = L.r4dxb_trellis_quantize(_ptr(W), N, K, kb, seed, threads, _ptr(words), _ptr(suh), _ptr(svh))
    if err < 0:
        raise ValueError("r4dxb_trellis_quantize rejected the arguments")
    return TrellisWeight(words, suh, svh, N, K, kb), float(err)


def quantize_ldlq(W: torch.Tensor, H: torch.Tensor, kb: int, seed: int = 0, damp: float = 0.01,
                  threads: int | None = None) -> tuple[TrellisWeight, float, float]:
    """Error-compensated trellis quantization (block LDLQ): tile columns are encoded last to first and each absorbs, through
    the block LDL factor of the rotated Hessian, the error already made to its right.  ``H`` [K, K] is the second-moment
    matrix of the layer's inputs (``calibrate.capture_hessians``).  Same regularisation (signs, scales) as ``quantize`` for
    the same seed.  Returns (weight, relative squared error of the codes, proxy loss tr(E H' E^T) / tr(D H' D^T))."""
    import ctypes
    L = native.host()
    W = W.detach().to(torch.float32).contiguous().cpu()
    H = H.detach().to(torch.float32).contiguous().cpu()
    N, K = W.shape
    if N % 128 or K % 128:
        raise ValueError(f"trellis needs N and K multiples of 128, got {N}x{K}")
    if H.shape != (K, K):
        raise ValueError(f"Hessian must be [{K}, {K}], got {tuple(H.shape)}")
    words = torch.empty(packed_words(N, K, kb), dtype=torch.int32)
    suh = torch.empty(K, dtype=torch.float16)
    svh = torch.empty(N, dtype=torch.float16)
    proxy = ctypes.c_double(0.0)
    threads = threads or min(32, os.cpu_count() or 1)
    err = L.r4dxb_trellis_quantize_ldlq(_ptr(W), _ptr(H), N, K, kb, seed, threads, float(damp), _ptr(words), _ptr(suh), _ptr(svh),
                                        ctypes.addressof(proxy))
    if err < 0:
        raise ValueError("r4dxb_trellis_quantize_ldlq rejected the arguments")
    return TrellisWeight(words, suh, svh, N, K, kb), float(err), float(proxy.value)


def quantize_cuda(W: torch.Tensor, kb: int, seed: int = 0, device: str = "cuda") -> tuple[TrellisWeight, float]:
    """The same quantizer with the Viterbi search on the GPU (one CTA per 16x16 tile): regularisation (per-channel
    scale, random signs, Hadamard sandwich, global scale) in torch on the device, then ``r4dxb_trellis_encode_tiles``.
    Returns (weight on ``device``, relative squared error).  The random signs come from torch's generator, so the
    result is a different - equally valid - encoding than the host quantizer's for the same seed."""
    import ctypes
    from ..native import c_f32, c_int, c_ptr, register_cuda_sig
    from ..ops.reference import fwht
    register_cuda_sig("r4dxb_trellis_encode_scratch_bytes", ctypes.c_longlong, [c_int, c_int])
    register_cuda_sig("r4dxb_trellis_encode_tiles", c_int, [c_ptr, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr])
    L = native.cuda()
    Wd = W.detach().to(device, torch.float32)
    N, K = Wd.shape
    if N % 128 or K % 128:
        raise ValueError(f"trellis needs N and K multiples of 128, got {N}x{K}")
    g = torch.Generator(device=device).manual_seed(seed)
    su = Wd.pow(2).mean(0).sqrt()
    mean_su = su.mean()
    su = torch.where((su > 0) & (mean_su > 0), su / mean_su, torch.ones_like(su)).clamp(1.0 / 16, 16.0)
    su = (su * (torch.randint(0, 2, (K,), device=device, generator=g) * 2 - 1)).to(torch.float16).float()
    sv = (torch.randint(0, 2, (N,), device=device, generator=g) * 2 - 1).float()
    D = fwht(Wd / su[None, :] * sv[:, None])                                    # rows: Hadamard along K (normalised)
    D = fwht(D.t().contiguous()).t().contiguous()                               # columns: Hadamard along N
    sigma = D.pow(2).mean().sqrt()
    sigma_h = (sigma if float(sigma) > 0 else torch.ones_like(sigma)).to(torch.float16).float()
    D = D / sigma_h
    # tiles in word order [N/128][K/16][8 row tiles][16 x 16 positions]
    tiles = D.view(N // 128, 8, 16, K // 16, 16).permute(0, 3, 1, 2, 4).contiguous().view(-1, 256)
    ntiles = tiles.shape[0]
    ctas = min(ntiles, 148)
    words = torch.empty(ntiles * 8 * kb, dtype=torch.int32, device=device)
    err = torch.empty(ntiles, dtype=torch.float32, device=device)
    scratch = torch.empty(int(L.r4dxb_trellis_encode_scratch_bytes(kb, ctas)), dtype=torch.uint8, device=device)
    rc = L.r4dxb_trellis_encode_tiles(tiles.data_ptr(), ntiles, kb, words.data_ptr(), err.data_ptr(), scratch.data_ptr(), ctas,
                                      torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise ValueError(f"r4dxb_trellis_encode_tiles failed with code {rc}")
    rel = float(err.double().sum().item() / (N * K))
    return TrellisWeight(words, su.to(torch.float16), (sv * sigma_h).to(torch.float16), N, K, kb), rel


def random_weight(N: int, K: int, kb: int, seed: int = 0, sigma: float = 0.02, device="cpu") -> TrellisWeight:
    """Synthetic weight: random code bits (values ~ N(0,1)), random signs, global scale sigma."""
    g = torch.Generator().manual_seed(seed)
    n_words = packed_words(N, K, kb)
    if str(device).startswith("cuda"):
        gg = torch.Generator(device=device).manual_seed(seed)
        words = torch.randint(-2**31, 2**31 - 1, (n_words,), dtype=torch.int32, device=device, generator=gg)
    else:
        words = torch.empty(n_words, dtype=torch.int32)
        native.host().r4dxb_trellis_random_fill(_ptr(words), n_words, seed)
    suh = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.float16)
    svh = ((torch.randint(0, 2, (N,), generator=g) * 2 - 1).float() * sigma).to(torch.float16)
    return TrellisWeight(words.to(device), suh.to(device), svh.to(device), N, K, kb)


def decode_codes(tw: TrellisWeight) -> torch.Tensor:
    """Q [N, K] fp16: the raw code values before the Hadamard sandwich."""
    L = native.host()
    words = tw.words.cpu().contiguous()
    q = torch.empty(tw.N, tw.K, dtype=torch.float16)
    L.r4dxb_trellis_decode(_ptr(words), tw.N, tw.K, tw.kb, _ptr(q))
    return q


def reconstruct(tw: TrellisWeight, threads: int | None = None) -> torch.Tensor:
    """Effective dense weight [N, K] fp32 = diag(svh) H_N Q H_K diag(suh)."""
    L = native.host()
    words, suh, svh = tw.words.cpu().contiguous(), tw.suh.cpu().contiguous(), tw.svh.cpu().contiguous()
    W = torch.empty(tw.N, tw.K, dtype=torch.float32)
    threads = threads or min(32, os.cpu_count() or 1)
    L.r4dxb_trellis_reconstruct(_ptr(words), _ptr(suh), _ptr(svh), tw.N, tw.K, tw.kb, threads, _ptr(W))
    return W


def linear_reference(tw: TrellisWeight, x: torch.Tensor) -> torch.Tensor:
    """y = svh * H_N(Q . H_K(suh * x)) in fp32 on the CPU (x: [T, K])."""
    from ..ops.reference import fwht
    q = decode_codes(tw).float()
    xt = fwht(x.float().cpu() * tw.suh.float().cpu()[None, :])
    y = xt @ q.T
    return fwht(y) * tw.svh.float().cpu()[None, :]
