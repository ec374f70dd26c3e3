"""Residual-stream rotation ("q2a"): the layer stack runs in a rotated basis x' = x Q that spreads outliers of the
residual stream over all channels before the weights that read it are quantized.

    Q = diag(signs) . blockdiag(H_block / sqrt(block)) . (mix (x) I_block)        (row-vector convention, x' = x Q)

``signs`` are +-1 per channel, ``H_block`` the Sylvester Hadamard matrix of the block size (1024 when the hidden size
allows), ``mix`` a small orthogonal matrix over the hidden/block blocks (5 x 5 for hidden 5120).  A weightless RMSNorm
commutes with Q; a zero-centred norm's (1 + w) does not, so it is folded into the linears that read the normalised
rows and the stored norm weight becomes 0:

    every in-projection (reads the normalised residual)   W' = W diag(1 + w_norm) Q
    every out-projection (writes the residual)            W' = Q^T W
    embeddings, final norm, head, MTP head, drafters      unchanged

At run time the model applies Q once where rows enter the stack (after the embedding gather and any spliced image /
audio rows) and Q^T once where they leave it (before the final norm, MTP priming, feature captures); a container that
carries ``rotation.signs`` switches those two kernels on, nothing else changes.

In the trellis layout every linear already carries its own 128-wide input and output Hadamard transforms, so the
reference's second stage ("q2ab": block Hadamards on the inputs of down / o / out_proj) adds nothing there:
``q2ab`` is accepted for trellis bodies and means the same as ``q2a``.

(reference: docs/quant2.md section 3 "Q2a -- residual-stream rotation", src/kernels/src/rotate_residual.hip:79-333,
src/convert/rotation.hpp; the fold table and the entry / exit sites follow that document.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..config import ModelConfig

KINDS = ("q2a", "q2ab")


@dataclass
class RotationSpec:
    kind: str
    seed: int
    hidden: int
    block: int

    @property
    def nblk(self) -> int:
        return self.hidden // self.block

    def to_meta(self) -> Dict[str, object]:
        return {"kind": self.kind, "seed": self.seed, "hidden": self.hidden, "block": self.block}

    @staticmethod
    def from_meta(m: Dict[str, object], hidden: int) -> "RotationSpec":
        if m.get("kind") not in KINDS:
            raise ValueError(f"unknown rotation kind {m.get('kind')!r}")
        seed, block = m.get("seed"), m.get("block")
        if not isinstance(seed, int) or seed < 0:
            raise ValueError("rotation seed must be a non-negative integer")
        if m.get("hidden") != hidden or not isinstance(block, int) or block < 2 or block & (block - 1) or hidden % block:
            raise ValueError(f"rotation geometry {m.get('hidden')}/{block} does not fit hidden size {hidden}")
        return RotationSpec(str(m["kind"]), seed, hidden, block)


def default_block(hidden: int) -> int:
    b = 1
    while b < 1024 and hidden % (2 * b) == 0:
        b *= 2
    return b


def make_spec(kind: str, seed: int, hidden: int, block: Optional[int] = None) -> RotationSpec:
    if kind not in KINDS:
        raise ValueError(f"--rotate {kind}: one of {KINDS}")
    block = block or default_block(hidden)
    if block < 2 or block & (block - 1) or hidden % block:
        raise ValueError(f"rotation block {block} must be a power of two that divides {hidden}")
    return RotationSpec(kind, seed, hidden, block)


def rotation_tensors(spec: RotationSpec) -> Dict[str, torch.Tensor]:
    """signs [hidden] (+-1) and mix [nblk, nblk] (orthogonal), both fp32, derived from the seed alone."""
    g = torch.Generator().manual_seed(spec.seed)
    signs = (torch.randint(0, 2, (spec.hidden,), generator=g) * 2 - 1).to(torch.float32)
    a = torch.randn(spec.nblk, spec.nblk, generator=g, dtype=torch.float64)
    qm, r = torch.linalg.qr(a)
    qm = qm * torch.sign(torch.diagonal(r)).unsqueeze(0)         # a unique factorisation: the result depends on the seed only
    return {"rotation.signs": signs, "rotation.mix": qm.to(torch.float32).contiguous()}


def check_rotation_tensors(spec: RotationSpec, signs: torch.Tensor, mix: torch.Tensor) -> None:
    if signs.numel() != spec.hidden or not bool((signs.float().abs() == 1).all()):
        raise ValueError("rotation.signs must hold exactly +-1 for every channel")
    m = mix.float().cpu()
    if m.shape != (spec.nblk, spec.nblk) or float((m @ m.T - torch.eye(spec.nblk)).abs().max()) > 1e-5:
        raise ValueError("rotation.mix is not an orthogonal matrix of the block count")


def _fwht_last(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester-Hadamard transform over the last dimension (a power of two)."""
    n = x.shape[-1]
    y = x
    h = 1
    while h < n:
        y = y.reshape(*x.shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(*x.shape[:-1], n)
        h *= 2
    return y


def apply_q(x: torch.Tensor, spec: RotationSpec, signs: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """x Q over the last dimension (fp32 / fp64 math in the input's dtype)."""
    lead = x.shape[:-1]
    h = (x * signs.to(x.dtype)).reshape(*lead, spec.nblk, spec.block)
    h = _fwht_last(h) * (1.0 / math.sqrt(spec.block))
    y = torch.einsum("...bc,bd->...dc", h, mix.to(x.dtype))
    return y.reshape(*lead, spec.hidden)


def apply_qt(x: torch.Tensor, spec: RotationSpec, signs: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """x Q^T: the inverse of ``apply_q``."""
    lead = x.shape[:-1]
    h = torch.einsum("...dc,bd->...bc", x.reshape(*lead, spec.nblk, spec.block), mix.to(x.dtype))
    h = _fwht_last(h) * (1.0 / math.sqrt(spec.block))
    return h.reshape(*lead, spec.hidden) * signs.to(x.dtype)


_IN = ("gdn.in_proj_qkv", "gdn.in_proj_z", "gdn.in_proj_a", "gdn.in_proj_b", "attn.qg", "attn.k", "attn.v", "mlp.gate_up")
_OUT = ("gdn.out_proj", "attn.o", "mlp.down")


def check_supported(cfg: ModelConfig) -> None:
    if cfg.is_moe or cfg.has_conv_layers or cfg.sandwich_norm or not cfg.norm_zero_centered:
        raise ValueError("residual rotation is implemented for the dense hybrid family (zero-centred norms, no experts, no "
                         "short-conv or sandwich-norm layers)")


def fold_rotation(cfg: ModelConfig, w: Dict[str, torch.Tensor], spec: RotationSpec) -> Dict[str, torch.Tensor]:
    """The fp32 weight set of the rotated model (done before quantization; the source dict is not modified)."""
    check_supported(cfg)
    rt = rotation_tensors(spec)
    signs, mix = rt["rotation.signs"].double(), rt["rotation.mix"].double()
    out = dict(w)
    for i in range(cfg.num_hidden_layers):
        p = f"text.layers.{i}."
        for norm, names in (("input_layernorm", [n for n in _IN if not n.startswith("mlp.")]), ("post_attention_layernorm", ["mlp.gate_up"])):
            g = 1.0 + w[p + norm].double()
            for n in names:
                if p + n in w:
                    out[p + n] = apply_q(w[p + n].double() * g, spec, signs, mix).float()
            out[p + norm] = torch.zeros_like(w[p + norm])
        for n in _OUT:
            if p + n in w:
                out[p + n] = apply_q(w[p + n].double().T.contiguous(), spec, signs, mix).T.contiguous().float()
    out.update(rt)
    return out
