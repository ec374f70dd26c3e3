"""Vision tower: host preprocessing and the device ViT encoder that turns images into text-width embeddings.

Host half (CPU): ``smart_resize`` (area-bounded, multiple-of-28 sides), antialiased bicubic resize, normalisation,
patches in 2x2-merge-major order, (row, column) position ids, bilinear taps into the learned position table and
one attention segment per frame (reference: src/vision/preprocess.h:1-40, position_ids.*, vision_index.*).
Device half: patch-embed product -> position embedding -> ``depth`` blocks of {LayerNorm, qkv + bias, axial rope,
bidirectional segment attention, projection, GELU-tanh MLP} -> merger {LayerNorm, fc1 over 2x2 neighbours, GELU-erf,
fc2} (reference: src/vision/vision_tower.h:1-45, docs/architecture.md:174-201).  The dense bf16 products are plain
library GEMMs (torch); LayerNorm, bias+GELU, rope and attention are this package's kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..native import c_f32, c_int, c_ptr, register_cuda_sig

BF = torch.bfloat16
register_cuda_sig("r4dxb_vit_rope", c_int, [c_ptr, c_ptr, c_int, c_int, c_int, c_f32, c_ptr])
register_cuda_sig("r4dxb_vit_attention", c_int, [c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr])


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 5120
    num_position_embeddings: int = 2304      # a square table (48 x 48)
    rope_theta: float = 10000.0
    layer_norm_eps: float = 1e-6
    image_mean: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    image_std: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    min_pixels: int = 64 * 64
    max_pixels: int = 16384 * 32 * 32

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @staticmethod
    def from_weights(w: Dict[str, torch.Tensor], **overrides) -> "VisionConfig":
        """The geometry a stored tower implies (containers carry the tensors, not a separate vision config): sizes from
        the tensor shapes, head count from the family's head width of 72 where it divides the hidden size."""
        H, pd = w["patch_embed.weight"].shape
        depth = 1 + max(int(k.split(".")[1]) for k in w if k.startswith("blocks."))
        merged = w["merger.fc1.weight"].shape[0]
        merge = int(round(math.sqrt(merged // H)))
        c = VisionConfig()
        patch = int(round(math.sqrt(pd / (c.in_channels * c.temporal_patch_size))))
        kw = dict(depth=depth, hidden_size=H, num_heads=(H // 72 if H % 72 == 0 else c.num_heads), intermediate_size=w["blocks.0.fc1.weight"].shape[0],
                  patch_size=patch, spatial_merge_size=merge, out_hidden_size=w["merger.fc2.weight"].shape[0],
                  num_position_embeddings=w["pos_embed"].shape[0])
        kw.update(overrides)
        return VisionConfig(**kw)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


def tiny_vision_config() -> VisionConfig:
    """Two blocks with the 72-wide heads of the full tower, narrow everywhere else."""
    return VisionConfig(depth=2, hidden_size=144, num_heads=2, intermediate_size=256, patch_size=8, out_hidden_size=256,
                        num_position_embeddings=64, max_pixels=256 * 256)


# ---------------------------------------------------------------- host half -----------------------------------
def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Sides rounded to multiples of ``factor`` with the area clamped to [min_pixels, max_pixels], aspect kept."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def preprocess_image(img: torch.Tensor, cfg: VisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """img: uint8 [H, W, 3].  Returns (patches fp32 [T, patch_dim] in merge-major order, grid (t, h, w) in patches)."""
    ps, m, tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    H, W = int(img.shape[0]), int(img.shape[1])
    h, w = smart_resize(H, W, ps * m, cfg.min_pixels, cfg.max_pixels)
    x = img.permute(2, 0, 1).unsqueeze(0).float()
    x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255).round_()
    x = x / 255.0
    mean = torch.tensor(cfg.image_mean).view(1, 3, 1, 1)
    std = torch.tensor(cfg.image_std).view(1, 3, 1, 1)
    x = (x - mean) / std
    x = x.repeat(tp, 1, 1, 1)                                   # a still image fills every temporal slot
    gh, gw = h // ps, w // ps
    x = x.view(1, tp, 3, gh // m, m, ps, gw // m, m, ps)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                    # [t, gh/m, gw/m, m, m, C, tp, ps, ps]
    return x.reshape(gh * gw, cfg.patch_dim).contiguous(), (1, gh, gw)


def position_ids(grid: Tuple[int, int, int], merge: int) -> torch.Tensor:
    """(row, column) of every patch, in the merge-major token order, repeated per frame: int32 [T, 2]."""
    t, gh, gw = grid
    hh = torch.arange(gh).view(gh // merge, 1, merge, 1).expand(gh // merge, gw // merge, merge, merge)
    ww = torch.arange(gw).view(1, gw // merge, 1, merge).expand(gh // merge, gw // merge, merge, merge)
    ids = torch.stack([hh.reshape(-1), ww.reshape(-1)], -1)
    return ids.repeat(t, 1).to(torch.int32)


def pos_embed_taps(grid: Tuple[int, int, int], side: int, merge: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Bilinear taps of the [side x side] learned table for a gh x gw grid: (indices int64 [T, 4], weights fp32 [T, 4])."""
    t, gh, gw = grid
    ys = torch.linspace(0, side - 1, gh)
    xs = torch.linspace(0, side - 1, gw)
    y0, x0 = ys.floor().long(), xs.floor().long()
    y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
    fy, fx = (ys - y0).view(gh, 1), (xs - x0).view(1, gw)
    idx = torch.stack([y0.view(gh, 1) * side + x0.view(1, gw), y0.view(gh, 1) * side + x1.view(1, gw),
                       y1.view(gh, 1) * side + x0.view(1, gw), y1.view(gh, 1) * side + x1.view(1, gw)], -1)
    wts = torch.stack([(1 - fy) * (1 - fx), (1 - fy) * fx, fy * (1 - fx), fy * fx], -1)

    def merge_major(a):
        a = a.view(gh // merge, merge, gw // merge, merge, 4).permute(0, 2, 1, 3, 4)
        return a.reshape(gh * gw, 4)

    return merge_major(idx).repeat(t, 1), merge_major(wts.expand(gh, gw, 4)).repeat(t, 1).float()


def segment_offsets(grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
    """cu_seqlens: attention is confined to one frame of one image."""
    cu = [0]
    for t, gh, gw in grids:
        for _ in range(t):
            cu.append(cu[-1] + gh * gw)
    return torch.tensor(cu, dtype=torch.int32)


# ---------------------------------------------------------------- weights -------------------------------------
def init_vision_weights(cfg: VisionConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    n = lambda *s, sc=0.05: torch.randn(*s, generator=g) * sc
    H, I = cfg.hidden_size, cfg.intermediate_size
    w = {"patch_embed.weight": n(H, cfg.patch_dim), "patch_embed.bias": n(H), "pos_embed": n(cfg.num_position_embeddings, H)}
    for i in range(cfg.depth):
        p = f"blocks.{i}."
        w.update({p + "norm1.weight": 1 + n(H), p + "norm1.bias": n(H), p + "norm2.weight": 1 + n(H), p + "norm2.bias": n(H),
                  p + "qkv.weight": n(3 * H, H), p + "qkv.bias": n(3 * H), p + "proj.weight": n(H, H), p + "proj.bias": n(H),
                  p + "fc1.weight": n(I, H), p + "fc1.bias": n(I), p + "fc2.weight": n(H, I), p + "fc2.bias": n(H)})
    M = H * cfg.spatial_merge_size ** 2
    w.update({"merger.norm.weight": 1 + n(H), "merger.norm.bias": n(H), "merger.fc1.weight": n(M, M), "merger.fc1.bias": n(M),
              "merger.fc2.weight": n(cfg.out_hidden_size, M), "merger.fc2.bias": n(cfg.out_hidden_size)})
    return w


# ---------------------------------------------------------------- fp32 reference ------------------------------
def _rope_ref(x: torch.Tensor, pos_hw: torch.Tensor, theta: float) -> torch.Tensor:
    T, H, D = x.shape
    half, quarter = D // 2, D // 4
    inv = theta ** (-(torch.arange(quarter).float() * 2.0 / half))
    ang = torch.cat([pos_hw[:, :1].float() * inv, pos_hw[:, 1:].float() * inv], -1)      # [T, half]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def vision_forward_reference(cfg: VisionConfig, w: Dict[str, torch.Tensor], patches, pos_hw, idx, wts, cu) -> torch.Tensor:
    """fp32 CPU restatement of the tower; bf16 rounding at the same points as the device path."""
    r = lambda t: t.to(BF).float()
    W = {k: r(v) for k, v in w.items()}
    T, H, Hn, D = patches.shape[0], cfg.hidden_size, cfg.num_heads, cfg.head_dim
    x = r(F.linear(r(patches), W["patch_embed.weight"], W["patch_embed.bias"]))
    x = r(x + (W["pos_embed"][idx] * wts[..., None]).sum(1))
    for i in range(cfg.depth):
        p = f"blocks.{i}."
        h = r(F.layer_norm(x, (H,), W[p + "norm1.weight"], W[p + "norm1.bias"], cfg.layer_norm_eps))
        qkv = r(F.linear(h, W[p + "qkv.weight"], W[p + "qkv.bias"])).view(T, 3, Hn, D)
        q, k, v = r(_rope_ref(qkv[:, 0], pos_hw, cfg.rope_theta)), r(_rope_ref(qkv[:, 1], pos_hw, cfg.rope_theta)), qkv[:, 2]
        o = torch.zeros(T, Hn, D)
        for s in range(len(cu) - 1):
            a, b = int(cu[s]), int(cu[s + 1])
            att = torch.einsum("qhd,khd->hqk", q[a:b], k[a:b]) / math.sqrt(D)
            o[a:b] = torch.einsum("hqk,khd->qhd", att.softmax(-1), v[a:b])
        x = r(x + r(F.linear(r(o).reshape(T, H), W[p + "proj.weight"], W[p + "proj.bias"])))
        h = r(F.layer_norm(x, (H,), W[p + "norm2.weight"], W[p + "norm2.bias"], cfg.layer_norm_eps))
        h = r(F.gelu(r(F.linear(h, W[p + "fc1.weight"])) + W[p + "fc1.bias"], approximate="tanh"))
        x = r(x + r(F.linear(h, W[p + "fc2.weight"], W[p + "fc2.bias"])))
    m = cfg.spatial_merge_size ** 2
    h = r(F.layer_norm(x, (H,), W["merger.norm.weight"], W["merger.norm.bias"], cfg.layer_norm_eps)).view(T // m, m * H)
    h = r(F.gelu(r(F.linear(h, W["merger.fc1.weight"])) + W["merger.fc1.bias"]))
    return r(F.linear(h, W["merger.fc2.weight"], W["merger.fc2.bias"]))


# ---------------------------------------------------------------- device tower --------------------------------
class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: Dict[str, torch.Tensor], device: str = "cuda"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = {k: v.to(self.device, BF).contiguous() for k, v in weights.items()}

    def forward(self, patches: torch.Tensor, pos_hw: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor,
                cu: torch.Tensor) -> torch.Tensor:
        """patches fp32/bf16 [T, patch_dim] -> bf16 [T / merge^2, out_hidden] on the device."""
        from .. import native
        from ..ops import kernels as K
        L = native.cuda()
        cfg, w, dev = self.cfg, self.w, self.device
        T, H, Hn, D = patches.shape[0], cfg.hidden_size, cfg.num_heads, cfg.head_dim
        st = torch.cuda.current_stream().cuda_stream
        pos_hw = pos_hw.to(dev, torch.int32).contiguous()
        cu_d = cu.to(dev, torch.int32).contiguous()
        x = K.linear_tc(w["patch_embed.weight"], patches.to(dev, BF), bias=w["patch_embed.bias"])
        pe = (w["pos_embed"][idx.to(dev)].float() * wts.to(dev)[..., None]).sum(1)
        x = (x.float() + pe).to(BF)
        for i in range(cfg.depth):
            p = f"blocks.{i}."
            h = K.layernorm(x, w[p + "norm1.weight"], w[p + "norm1.bias"], cfg.layer_norm_eps)
            qkv = K.linear_tc(w[p + "qkv.weight"], h, bias=w[p + "qkv.bias"])
            rc = L.r4dxb_vit_rope(qkv.data_ptr(), pos_hw.data_ptr(), T, Hn, D, cfg.rope_theta, st)
            assert rc == 0, rc
            o = torch.empty(T, H, dtype=BF, device=dev)
            rc = L.r4dxb_vit_attention(qkv.data_ptr(), o.data_ptr(), cu_d.data_ptr(), cu_d.numel() - 1, T, Hn, D, st)
            assert rc == 0, rc
            x = K.linear_tc(w[p + "proj.weight"], o, bias=w[p + "proj.bias"], residual=x)
            h = K.layernorm(x, w[p + "norm2.weight"], w[p + "norm2.bias"], cfg.layer_norm_eps)
            h = K.linear_tc(w[p + "fc1.weight"], h, bias=w[p + "fc1.bias"], act=1)
            x = K.linear_tc(w[p + "fc2.weight"], h, bias=w[p + "fc2.bias"], residual=x)
        m = cfg.spatial_merge_size ** 2
        h = K.layernorm(x, w["merger.norm.weight"], w["merger.norm.bias"], cfg.layer_norm_eps).view(T // m, m * H)
        h = K.linear_tc(w["merger.fc1.weight"], h.contiguous(), bias=w["merger.fc1.bias"], act=2)
        return K.linear_tc(w["merger.fc2.weight"], h, bias=w["merger.fc2.bias"])

    def encode_images(self, images: List[torch.Tensor]) -> torch.Tensor:
        """uint8 [H, W, 3] images -> bf16 embeddings [sum tokens, out_hidden] ready to replace image placeholders."""
        cfg = self.cfg
        side = int(round(math.sqrt(cfg.num_position_embeddings)))
        ps, grids, ids, taps_i, taps_w = [], [], [], [], []
        for img in images:
            p, g = preprocess_image(img, cfg)
            ps.append(p); grids.append(g)
            ids.append(position_ids(g, cfg.spatial_merge_size))
            ti, tw = pos_embed_taps(g, side, cfg.spatial_merge_size)
            taps_i.append(ti); taps_w.append(tw)
        return self.forward(torch.cat(ps), torch.cat(ids), torch.cat(taps_i), torch.cat(taps_w), segment_offsets(grids))
