"""Host half of the Gemma-style (encoder-free) vision path: image preprocessor, placeholder expansion, image-block
bookkeeping for the bidirectional in-block mask, prefill chunk planning that never splits a block, and a host reference of
the embedder chain.  CPU only.  (reference: src/vision/gemma_vision.h:1-140.)

Preprocessor: antialiased bicubic resize to the largest (h, w), both multiples of 48, with h * w <= max_soft_tokens * 48^2
(aspect preserving, floor; small images are grown too), rescale by 1/255 (no mean / std), 16-pixel patches merged 3 x 3
into 48 x 48 x 3 HWC rasters (6912 values) in row-major order of the merged grid; a merged patch's position is (x, y) in
merged-grid cells.  Soft tokens = (h / 48) * (w / 48).

Mask: an image block is a maximal run of image soft tokens.  On sliding-window layers a query inside a block may also
attend every key of its block (up to the block's last position); full-attention layers and decode stay causal.  A block
must therefore sit inside ONE prefill chunk: all its keys are written before its first query runs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch
import torch.nn.functional as F

PATCH, POOL = 16, 3
SIDE = PATCH * POOL                       # 48
PATCH_DIM = SIDE * SIDE * 3               # 6912
SOFT_TOKEN_BUDGETS = (70, 140, 280, 560, 1120)
MAX_IMAGE_BLOCK_TOKENS = 288              # a single image's block must fit one prefill chunk and the sliding KV window


def target_size(height: int, width: int, max_soft_tokens: int = 280) -> Tuple[int, int]:
    """Largest aspect-preserving (h, w), both multiples of 48, with h * w within the soft-token budget."""
    if max_soft_tokens not in SOFT_TOKEN_BUDGETS:
        raise ValueError(f"max_soft_tokens must be one of {SOFT_TOKEN_BUDGETS}")
    if height <= 0 or width <= 0:
        raise ValueError("empty image")
    budget = max_soft_tokens * SIDE * SIDE
    f = math.sqrt(budget / (height * width))
    h = int(math.floor(height * f / SIDE)) * SIDE
    w = int(math.floor(width * f / SIDE)) * SIDE
    if h == 0 or w == 0:
        raise ValueError("image too elongated for the soft-token budget (one side rounds to zero)")
    return h, w


def preprocess(img: torch.Tensor, max_soft_tokens: int = 280) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
    """uint8 [H, W, 3] -> (pixel_values fp32 [n, 6912], positions int32 [n, 2] as (x, y), merged grid (rows, cols))."""
    H, W = int(img.shape[0]), int(img.shape[1])
    h, w = target_size(H, W, max_soft_tokens)
    x = img.permute(2, 0, 1).unsqueeze(0).float()
    if (h, w) != (H, W):
        x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255).round_()
    x = (x * (1.0 / 255.0))[0]                                   # [3, h, w]
    gh, gw = h // SIDE, w // SIDE
    r = x.view(3, gh, SIDE, gw, SIDE).permute(1, 3, 2, 4, 0)     # [gh, gw, 48, 48, 3]: HWC raster per merged patch
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    pos = torch.stack([xs.reshape(-1), ys.reshape(-1)], 1).to(torch.int32)
    return r.reshape(gh * gw, PATCH_DIM).contiguous(), pos, (gh, gw)


# ---- prompt expansion and block bookkeeping --------------------------------------------------------------
def expand_placeholders(tokens: Sequence[int], soft_tokens: Sequence[int], image_id: int, boi_id: int, eoi_id: int):
    """One image placeholder per image -> boi + n x placeholder + eoi.  Returns (tokens, [(offset of first soft token, n)])."""
    out: List[int] = []
    spans: List[Tuple[int, int]] = []
    k = 0
    for t in tokens:
        if t != image_id:
            out.append(int(t))
            continue
        if k >= len(soft_tokens):
            raise ValueError("more image placeholders than images")
        out.append(boi_id)
        spans.append((len(out), int(soft_tokens[k])))
        out += [image_id] * int(soft_tokens[k])
        out.append(eoi_id)
        k += 1
    if k != len(soft_tokens):
        raise ValueError(f"{k} image placeholders for {len(soft_tokens)} images")
    return out, spans


def find_blocks(tokens: Sequence[int], image_id: int, base: int = 0) -> List[Tuple[int, int]]:
    """Maximal runs of the image token as absolute [start, end) positions."""
    blocks, start = [], None
    for i, t in enumerate(tokens):
        if t == image_id and start is None:
            start = i
        elif t != image_id and start is not None:
            blocks.append((base + start, base + i))
            start = None
    if start is not None:
        blocks.append((base + start, base + len(tokens)))
    return blocks


def plan_prefill_chunks(total: int, blocks: Sequence[Tuple[int, int]], max_rows: int,
                        max_block: int = MAX_IMAGE_BLOCK_TOKENS) -> List[Tuple[int, int]]:
    """Splits ``total`` rows into (start, len) chunks of at most ``max_rows`` rows that never cut an image block: a block
    that would not fit ends the chunk at its start; a block that starts a chunk extends the chunk to the block's end."""
    for a, b in blocks:
        if not 0 <= a < b <= total:
            raise ValueError("image block outside the prompt")
        if b - a > max_block:
            raise ValueError(f"image block of {b - a} tokens exceeds the limit of {max_block}")
    chunks, at = [], 0
    while at < total:
        end = min(total, at + max_rows)
        for a, b in blocks:
            if a < end < b:                         # the chunk would cut this block
                end = a if a > at else b
                break
        chunks.append((at, end - at))
        at = end
    return chunks


def key_limit_ext(abs_start: int, length: int, blocks: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """Per row of [abs_start, abs_start + length): the last key position of the row's block, or -1 (plain causal)."""
    out = torch.full((length,), -1, dtype=torch.int32)
    for a, b in blocks:
        lo, hi = max(a, abs_start), min(b, abs_start + length)
        if lo < hi:
            out[lo - abs_start:hi - abs_start] = b - 1
    return out


def dense_mask(T: int, window: int, bidirectional: bool, blocks: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """Reference mask [T, T] (True = attend): (causal OR same block when ``bidirectional``) AND window (window <= 0: none)."""
    q = torch.arange(T)[:, None]
    k = torch.arange(T)[None, :]
    allow = k <= q
    if bidirectional:
        blk = torch.full((T,), -1, dtype=torch.long)
        for i, (a, b) in enumerate(blocks):
            blk[a:b] = i
        allow = allow | ((blk[:, None] == blk[None, :]) & (blk[:, None] >= 0))
    if window > 0:
        allow = allow & (k > q - window)
    return allow


# ---- embedder host reference ---------------------------------------------------------------------------------
def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def _layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return _bf((x - mu) * torch.rsqrt(var + eps) * w + b)


@dataclass
class GemmaEmbedderWeights:
    ln1_w: torch.Tensor            # [patch_dim]
    ln1_b: torch.Tensor
    dense_w: torch.Tensor          # [mm_dim, patch_dim]
    dense_b: torch.Tensor
    ln2_w: torch.Tensor            # [mm_dim]
    ln2_b: torch.Tensor
    pos_embedding: torch.Tensor    # [posemb_size, 2, mm_dim]: [.., 0] indexed by x, [.., 1] by y
    pos_norm_w: torch.Tensor       # [mm_dim]
    pos_norm_b: torch.Tensor
    proj_w: torch.Tensor           # [out_dim, mm_dim]
    eps: float = 1e-6


def embed_reference(pixels: torch.Tensor, positions: torch.Tensor, w: GemmaEmbedderWeights) -> torch.Tensor:
    """pixel_values [n, patch_dim] + positions [n, 2] -> rows [n, out_dim] (bf16 values in fp32), with a bf16 rounding after
    every op and fp32 accumulation inside the norms and the products:
        x = bf16(pixel); h = LN1(x); h = dense(h) + bias; h = LN2(h)
        pos = bf16(pos_embedding[x][0] + pos_embedding[y][1]); h = bf16(h + pos); h = pos_norm(h)
        h = RMSNorm_noscale(h); out = proj(h)"""
    f = lambda t: _bf(t.float())
    x = _bf(pixels.float())
    h = _layer_norm(x, f(w.ln1_w), f(w.ln1_b), w.eps)
    h = _bf(h @ f(w.dense_w).T + f(w.dense_b))
    h = _layer_norm(h, f(w.ln2_w), f(w.ln2_b), w.eps)
    pe = f(w.pos_embedding)
    pos = _bf(pe[positions[:, 0].long(), 0] + pe[positions[:, 1].long(), 1])
    h = _bf(h + pos)
    h = _layer_norm(h, f(w.pos_norm_w), f(w.pos_norm_b), w.eps)
    h = _bf(h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + w.eps))
    return _bf(h @ f(w.proj_w).T)


class GemmaEmbedder:
    """Device half of the encoder-free embedder: the chain of ``embed_reference`` with the two products on the
    tensor-core linear (bias fused) and the norms on the LayerNorm / RMSNorm kernels; the positional rows are two table
    gathers.  Rows come back in bf16, ready to override the image placeholders' embeddings.
    (reference: src/vision/gemma_vision.cpp runs the same chain on its GEMM library.)"""

    def __init__(self, w: GemmaEmbedderWeights, device="cuda"):
        BF = torch.bfloat16
        d = torch.device(device)
        t = lambda x: x.to(d, BF).contiguous()
        self.eps, self.device = w.eps, d
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = t(w.ln1_w), t(w.ln1_b), t(w.ln2_w), t(w.ln2_b)
        self.dense_w, self.dense_b, self.proj_w = t(w.dense_w), t(w.dense_b), t(w.proj_w)
        self.pos_embedding, self.pos_norm_w, self.pos_norm_b = t(w.pos_embedding), t(w.pos_norm_w), t(w.pos_norm_b)
        self.ones = torch.ones(w.proj_w.shape[1], dtype=BF, device=d)

    def embed(self, pixels: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        from ..ops import kernels as K
        BF = torch.bfloat16
        x = pixels.to(self.device, BF).contiguous()
        pos = positions.to(self.device, torch.long)
        h = K.layernorm(x, self.ln1_w, self.ln1_b, self.eps)
        h = K.linear_tc(self.dense_w, h, bias=self.dense_b)
        h = K.layernorm(h, self.ln2_w, self.ln2_b, self.eps)
        pe = (self.pos_embedding[pos[:, 0], 0].float() + self.pos_embedding[pos[:, 1], 1].float()).to(BF)
        h = K.residual_add(h, pe)
        h = K.layernorm(h, self.pos_norm_w, self.pos_norm_b, self.eps)
        h = K.rmsnorm(h, self.ones, self.eps, zero_centered=False)
        return K.linear_tc(self.proj_w, h)


EMBEDDER_FIELDS = ("ln1_w", "ln1_b", "dense_w", "dense_b", "ln2_w", "ln2_b", "pos_embedding", "pos_norm_w", "pos_norm_b", "proj_w")


def random_embedder_weights(out_dim: int, mm_dim: int = 256, posemb: int = 64, seed: int = 0) -> GemmaEmbedderWeights:
    """A random embedder for synthetic models and tests."""
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g) * 0.05
    return GemmaEmbedderWeights(1 + n(PATCH_DIM), n(PATCH_DIM), n(mm_dim, PATCH_DIM), n(mm_dim), 1 + n(mm_dim), n(mm_dim),
                                n(posemb, 2, mm_dim), 1 + n(mm_dim), n(mm_dim), n(out_dim, mm_dim))


class GemmaVisionFront:
    """What the serving layer needs of this family's image path: how many soft tokens an image takes, the rows for a list
    of images, and the fact that image rows form bidirectional blocks (the engine then passes the blocks to the prefill).
    Weights ride in the container as ``vision.embedder.<field>``."""

    bidirectional_blocks = True

    def __init__(self, w: GemmaEmbedderWeights, device="cuda", max_soft_tokens: int = 280):
        self.embedder = GemmaEmbedder(w, device)
        self.max_soft_tokens = max_soft_tokens
        self.posemb = w.pos_embedding.shape[0]

    @staticmethod
    def from_container_tensors(vw: dict, device="cuda") -> "GemmaVisionFront":
        missing = [f for f in EMBEDDER_FIELDS if "embedder." + f not in vw]
        if missing:
            raise ValueError(f"the container's vision tensors lack embedder.{missing[0]}")
        return GemmaVisionFront(GemmaEmbedderWeights(*[vw["embedder." + f].float() for f in EMBEDDER_FIELDS]), device)

    def token_count(self, img: torch.Tensor) -> int:
        h, w = target_size(int(img.shape[0]), int(img.shape[1]), self.max_soft_tokens)
        return (h // SIDE) * (w // SIDE)

    def encode_images(self, images) -> torch.Tensor:
        rows = []
        for img in images:
            px, pos, (gh, gw) = preprocess(img, self.max_soft_tokens)
            if max(gh, gw) > self.posemb:
                raise ValueError(f"image grid {gh}x{gw} exceeds the positional table ({self.posemb})")
            rows.append(self.embedder.embed(px, pos))
        return torch.cat(rows, 0)
