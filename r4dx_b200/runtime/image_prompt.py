"""Image parts of a chat request: decoding, placeholder accounting and prompt assembly.

An ``image_url`` part carries a ``data:`` URI (base64 PNG / JPEG / anything Pillow reads) or raw RGB bytes with
explicit dimensions.  In the rendered prompt every image becomes ``n`` copies of the image placeholder token, where
``n`` is the number of merged patches the vision tower will produce for it, so that the tower's output rows replace
exactly those tokens' embeddings (reference: src/vision/image_prompt.h, src/server/prefix_state.h image keys).
"""
from __future__ import annotations

import base64
import io
from typing import List, Sequence, Tuple

import torch

MARK = "\x00<r4dxb-image-%d>\x00"
AUDIO_MARK = "\x00<r4dxb-audio-%d>\x00"


def decode_audio(part) -> bytes:
    """An ``input_audio`` content part ({"data": base64, "format": "wav"}) or a ``data:`` URI -> WAVE bytes."""
    if isinstance(part, dict):
        fmt = str(part.get("format", "wav")).lower()
        if fmt != "wav":
            raise ValueError(f"audio format {fmt!r} is not supported (wav only)")
        data = part.get("data", "")
    else:
        data = str(part)
    if data.startswith("data:"):
        head, _, data = data.partition(",")
        if ";base64" not in head:
            raise ValueError("audio data URI must be base64")
    try:
        return base64.b64decode(data, validate=False)
    except Exception:
        raise ValueError("audio data is not valid base64")


def assemble_media_prompt(rendered: str, spans: Sequence[Tuple[str, int, int]], encode) -> List[int]:
    """Tokenizes the text around media markers.  ``spans``: (marker, placeholder token id, count) in any order; each marker is
    replaced by ``count`` copies of its token where it stands in the rendered prompt."""
    found = []
    for marker, tok, n in spans:
        at = rendered.find(marker)
        if at < 0:
            raise ValueError("a media part has no placeholder in the rendered prompt")
        found.append((at, marker, tok, n))
    ids: List[int] = []
    cur = 0
    for at, marker, tok, n in sorted(found):
        ids += encode(rendered[cur:at]) + [tok] * n
        cur = at + len(marker)
    return ids + encode(rendered[cur:])


def decode_image(url: str) -> torch.Tensor:
    """``data:[mime];base64,....`` -> uint8 [H, W, 3]."""
    if not url.startswith("data:"):
        raise ValueError("only data: URIs are accepted for images (no network access from the server)")
    head, _, payload = url.partition(",")
    if ";base64" not in head:
        raise ValueError("image data URI must be base64")
    raw = base64.b64decode(payload)
    from PIL import Image
    import numpy as np
    img = Image.open(io.BytesIO(raw)).convert("RGB")
    return torch.from_numpy(np.asarray(img, dtype=np.uint8).copy())


def image_token_count(img: torch.Tensor, vcfg) -> int:
    if hasattr(vcfg, "token_count"):           # families with their own sizing rule (soft-token budgets)
        return int(vcfg.token_count(img))
    from ..models.vision import smart_resize
    f = vcfg.patch_size * vcfg.spatial_merge_size
    h, w = smart_resize(int(img.shape[0]), int(img.shape[1]), f, vcfg.min_pixels, vcfg.max_pixels)
    return (h // f) * (w // f)


def assemble_prompt(rendered: str, counts: Sequence[int], encode, image_token_id: int) -> List[int]:
    """Tokenizes the text around the image markers and puts ``counts[i]`` placeholder tokens where marker i stood."""
    ids: List[int] = []
    rest = rendered
    for i, n in enumerate(counts):
        m = MARK % i
        before, sep, rest = rest.partition(m)
        if not sep:
            raise ValueError(f"image {i} has no placeholder in the rendered prompt")
        ids += encode(before) + [image_token_id] * n
    return ids + encode(rest)


def split_content(parts) -> Tuple[str, List[str]]:
    """OpenAI content parts -> (text with one marker per image, image URLs in order)."""
    text, urls = [], []
    for p in parts:
        t = p.get("type")
        if t == "text":
            text.append(p.get("text", ""))
        elif t == "image_url":
            u = p.get("image_url")
            urls.append(u.get("url", "") if isinstance(u, dict) else str(u))
            text.append("\x00IMG\x00")
        else:
            raise ValueError(f"unsupported content part type {t!r}")
    return "".join(text), urls
