"""Audio front end of the Gemma-style family: WAV reader, framing, and the encoder-free audio embedder.

    frames [n, 640] f32 -> bf16 -> RMSNorm(640, no weight, eps 1e-6; fp32 math, bf16 result)
                        -> Linear(640 -> hidden, no bias; fp32 accumulate, bf16 result)          [n, hidden] bf16

The waveform is cast to bf16 BEFORE the norm (the embedder casts its input to the projection weight's dtype), and the rows
are NOT multiplied by the embedding scale: they overwrite the (already scaled) token embeddings at the audio placeholder
positions.  A clip is a few hundred rows, so this runs on the host once per clip and the rows enter the model through the
same embedding-override path as image rows (reference: src/audio/audio_embed.h:1-30).
"""
from __future__ import annotations

import io
import struct
from typing import Tuple

import torch

FRAME = 640                      # samples per row: 40 ms at 16 kHz
SAMPLE_RATE = 16000
WEIGHT_NAME = "audio.embed_audio.embedding_projection.weight"


def read_wav(data: bytes) -> Tuple[torch.Tensor, int]:
    """RIFF/WAVE bytes -> (mono float32 waveform in [-1, 1], sample rate).  PCM 8/16/24/32-bit and IEEE float 32/64,
    WAVE_FORMAT_EXTENSIBLE included; channels are averaged."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    at, fmt, pcm = 12, None, None
    while at + 8 <= len(data):
        tag, size = data[at:at + 4], struct.unpack_from("<I", data, at + 4)[0]
        body = data[at + 8:at + 8 + size]
        if tag == b"fmt ":
            if size < 16:
                raise ValueError("short fmt chunk")
            code, ch, rate, _, _, bits = struct.unpack_from("<HHIIHH", body, 0)
            if code == 0xFFFE and size >= 26:
                code = struct.unpack_from("<H", body, 24)[0]          # sub-format GUID's first field
            fmt = (code, ch, rate, bits)
        elif tag == b"data":
            pcm = body
        at += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError("WAVE file without fmt or data chunk")
    code, ch, rate, bits = fmt
    if ch < 1:
        raise ValueError("WAVE file with no channels")
    import numpy as np
    if code == 1 and bits == 16:
        x = np.frombuffer(pcm, dtype="<i2").astype(np.float32) / 32768.0
    elif code == 1 and bits == 8:
        x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif code == 1 and bits == 24:
        b = np.frombuffer(pcm[:len(pcm) // 3 * 3], dtype=np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = (np.where(v >= 1 << 23, v - (1 << 24), v)).astype(np.float32) / float(1 << 23)
    elif code == 1 and bits == 32:
        x = np.frombuffer(pcm, dtype="<i4").astype(np.float32) / float(1 << 31)
    elif code == 3 and bits == 32:
        x = np.frombuffer(pcm, dtype="<f4").astype(np.float32)
    elif code == 3 and bits == 64:
        x = np.frombuffer(pcm, dtype="<f8").astype(np.float32)
    else:
        raise ValueError(f"unsupported WAVE encoding (format {code}, {bits} bits)")
    x = x[:len(x) // ch * ch].reshape(-1, ch).mean(axis=1)
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)), int(rate)


def write_wav(wave: torch.Tensor, rate: int = SAMPLE_RATE) -> bytes:
    """Mono float waveform -> 16-bit PCM WAVE bytes (for tests and tools)."""
    pcm = (wave.float().clamp(-1, 1) * 32767.0).round().to(torch.int16).numpy().tobytes()
    head = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVE" + b"fmt " + struct.pack("<IHHIIHH", 16, 1, 1, rate, rate * 2, 2, 16)
    return head + b"data" + struct.pack("<I", len(pcm)) + pcm


def resample(wave: torch.Tensor, rate: int, to: int = SAMPLE_RATE) -> torch.Tensor:
    """Linear-interpolation resampling (clips that are not already at the model's rate)."""
    if rate == to or wave.numel() == 0:
        return wave
    n = max(1, int(round(wave.numel() * to / rate)))
    pos = torch.arange(n, dtype=torch.float64) * (rate / to)
    i0 = pos.floor().long().clamp(0, wave.numel() - 1)
    i1 = (i0 + 1).clamp(0, wave.numel() - 1)
    f = (pos - i0).float()
    return wave[i0] * (1 - f) + wave[i1] * f


def frame_waveform(wave: torch.Tensor, frame: int = FRAME) -> torch.Tensor:
    """[samples] -> [ceil(samples / frame), frame], the tail padded with zeros."""
    n = (wave.numel() + frame - 1) // frame
    out = torch.zeros(max(n, 0) * frame, dtype=torch.float32)
    out[:wave.numel()] = wave.float()
    return out.view(n, frame)


class AudioEmbedder:
    def __init__(self, weight: torch.Tensor, eps: float = 1e-6):
        """``weight`` [hidden, frame] (any float dtype; used as bf16 values)."""
        self.w = weight.detach().to(torch.bfloat16).float().cpu()
        self.eps = eps

    @property
    def in_dim(self) -> int:
        return self.w.shape[1]

    @property
    def out_dim(self) -> int:
        return self.w.shape[0]

    def embed(self, frames: torch.Tensor) -> torch.Tensor:
        """[n, frame] f32 -> [n, hidden] bf16; every row depends on its own frame only (any batching gives the same bits)."""
        if frames.dim() != 2 or frames.shape[1] != self.in_dim:
            raise ValueError(f"frames must be [n, {self.in_dim}]")
        x = frames.to(torch.bfloat16).float()
        x = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)).to(torch.bfloat16).float()
        return (x @ self.w.T).to(torch.bfloat16)

    def embed_clip(self, wav_bytes: bytes) -> torch.Tensor:
        wave, rate = read_wav(wav_bytes)
        return self.embed(frame_waveform(resample(wave, rate)))


def load_audio_embedder(weights) -> AudioEmbedder:
    """From a weight dict that holds the projection (a container converted with the audio tensor kept)."""
    if WEIGHT_NAME not in weights:
        raise ValueError(f"the model was converted without its audio projection ({WEIGHT_NAME})")
    w = weights[WEIGHT_NAME]
    if w.dim() != 2:
        raise ValueError("audio projection must be [hidden, frame]")
    return AudioEmbedder(w)
