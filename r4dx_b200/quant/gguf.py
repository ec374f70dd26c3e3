"""GGUF reader: header, metadata, tensor directory, dequantisation of the common block formats, and the mapping of a
dense Llama-style / Qwen-style GGUF checkpoint onto this engine's weight names (the converter then re-quantizes it).

File layout (GGUF v2/v3, little endian): magic "GGUF", u32 version, u64 tensor count, u64 metadata count, metadata
(key string, u32 value type, value), tensor infos (name, u32 n_dims, u64 dims[n_dims] innermost first, u32 ggml type,
u64 offset), padding to ``general.alignment`` (default 32), tensor data.
(reference: the converter's GGUF reader and the drafter's GGUF import, src/convert/main.cpp:1-30 flags
``--dflash-gguf``; dequantisation checks in tests/reference.)

Block formats decoded here (values per block / bytes per block):
  F32, F16, BF16; Q8_0 (32 / 34: f16 d, 32 x i8); Q4_0 (32 / 18: f16 d, 16 bytes of nibbles, value (q - 8) d, low nibbles
  are elements 0..15, high nibbles 16..31); Q4_1 (32 / 20: f16 d, f16 m, value q d + m); Q5_0 (32 / 22: f16 d, u32 high bits);
  Q4_K (256 / 144: f16 d, f16 dmin, 12 bytes of 6-bit scales and mins for 8 sub-blocks, 128 bytes of nibbles);
  Q6_K (256 / 210: 128 bytes low nibbles, 64 bytes high 2-bit pairs, 16 x i8 scales, f16 d).
The K-quant decoders are checked against scalar restatements of the format only: no file written by another tool was
available to test against.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np
import torch

from ..config import ModelConfig

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 3, 6, 8, 12, 14, 30
# type -> (values per block, bytes per block)
BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q8_0: (32, 34), GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20),
         GGML_Q5_0: (32, 22), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class GgufTensor:
    name: str
    shape: Tuple[int, ...]        # outermost first (torch order)
    ggml_type: int
    offset: int                   # absolute file offset
    nbytes: int


class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata: Dict[str, object] = {}
        self.tensors: Dict[str, GgufTensor] = {}
        self._parse()

    # ---- parsing --------------------------------------------------------------------------------
    def _parse(self) -> None:
        mm = self._mm
        if mm[:4] != b"GGUF":
            raise ValueError(f"{self.path}: not a GGUF file")
        self.version, = struct.unpack_from("<I", mm, 4)
        if self.version < 2:
            raise ValueError("GGUF v1 (32-bit counts) is not supported")
        n_tensors, n_kv = struct.unpack_from("<QQ", mm, 8)
        self._at = 24
        for _ in range(n_kv):
            key = self._string()
            vtype, = self._unpack("<I")
            self.metadata[key] = self._value(vtype)
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            nd, = self._unpack("<I")
            dims = [self._unpack("<Q")[0] for _ in range(nd)]
            gtype, = self._unpack("<I")
            off, = self._unpack("<Q")
            infos.append((name, tuple(reversed(dims)), gtype, off))
        align = int(self.metadata.get("general.alignment", 32))
        base = (self._at + align - 1) // align * align
        for name, shape, gtype, off in infos:
            if gtype not in BLOCK:
                raise ValueError(f"{name}: ggml type {gtype} is not supported")
            per, size = BLOCK[gtype]
            n = int(np.prod(shape)) if shape else 1
            if n % per:
                raise ValueError(f"{name}: {n} elements do not fill whole blocks of {per}")
            self.tensors[name] = GgufTensor(name, shape, gtype, base + off, n // per * size)
            if base + off + n // per * size > len(mm):
                raise ValueError(f"{name}: data runs past the end of the file")

    def _unpack(self, fmt: str):
        v = struct.unpack_from(fmt, self._mm, self._at)
        self._at += struct.calcsize(fmt)
        return v

    def _string(self) -> str:
        n, = self._unpack("<Q")
        s = self._mm[self._at:self._at + n].decode("utf-8", errors="replace")
        self._at += n
        return s

    def _value(self, vtype: int):
        if vtype in _SCALAR:
            return self._unpack(_SCALAR[vtype])[0]
        if vtype == 8:
            return self._string()
        if vtype == 9:
            etype, = self._unpack("<I")
            n, = self._unpack("<Q")
            return [self._value(etype) for _ in range(n)]
        raise ValueError(f"unknown metadata value type {vtype}")

    # ---- data -----------------------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=t.offset)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor dequantised to fp32, shaped outermost-first."""
        t = self.tensors[name]
        return torch.from_numpy(dequantize(self.raw(name), t.ggml_type).reshape(t.shape).copy())

    def close(self) -> None:
        self._mm.close()
        self._f.close()


# ---- block formats ---------------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def dequantize(raw: np.ndarray, gtype: int) -> np.ndarray:
    """uint8 bytes of whole blocks -> flat fp32 values."""
    if gtype == GGML_F32:
        return raw.view(np.float32).copy()
    if gtype == GGML_F16:
        return raw.view(np.float16).astype(np.float32)
    if gtype == GGML_BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    per, size = BLOCK[gtype]
    b = raw.reshape(-1, size)
    if gtype == GGML_Q8_0:
        return (_f16(b[:, :2]) * b[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if gtype in (GGML_Q4_0, GGML_Q4_1):
        hdr = 2 if gtype == GGML_Q4_0 else 4
        q = b[:, hdr:]
        v = np.concatenate([q & 0xF, q >> 4], axis=1).astype(np.float32)
        d = _f16(b[:, :2])
        if gtype == GGML_Q4_0:
            return ((v - 8.0) * d).reshape(-1)
        return (v * d + _f16(b[:, 2:4])).reshape(-1)
    if gtype == GGML_Q5_0:
        d = _f16(b[:, :2])
        qh = np.ascontiguousarray(b[:, 2:6]).view(np.uint32)                       # [blocks, 1]
        q = b[:, 6:]
        lo = np.concatenate([q & 0xF, q >> 4], axis=1).astype(np.int32)            # [blocks, 32]
        hi = ((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32) << 4
        return (((lo | hi) - 16).astype(np.float32) * d).reshape(-1)
    if gtype == GGML_Q4_K:
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        s = b[:, 4:16].astype(np.int32)
        sc = np.empty((b.shape[0], 8), np.int32)
        mn = np.empty((b.shape[0], 8), np.int32)
        sc[:, :4], mn[:, :4] = s[:, 0:4] & 63, s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        q = b[:, 16:].reshape(-1, 4, 32)                                            # four 64-value chunks of 32 bytes
        vals = np.stack([q & 0xF, q >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)   # sub-blocks 2c (low), 2c+1 (high)
        out = vals * (d[:, :, None] * sc[:, :, None]) - dmin[:, :, None] * mn[:, :, None]
        return out.reshape(-1)
    if gtype == GGML_Q6_K:
        ql = b[:, :128].reshape(-1, 2, 64).astype(np.int32)
        qh = b[:, 128:192].reshape(-1, 2, 32).astype(np.int32)
        sc = b[:, 192:208].view(np.int8).reshape(-1, 2, 8).astype(np.float32)
        d = _f16(b[:, 208:210])
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q1 = ((l0 & 0xF) | ((qh & 3) << 4)) - 32
        q2 = ((l1 & 0xF) | (((qh >> 2) & 3) << 4)) - 32
        q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)) - 32
        q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)) - 32
        q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32)                   # [blocks, 2 halves, 4 groups, 32]
        idx = (np.arange(32) // 16)[None, :] + 2 * np.arange(4)[:, None]            # scale index of (group, l)
        scale = sc[:, :, idx]                                                       # [blocks, 2, 4, 32]
        return (q * scale * d[:, :, None, None]).reshape(-1)
    raise ValueError(f"ggml type {gtype} is not supported")


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """fp32 values (a multiple of 32) -> Q8_0 bytes; used to write test files and to round-trip imports."""
    x = x.reshape(-1, 32).astype(np.float32)
    d = np.abs(x).max(axis=1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(x / np.where(d > 0, d, 1.0)), 0).astype(np.int8)
    out = np.empty((x.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def write_gguf(path: str, metadata: Dict[str, object], tensors: Dict[str, Tuple[np.ndarray, int]], alignment: int = 32) -> None:
    """Minimal GGUF v3 writer: ``tensors`` name -> (fp32 array in torch order, ggml type in {F32, F16, BF16, Q8_0})."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2**32 else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(e) for e in v)
            if all(isinstance(e, int) for e in v):
                return struct.pack("<IIQ", 9, 5, len(v)) + b"".join(struct.pack("<i", e) for e in v)
            return struct.pack("<IIQ", 9, 6, len(v)) + b"".join(struct.pack("<f", float(e)) for e in v)
        raise TypeError(type(v))

    blobs, infos, off = [], b"", 0
    for name, (arr, gtype) in tensors.items():
        a = np.ascontiguousarray(arr, dtype=np.float32)
        if gtype == GGML_F32:
            data = a.tobytes()
        elif gtype == GGML_F16:
            data = a.astype(np.float16).tobytes()
        elif gtype == GGML_BF16:
            data = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        elif gtype == GGML_Q8_0:
            data = quantize_q8_0(a).tobytes()
        else:
            raise ValueError("writer supports F32, F16, BF16 and Q8_0")
        infos += s(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(a.shape))
        infos += struct.pack("<IQ", gtype, off)
        pad = (-len(data)) % alignment
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    md = dict(metadata)
    md.setdefault("general.alignment", alignment)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(md)) + b"".join(s(k) + val(v) for k, v in md.items()) + infos
    with open(path, "wb") as f:
        f.write(head + b"\0" * ((-len(head)) % alignment))
        for b_ in blobs:
            f.write(b_)


# ---- checkpoint import ------------------------------------------------------------------------------
_LAYER_NAMES = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
                "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
                "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm", "ffn_gate": "mlp.gate_proj",
                "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


def _unpermute_rope(w: torch.Tensor, heads: int) -> torch.Tensor:
    """Llama-architecture GGUF files store q/k projection rows with each head's rotary pairs interleaved
    ([head][d/2][2]); the engine (like the Hugging Face layout) keeps the two halves apart ([head][2][d/2])."""
    rows = w.shape[0]
    return w.reshape(heads, rows // heads // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape).contiguous()


def config_from_gguf(g: GgufFile) -> ModelConfig:
    md = g.metadata
    arch = str(md.get("general.architecture", "llama"))
    if arch not in ("llama", "qwen2", "qwen3", "mistral", "qwen2moe", "qwen3moe"):
        raise ValueError(f"GGUF architecture {arch!r} has no mapping onto this engine's decoders")
    k = lambda name, default=None: md.get(f"{arch}.{name}", default)
    H, L, heads = int(k("embedding_length")), int(k("block_count")), int(k("attention.head_count"))
    kv = int(k("attention.head_count_kv", heads))
    vocab = int(k("vocab_size", g.tensors["token_embd.weight"].shape[0]))
    cfg = ModelConfig(arch="llama", hidden_size=H, num_hidden_layers=L, layer_types=["full_attention"] * L,
                      num_attention_heads=heads, num_key_value_heads=kv, head_dim=int(k("attention.key_length", H // heads)),
                      attn_output_gate=False, qk_norm="blk.0.attn_q_norm.weight" in g.tensors, norm_zero_centered=False,
                      intermediate_size=int(k("feed_forward_length")), partial_rotary_factor=1.0,
                      rope_theta=float(k("rope.freq_base", 1.0e4)), rms_norm_eps=float(k("attention.layer_norm_rms_epsilon", 1e-6)),
                      vocab_size=vocab, tie_word_embeddings="output.weight" not in g.tensors, mtp_num_hidden_layers=0,
                      max_position_embeddings=int(k("context_length", 8192)))
    if arch.endswith("moe"):
        # attention in every layer, routed experts (stacked per projection in the file) and, for qwen2moe, a shared expert
        # with a sigmoid gate: the engine's MoE family with no linear-attention layers
        cfg.arch = "qwen_hybrid_moe"
        cfg.num_experts = int(k("expert_count"))
        cfg.num_experts_per_tok = int(k("expert_used_count"))
        cfg.moe_intermediate_size = int(k("expert_feed_forward_length", cfg.intermediate_size))
        cfg.shared_expert_intermediate_size = int(k("expert_shared_feed_forward_length", 0)) if "blk.0.ffn_gate_shexp.weight" in g.tensors else 0
        cfg.norm_topk_prob = arch == "qwen3moe"
        cfg.intermediate_size = 0
    cfg.validate()
    return cfg


def _moe_tensors(g: GgufFile, cfg: ModelConfig, i: int, hf: Dict[str, torch.Tensor]) -> None:
    """Layer i's experts: the file stacks them per projection ([experts, out, in]); the importer takes them one by one."""
    p = f"model.layers.{i}.mlp."
    hf[p + "gate.weight"] = g.tensor(f"blk.{i}.ffn_gate_inp.weight")
    stacks = {n: g.tensor(f"blk.{i}.ffn_{n}_exps.weight") for n in ("gate", "up", "down")}
    for n, t in stacks.items():
        if t.dim() != 3 or t.shape[0] != cfg.num_experts:
            raise ValueError(f"blk.{i}.ffn_{n}_exps.weight: shape {tuple(t.shape)} is not [experts, out, in]")
    for e in range(cfg.num_experts):
        for n in ("gate", "up", "down"):
            hf[p + f"experts.{e}.{n}_proj.weight"] = stacks[n][e]
    if cfg.shared_expert_intermediate_size:
        for n in ("gate", "up", "down"):
            hf[p + f"shared_expert.{n}_proj.weight"] = g.tensor(f"blk.{i}.ffn_{n}_shexp.weight")
        hf[p + "shared_expert_gate.weight"] = g.tensor(f"blk.{i}.ffn_gate_inp_shexp.weight").reshape(1, -1)


def import_gguf(path: str) -> Tuple[ModelConfig, Dict[str, torch.Tensor]]:
    """GGUF checkpoint of a dense Llama-style / Qwen-style decoder, or of a Qwen-style MoE decoder (qwen2moe / qwen3moe:
    experts stacked per projection, optional shared expert) -> (config, fp32 weights in this engine's names).
    Tensors are dequantised block by block; the converter then quantizes them into its own layouts."""
    from .hf_import import import_hf_weights
    g = GgufFile(path)
    try:
        cfg = config_from_gguf(g)
        permuted = str(g.metadata.get("general.architecture", "llama")) in ("llama", "mistral")
        hf: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": g.tensor("token_embd.weight"),
                                       "model.norm.weight": g.tensor("output_norm.weight")}
        if "output.weight" in g.tensors:
            hf["lm_head.weight"] = g.tensor("output.weight")
        for i in range(cfg.num_hidden_layers):
            for theirs, mine in _LAYER_NAMES.items():
                name = f"blk.{i}.{theirs}.weight"
                if name not in g.tensors:
                    continue
                t = g.tensor(name)
                if permuted and theirs == "attn_q":
                    t = _unpermute_rope(t, cfg.num_attention_heads)
                elif permuted and theirs == "attn_k":
                    t = _unpermute_rope(t, cfg.num_key_value_heads)
                hf[f"model.layers.{i}.{mine}.weight"] = t
            if cfg.is_moe:
                _moe_tensors(g, cfg, i, hf)
        return cfg, import_hf_weights(cfg, hf)
    finally:
        g.close()
