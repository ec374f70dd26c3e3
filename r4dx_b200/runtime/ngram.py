"""Hashed n-gram embedding table: file format, row ids, and the three placements of the table.

Every token owns ``heads`` rows of the table (half of them hash the 2-gram, half the 3-gram ending in the token), each head
modulo its own prime plus its own row offset; the rows, concatenated, are the input of the n-gram embedding layer.  The
table of the full model is 320,001,536 rows x 160 bf16 = 95.4 GiB.

File ("sidecar"): a 4096-byte little-endian header, then ``rows`` rows of ``row_bytes`` bytes in row-id order

    0  char[8] "R4DXNGRM" | 8 u32 version | 12 u64 rows | 20 u32 row_bytes | 24 u32 heads | 28 u32 head_dim
    32 u32 ngram_size | 36 u32 heads_per_ngram | 40 i64 eos | 48 u64 seed | 56 i64[3] multipliers
    80 u64[16] head offsets | 208 u64[16] head primes | 336 u64 padded_rows | 344 u8[32] sha256 of the body | zeros

(reference: src/model/qwen4exp/include/r4dx/model/qwen4exp/ngram_sidecar.h:8-35; ids: ngram_ids.h:8-20).

Placement (``NgramTable.open(mode=...)``): the reference reads 16 rows per token from NVMe on the decode critical path
because two 32 GB cards cannot hold the table.  One B200 can (95 GiB of 180 GB next to ~51 GiB of weights), so the default
here is ``"device"``: the body is loaded once, and one kernel computes the ids from the token history and gathers the rows,
with no host work per token (``ops.kernels.q4x_ngram_gather``).  ``"pinned"`` keeps the body in page-locked host memory and
``"file"`` reads rows with positioned reads (host ids, one host-to-device copy of the gathered rows per call) for machines
where the table does not fit next to the weights.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch

from .. import native

MAGIC = b"R4DXNGRM"
HEADER_BYTES = 4096
VERSION = 1
NGRAM_SIZE = 3
_I64_MAX = (1 << 63) - 1

native.register_host_sig("r4dxb_ngram_ids", ctypes.c_int,
                         [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                          ctypes.c_int, ctypes.c_int64, ctypes.c_void_p])
native.register_host_sig("r4dxb_ngram_read_rows", ctypes.c_int64,
                         [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
                          ctypes.c_void_p, ctypes.c_int])


native.register_host_sig("r4dxb_ngram_read_rows_direct", ctypes.c_int64,
                         [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                          ctypes.c_void_p, ctypes.c_int])


class NgramError(RuntimeError):
    pass


@dataclass
class NgramHeader:
    rows: int
    head_dim: int
    eos_token_id: int
    seed: int
    multipliers: List[int]
    head_offsets: List[int]
    head_primes: List[int]
    padded_rows: int
    heads: int = 16
    heads_per_ngram: int = 8
    body_sha256: bytes = b"\0" * 32
    version: int = VERSION

    @property
    def row_bytes(self) -> int:
        return self.head_dim * 2

    @property
    def body_bytes(self) -> int:
        return self.rows * self.row_bytes

    def pack(self) -> bytes:
        if len(self.head_offsets) != 16 or len(self.head_primes) != 16 or len(self.multipliers) != 3:
            raise NgramError("header tables: 16 offsets, 16 primes, 3 multipliers")
        b = MAGIC + struct.pack("<IQIIIIIqQ", self.version, self.rows, self.row_bytes, self.heads, self.head_dim, NGRAM_SIZE,
                                self.heads_per_ngram, self.eos_token_id, self.seed)
        b += struct.pack("<3q", *self.multipliers) + struct.pack("<16Q", *self.head_offsets) + struct.pack("<16Q", *self.head_primes)
        b += struct.pack("<Q", self.padded_rows) + self.body_sha256
        assert len(b) == 376
        return b + b"\0" * (HEADER_BYTES - len(b))

    @staticmethod
    def parse(buf: bytes) -> "NgramHeader":
        if len(buf) < HEADER_BYTES:
            raise NgramError("n-gram table: file shorter than its header")
        if buf[:8] != MAGIC:
            raise NgramError("n-gram table: bad magic")
        version, rows, row_bytes, heads, head_dim, ngram, per, eos, seed = struct.unpack_from("<IQIIIIIqQ", buf, 8)
        mult = list(struct.unpack_from("<3q", buf, 56))
        offs = list(struct.unpack_from("<16Q", buf, 80))
        primes = list(struct.unpack_from("<16Q", buf, 208))
        (padded,) = struct.unpack_from("<Q", buf, 336)
        sha = bytes(buf[344:376])
        if version != VERSION:
            raise NgramError(f"n-gram table: version {version}")
        if heads != 16 or per != 8 or ngram != NGRAM_SIZE:
            raise NgramError(f"n-gram table: {heads} heads, {per} per order, {ngram}-grams (built for 16 / 8 / 3)")
        if row_bytes != head_dim * 2 or head_dim < 1:
            raise NgramError("n-gram table: row_bytes != 2 * head_dim")
        if any(m <= 0 for m in mult) or any(p == 0 for p in primes):
            raise NgramError("n-gram table: non-positive multiplier or prime")
        if any(o + p > padded for o, p in zip(offs, primes)) or rows > padded and padded:
            raise NgramError("n-gram table: a head's rows reach beyond padded_rows")
        if any(buf[376:HEADER_BYTES]):
            raise NgramError("n-gram table: header padding is not zero")
        max_token = min(_I64_MAX // m for m in mult)
        if not 0 <= eos <= max_token:
            raise NgramError("n-gram table: eos id would overflow the hash")
        return NgramHeader(rows=rows, head_dim=head_dim, eos_token_id=eos, seed=seed, multipliers=mult, head_offsets=offs,
                           head_primes=primes, padded_rows=padded, heads=heads, heads_per_ngram=per, body_sha256=sha,
                           version=version)

    @property
    def max_token_id(self) -> int:
        return min(_I64_MAX // m for m in self.multipliers)


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def _primes_after(start: int, count: int) -> List[int]:
    def is_prime(n: int) -> bool:
        if n < 2:
            return False
        i = 2
        while i * i <= n:
            if n % i == 0:
                return False
            i += 1
        return True
    out, n = [], start
    while len(out) < count:
        n += 1
        if is_prime(n):
            out.append(n)
    return out


def make_header(vocab_size: int, head_dim: int, eos_token_id: int, seed: int = 0, first_prime_after: int = 1000) -> NgramHeader:
    """Header of a new table: 16 consecutive primes after ``first_prime_after`` as the per-head vocabularies, offsets that
    concatenate them, multipliers below int64 max / vocab so that no product of the hash overflows."""
    primes = _primes_after(first_prime_after, 16)
    offs, at = [], 0
    for p in primes:
        offs.append(at)
        at += p
    bound = _I64_MAX // max(2, vocab_size)
    mult, x = [], seed
    for _ in range(3):
        x = _splitmix64(x)
        mult.append(x % (bound - 1) + 1)
    return NgramHeader(rows=at, head_dim=head_dim, eos_token_id=eos_token_id, seed=seed, multipliers=mult, head_offsets=offs,
                       head_primes=primes, padded_rows=at)


def write_sidecar(path: str, header: NgramHeader, blocks: Iterable[torch.Tensor]) -> NgramHeader:
    """Streams the rows (bf16 tensors [n, head_dim], in row-id order) into ``path`` and records the body's sha256."""
    sha = hashlib.sha256()
    n = 0
    with open(path, "wb") as f:
        f.write(b"\0" * HEADER_BYTES)
        for blk in blocks:
            if blk.dtype != torch.bfloat16 or blk.dim() != 2 or blk.shape[1] != header.head_dim:
                raise NgramError("rows must be bf16 [n, head_dim]")
            raw = blk.contiguous().view(torch.uint8).numpy().tobytes()
            sha.update(raw)
            f.write(raw)
            n += blk.shape[0]
        if n != header.rows:
            raise NgramError(f"wrote {n} rows, header says {header.rows}")
        header.body_sha256 = sha.digest()
        f.seek(0)
        f.write(header.pack())
    return header


def synthetic_sidecar(path: str, vocab_size: int, head_dim: int, eos_token_id: int, seed: int = 0, std: float = 0.02,
                      first_prime_after: int = 1000) -> NgramHeader:
    h = make_header(vocab_size, head_dim, eos_token_id, seed, first_prime_after)
    g = torch.Generator().manual_seed(seed + 17)

    def blocks():
        left = h.rows
        while left:
            n = min(left, 1 << 16)
            yield (torch.randn(n, head_dim, generator=g) * std).to(torch.bfloat16)
            left -= n
    return write_sidecar(path, h, blocks())


class NgramIds:
    """Row ids on the host; carries the last two tokens across calls, so any chunking of a sequence gives the same ids."""

    def __init__(self, header: NgramHeader):
        self.h = header
        self._mult = np.asarray(header.multipliers, dtype=np.int64)
        self._primes = np.asarray(header.head_primes, dtype=np.uint64)
        self._offs = np.asarray(header.head_offsets, dtype=np.uint64)
        self.reset()

    def reset(self) -> None:
        self.history = np.asarray([self.h.eos_token_id] * 2, dtype=np.int64)

    def snapshot(self):
        return self.history.copy()

    def restore(self, snap) -> None:
        snap = np.asarray(snap, dtype=np.int64)
        if snap.shape != (2,) or (snap < 0).any() or (snap > self.h.max_token_id).any():
            raise NgramError("n-gram history snapshot out of range")
        self.history = snap.copy()

    def generate(self, tokens: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        out = np.empty((t.shape[0], self.h.heads), dtype=np.int64)
        hist = self.history.copy()
        rc = native.host().r4dxb_ngram_ids(t.ctypes.data, t.shape[0], hist.ctypes.data, self._mult.ctypes.data,
                                           self._primes.ctypes.data, self._offs.ctypes.data, self.h.heads,
                                           self.h.eos_token_id, out.ctypes.data)
        if rc:
            raise NgramError("n-gram ids: a token id is negative or too large for the overflow-free hash")
        self.history = hist
        return out


def ngram_ids_reference(tokens: Sequence[int], header: NgramHeader, history: Optional[Sequence[int]] = None) -> List[List[int]]:
    """The same ids in plain Python integers (the test oracle of the native and device versions)."""
    eos = header.eos_token_id
    a, b = (history if history is not None else (eos, eos))
    m0, m1, m2 = header.multipliers
    mask = (1 << 64) - 1
    out = []
    for t in tokens:
        s1 = b
        s2 = eos if (a == eos or b == eos) else a
        bi = ((t * m0) & mask) ^ ((s1 * m1) & mask)
        tri = bi ^ ((s2 * m2) & mask)
        half = header.heads // 2
        out.append([(bi if h < half else tri) % header.head_primes[h] + header.head_offsets[h] for h in range(header.heads)])
        a, b = b, t
    return out


class NgramTable:
    """The opened table.  ``gather(tokens)`` returns the rows of the tokens, [n, heads * head_dim] bf16 on ``device``, and
    advances the history; ``device`` mode does both in one kernel on the current stream."""

    def __init__(self, path: str, header: NgramHeader, mode: str, device, fd: int, body: Optional[torch.Tensor], threads: int,
                 direct_fd: int = -1):
        self.path, self.header, self.mode, self.device, self._fd, self.body, self.threads = path, header, mode, device, fd, body, threads
        self._direct_fd = direct_fd          # >= 0: row reads bypass the page cache (O_DIRECT)
        self.ids = NgramIds(header)

    @staticmethod
    def open(path: str, mode: str = "device", device="cuda", threads: int = 8, allow_truncated: bool = False,
             direct: bool = False) -> "NgramTable":
        """``direct`` (file placement): row reads use O_DIRECT, so the 95 GiB table neither fills nor evicts the page cache
        (reference: docs/qwen4exp.md "Requirements": the sidecar is read with unbuffered I/O, never through the file cache)."""
        if mode not in ("device", "pinned", "file"):
            raise NgramError(f"n-gram table placement {mode!r}: device | pinned | file")
        fd = os.open(path, os.O_RDONLY)
        direct_fd = -1
        if direct and mode == "file":
            try:
                direct_fd = os.open(path, os.O_RDONLY | os.O_DIRECT)
            except OSError as e:
                os.close(fd)
                raise NgramError(f"n-gram table {path}: this file system refuses O_DIRECT ({e.strerror})")
        try:
            head = NgramHeader.parse(os.pread(fd, HEADER_BYTES, 0))
            size = os.fstat(fd).st_size
            if size != HEADER_BYTES + head.body_bytes and not (allow_truncated and size < HEADER_BYTES + head.body_bytes):
                raise NgramError(f"n-gram table: {size} bytes on disk, header says {HEADER_BYTES + head.body_bytes}")
            body = None
            if mode != "file":
                host = torch.empty(head.rows, head.head_dim, dtype=torch.bfloat16, pin_memory=(mode == "pinned" and torch.cuda.is_available()))
                buf = host.view(torch.uint8).numpy().reshape(-1)
                at = 0
                while at < head.body_bytes:               # 64 MiB reads: the body may be far larger than any one read should be
                    chunk = os.pread(fd, min(1 << 26, head.body_bytes - at), HEADER_BYTES + at)
                    if not chunk:
                        raise NgramError("n-gram table: short read of the body")
                    buf[at:at + len(chunk)] = np.frombuffer(chunk, dtype=np.uint8)
                    at += len(chunk)
                body = host.to(device) if mode == "device" else host
        except Exception:
            os.close(fd)
            if direct_fd >= 0:
                os.close(direct_fd)
            raise
        return NgramTable(path, head, mode, torch.device(device), fd, body, threads, direct_fd)

    @staticmethod
    def synthetic_device(header: NgramHeader, device="cuda", std: float = 0.02, seed: int = 0) -> "NgramTable":
        """A table of random rows created directly in device memory (benchmarks: no file behind it)."""
        g = torch.Generator(device=device).manual_seed(seed)
        body = torch.empty(header.rows, header.head_dim, dtype=torch.bfloat16, device=device)
        step = 1 << 22
        for at in range(0, header.rows, step):
            n = min(step, header.rows - at)
            body[at:at + n] = (torch.randn(n, header.head_dim, generator=g, device=device) * std).to(torch.bfloat16)
        return NgramTable("", header, "device", torch.device(device), -1, body, 1)

    def close(self) -> None:
        if self._fd >= 0:
            os.close(self._fd)
            self._fd = -1
        if self._direct_fd >= 0:
            os.close(self._direct_fd)
            self._direct_fd = -1

    def verify_sha256(self) -> bool:
        sha, at = hashlib.sha256(), 0
        while at < self.header.body_bytes:
            chunk = os.pread(self._fd, min(1 << 24, self.header.body_bytes - at), HEADER_BYTES + at)
            if not chunk:
                return False
            sha.update(chunk)
            at += len(chunk)
        return sha.digest() == self.header.body_sha256

    def rows(self, ids: np.ndarray) -> torch.Tensor:
        """Rows ``ids`` (int64, any shape) as a host bf16 tensor [..., head_dim]; a row that cannot be read in full raises."""
        flat = np.ascontiguousarray(ids.reshape(-1), dtype=np.int64)
        h = self.header
        if self.body is not None and self.mode == "pinned":
            if (flat < 0).any() or (flat >= h.rows).any():
                raise NgramError("n-gram row id out of range")
            return self.body[torch.from_numpy(flat)].view(*ids.shape, h.head_dim)
        out = torch.empty(flat.shape[0], h.head_dim, dtype=torch.bfloat16)
        rc = -1
        if self._direct_fd >= 0:
            rc = native.host().r4dxb_ngram_read_rows_direct(self._direct_fd, flat.ctypes.data, flat.shape[0], h.rows, h.row_bytes,
                                                            HEADER_BYTES, os.fstat(self._fd).st_size, out.data_ptr(), self.threads)
        if rc != 0:
            # no direct descriptor, or a direct read failed (some file systems accept the flag and then refuse the reads): the
            # buffered descriptor decides; a row it cannot deliver either is an error, never a zero row
            rc = native.host().r4dxb_ngram_read_rows(self._fd, flat.ctypes.data, flat.shape[0], h.rows, h.row_bytes, HEADER_BYTES,
                                                     out.data_ptr(), self.threads)
        if rc:
            raise NgramError(f"n-gram table: row {int(flat[rc - 1])} could not be read in full")
        return out.view(*ids.shape, h.head_dim)

    def gather_host(self, tokens: Sequence[int]) -> torch.Tensor:
        """Host ids + host rows: [n, heads * head_dim] bf16 on the host (``pinned`` and ``file`` placements, tools)."""
        ids = self.ids.generate(tokens)
        return self.rows(ids).reshape(len(tokens), self.header.heads * self.header.head_dim)


# ---- the table file from a checkpoint's own shards ---------------------------------------------------------------------
def repack_from_checkpoint(model_dir: str, out: str, log=None) -> NgramHeader:
    """Streams the n-gram table of a qwen4_exp checkpoint directory into one table file.

    The checkpoint stores the table as ``split_ngram_parts`` bf16 tensors
    ``model.language_model.layers.{L}.ple.ple_embedding.ngram_embedding.shard_{i}.weight`` ([rows_i, head_dim]) spread over its
    safetensors files and concatenated in shard order, next to three int64 buffers with the hash parameters
    (``layer_multipliers``, ``ngram_heads_vocab_sizes``, ``ngram_heads_offsets``); L is the single entry of ``ple_layer_ids``
    minus one.  One shard is in memory at a time.
    (reference: tools/reference/qwen4exp/ngram_sidecar.py:1-40, 126-205 describes the same source layout.)"""
    import json
    from safetensors import safe_open
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    tc = cfg.get("text_config", cfg)
    ple = tc.get("ple_layer_ids") or []
    if len(ple) != 1:
        raise NgramError(f"exactly one n-gram layer is supported, config has ple_layer_ids={ple}")
    parts = int(tc.get("split_ngram_parts", 512))
    prefix = f"model.language_model.layers.{int(ple[0]) - 1}.ple.ple_embedding."
    index = json.load(open(os.path.join(model_dir, "model.safetensors.index.json")))["weight_map"]
    want = [f"{prefix}ngram_embedding.shard_{i}.weight" for i in range(parts)]
    have = {k for k in index if k.startswith(prefix + "ngram_embedding.shard_")}
    if have != set(want):
        raise NgramError(f"the index lists {len(have)} n-gram shard tensors, expected shard_0..shard_{parts - 1}")

    def tensor(name: str) -> torch.Tensor:
        if name not in index:
            raise NgramError(f"{name} is not in model.safetensors.index.json")
        with safe_open(os.path.join(model_dir, index[name]), "pt") as sf:
            return sf.get_tensor(name)

    mult = [int(v) for v in tensor(prefix + "layer_multipliers").reshape(-1).tolist()]
    primes = [int(v) for v in tensor(prefix + "ngram_heads_vocab_sizes").reshape(-1).tolist()]
    offs = [int(v) for v in tensor(prefix + "ngram_heads_offsets").reshape(-1).tolist()]
    if len(mult) != NGRAM_SIZE or len(primes) != 16 or len(offs) != 16:
        raise NgramError("the checkpoint's hash buffers are not 3 multipliers, 16 vocabulary sizes and 16 offsets")
    first = tensor(want[0])
    if first.dtype != torch.bfloat16 or first.dim() != 2:
        raise NgramError(f"{want[0]}: {first.dtype} {tuple(first.shape)}, expected bf16 [rows, head_dim]")
    head_dim = first.shape[1]
    eos = int(tc.get("eos_token_id", cfg.get("eos_token_id", 248044)) or 248044)
    rows = 0
    shapes = []
    for name in want:                                   # a first pass over the headers only: the row count goes into the header
        with safe_open(os.path.join(model_dir, index[name]), "pt") as sf:
            shp = sf.get_slice(name).get_shape()
        if len(shp) != 2 or shp[1] != head_dim:
            raise NgramError(f"{name}: shape {shp}, expected [rows, {head_dim}]")
        shapes.append(shp[0])
        rows += shp[0]
    padded = max(o + p for o, p in zip(offs, primes))
    if rows < padded:
        raise NgramError(f"the shards hold {rows} rows, the head offsets reach {padded}")
    header = NgramHeader(rows=rows, head_dim=head_dim, eos_token_id=eos, seed=int(tc.get("ngram_seed", 0)), multipliers=mult,
                         head_offsets=offs, head_primes=primes, padded_rows=rows)

    def blocks():
        for i, name in enumerate(want):
            t = first if i == 0 else tensor(name)
            if log is not None:
                log(f"shard {i + 1}/{parts}: {t.shape[0]} rows")
            yield t
    return write_sidecar(out, header, blocks())


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser("r4dx_b200.runtime.ngram", description="n-gram table file: repack from a checkpoint, verify")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("repack", help="checkpoint directory -> table file")
    r.add_argument("--model-dir", required=True)
    r.add_argument("--out", required=True)
    v = sub.add_parser("verify", help="check the header, the size and the body's sha256")
    v.add_argument("--sidecar", required=True)
    a = ap.parse_args(argv)
    if a.cmd == "repack":
        h = repack_from_checkpoint(a.model_dir, a.out, log=print)
        print(f"wrote {a.out}: {h.rows} rows x {h.head_dim}, sha256 {h.body_sha256.hex()}")
        return 0
    t = NgramTable.open(a.sidecar, mode="file")
    ok = t.verify_sha256()
    print(f"{a.sidecar}: {t.header.rows} rows x {t.header.head_dim}, body sha256 {'matches' if ok else 'DOES NOT match'} the header")
    t.close()
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
