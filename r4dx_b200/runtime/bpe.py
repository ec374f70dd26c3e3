"""Own tokenizer: byte-level BPE (Qwen / Llama-3 / GPT-2 split patterns) and byte-fallback BPE (SentencePiece-style
vocabularies: "▁" for spaces, <0xNN> byte tokens), read from a ``tokenizer.json``.  Added / special tokens are split out
of the text before the model runs; every token id maps to exact bytes, so a streaming decoder can hold back an incomplete
UTF-8 sequence instead of emitting replacement characters.  No Unicode normalisation is applied.
(reference: src/tokenizer/tokenizer.h:1-80; golden tests against the Hugging Face implementation.)

Encoding a piece: start from its symbols (mapped bytes, or characters), then repeatedly merge the adjacent pair with the
lowest merge rank until none is left - the textbook BPE loop, with a per-piece cache.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import regex

GPT2_PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"


def _bytes_to_unicode() -> Dict[int, str]:
    """The reversible byte -> printable code point table of byte-level BPE vocabularies."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


_B2U = _bytes_to_unicode()
_U2B = {c: b for b, c in _B2U.items()}


class BpeTokenizer:
    def __init__(self, path: str):
        """``path``: a tokenizer.json, or a directory that holds one (generation_config.json beside it names the EOS ids)."""
        directory = path if os.path.isdir(path) else os.path.dirname(path)
        file = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
        spec = json.load(open(file, encoding="utf-8"))
        model = spec["model"]
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"tokenizer model {model.get('type')!r} is not BPE")
        self.vocab: Dict[str, int] = dict(model["vocab"])
        merges = model.get("merges", [])
        self.ranks: Dict[Tuple[str, str], int] = {}
        for i, m in enumerate(merges):
            a, b = m if isinstance(m, (list, tuple)) else m.split(" ", 1)
            self.ranks[(a, b)] = i
        self.byte_fallback = bool(model.get("byte_fallback", False))
        self.ignore_merges = bool(model.get("ignore_merges", False))
        self.unk = model.get("unk_token")
        self.byte_level, self.pattern, self.prefix_space = self._pre_tokenizer(spec.get("pre_tokenizer"))
        if not self.byte_level:
            # SentencePiece-style: the normalizer turns spaces into "▁" (and may prepend one)
            self.prefix_space = self._normalizer_prepends(spec.get("normalizer"))
        self.added: Dict[str, int] = {}
        self.special_ids = set()
        for t in spec.get("added_tokens", []):
            self.added[t["content"]] = t["id"]
            if t.get("special", False):
                self.special_ids.add(t["id"])
        self._added_re = (regex.compile("|".join(regex.escape(c) for c in sorted(self.added, key=len, reverse=True)))
                          if self.added else None)
        self.id_to_token: Dict[int, str] = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.added.items()})
        self.vocab_size = max(self.id_to_token) + 1 if self.id_to_token else 0
        self._cache: Dict[str, List[int]] = {}
        # SentencePiece-style vocabularies whose tokens carry "▁" only as a leading run never merge across the start of
        # such a run, so the text can be cut there and every piece encoded (and cached) on its own - same ids, far less work
        self._sp_split = (not self.byte_level and
                          all(regex.fullmatch(r"▁*[^▁]*", t) is not None for t in self.vocab))
        self._sp_pieces = regex.compile(r"▁*[^▁]+|▁+")
        self._native = None
        self._init_native()
        self.eos_ids: List[int] = []
        gen = os.path.join(directory, "generation_config.json")
        if os.path.exists(gen):
            e = json.load(open(gen)).get("eos_token_id", [])
            self.eos_ids = list(e) if isinstance(e, list) else [e]
        for name in ("<|im_end|>", "<|endoftext|>", "<|eot_id|>", "<end_of_turn>", "<eos>"):
            i = self.added.get(name, self.vocab.get(name))
            if i is not None and i not in self.eos_ids:
                self.eos_ids.append(i)

    # ---- tokenizer.json structure ----------------------------------------------------------------
    @staticmethod
    def _pre_tokenizer(pt) -> Tuple[bool, Optional["regex.Pattern"], bool]:
        """(byte level?, split pattern or None, add a prefix space?)"""
        byte_level, pattern, prefix = False, None, False
        steps = pt.get("pretokenizers", [pt]) if pt else []
        for s in steps:
            if s.get("type") == "Split":
                p = s.get("pattern", {})
                src = p.get("Regex") or regex.escape(p.get("String", ""))
                pattern = regex.compile(src)
            elif s.get("type") == "ByteLevel":
                byte_level = True
                prefix = bool(s.get("add_prefix_space", False))
                if s.get("use_regex", True) and pattern is None:
                    pattern = regex.compile(GPT2_PATTERN)
        return byte_level, pattern, prefix

    @staticmethod
    def _normalizer_prepends(nm) -> bool:
        steps = nm.get("normalizers", [nm]) if nm else []
        return any(s.get("type") == "Prepend" for s in steps)

    # ---- BPE ---------------------------------------------------------------------------------------
    def _init_native(self) -> None:
        """Hands the merge table to the native merge loop as (left id, right id, merged id) triples in rank order.  Needs
        every merge's two sides and product to be vocabulary entries (true of trained BPE vocabularies); otherwise, or when
        the native library is missing, pieces go through the Python loop."""
        if os.environ.get("R4DXB_BPE_NATIVE", "1") == "0":
            return
        try:
            import numpy as np
            from .. import native
            L = native.host()
            tri = np.empty((len(self.ranks), 3), dtype=np.int32)
            for (a, b), i in self.ranks.items():
                ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
                if ia is None or ib is None or im is None:
                    return
                tri[i] = (ia, ib, im)
            self._tri = np.ascontiguousarray(tri)
            self._np = np
            self._lib = L
            self._native = L.r4dxb_bpe_new(self._tri.ctypes.data, len(self.ranks))
        except Exception:
            self._native = None

    def __del__(self):
        try:
            if self._native:
                self._lib.r4dxb_bpe_free(self._native)
        except Exception:
            pass

    def _merge_native(self, ids0: List[int]) -> List[int]:
        np = self._np
        src = np.asarray(ids0, dtype=np.int32)
        out = np.empty(len(ids0), dtype=np.int32)
        n = self._lib.r4dxb_bpe_encode(self._native, src.ctypes.data, len(ids0), out.ctypes.data)
        return out[:n].tolist()

    def _merge(self, symbols: List[str]) -> List[str]:
        ranks = self.ranks
        while len(symbols) > 1:
            best, at = None, -1
            for i in range(len(symbols) - 1):
                r = ranks.get((symbols[i], symbols[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = symbols[at], symbols[at + 1]
            out, i = [], 0
            while i < len(symbols):                  # merge every occurrence of the pair, left to right
                if i + 1 < len(symbols) and symbols[i] == a and symbols[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(symbols[i])
                    i += 1
            symbols = out
        return symbols

    def _piece(self, piece: str) -> List[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        if self.byte_level:
            symbols = [_B2U[b] for b in piece.encode("utf-8")]
        else:
            symbols = list(piece)
        ids: List[int] = []
        whole = "".join(symbols)
        ids0 = [self.vocab.get(s) for s in symbols] if self._native else None
        if self.ignore_merges and whole in self.vocab:       # Llama-3 style: a piece that is a vocabulary entry is taken whole
            ids = [self.vocab[whole]]
        elif ids0 is not None and None not in ids0:
            ids = self._merge_native(ids0)
        else:
            for s in self._merge(symbols):
                i = self.vocab.get(s)
                if i is not None:
                    ids.append(i)
                elif self.byte_fallback:
                    for b in s.encode("utf-8"):
                        j = self.vocab.get(f"<0x{b:02X}>")
                        if j is not None:
                            ids.append(j)
                elif self.unk is not None and self.unk in self.vocab:
                    ids.append(self.vocab[self.unk])
        if len(self._cache) < 1 << 18:
            self._cache[piece] = ids
        return ids

    def _encode_plain(self, text: str, first: bool) -> List[int]:
        if not text:
            return []
        if self.byte_level:
            if self.prefix_space and first and not text.startswith(" "):
                text = " " + text
            pieces = self.pattern.findall(text) if self.pattern is not None else [text]
        else:
            if self.prefix_space and first:
                text = " " + text
            text = text.replace(" ", "▁")
            pieces = self._sp_pieces.findall(text) if self._sp_split else [text]
        out: List[int] = []
        for p in pieces:
            out += self._piece(p)
        return out

    def encode(self, text: str) -> List[int]:
        if self._added_re is None:
            return self._encode_plain(text, True)
        out: List[int] = []
        at, first = 0, True
        for m in self._added_re.finditer(text):
            out += self._encode_plain(text[at:m.start()], first)
            out.append(self.added[m.group(0)])
            at, first = m.end(), False
        return out + self._encode_plain(text[at:], first)

    # ---- decoding ----------------------------------------------------------------------------------
    def token_bytes(self, tid: int, skip_special: bool = True) -> bytes:
        tok = self.id_to_token.get(int(tid))
        if tok is None or (skip_special and tid in self.special_ids):
            return b""
        if self.byte_fallback and len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            try:
                return bytes([int(tok[3:5], 16)])
            except ValueError:
                pass
        if tok in self.added and self.added[tok] == tid:
            return tok.encode("utf-8")
        if self.byte_level:
            return bytes(_U2B[c] for c in tok if c in _U2B)
        return tok.replace("▁", " ").encode("utf-8")

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        text = b"".join(self.token_bytes(i, skip_special) for i in ids).decode("utf-8", errors="replace")
        if not self.byte_level and self.prefix_space and text.startswith(" "):
            text = text[1:]
        return text
