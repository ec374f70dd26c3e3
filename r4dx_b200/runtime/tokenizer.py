"""Tokenizer glue: Hugging Face ``tokenizers`` + a Jinja chat template when a tokenizer directory is
given, a byte-level fallback otherwise (tests, synthetic models).  Streaming decode never emits half
of a multi-byte character (reference: src/tokenizer/tokenizer.h:1-80, chat_template.h:1-50).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

DEFAULT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% if enable_thinking is defined and not enable_thinking %}"
    "<think>\n\n</think>\n\n{% endif %}{% endif %}")


class ByteTokenizer:
    """256 byte tokens + a few specials; ids are offset so that 0 is EOS."""

    SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>"]

    def __init__(self, vocab_size: int = 4096):
        self.vocab_size = vocab_size
        self.special_ids = {s: i for i, s in enumerate(self.SPECIALS)}
        self.offset = len(self.SPECIALS)
        self.eos_ids = [self.special_ids["<|endoftext|>"], self.special_ids["<|im_end|>"]]

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                out += [b + self.offset for b in text[i].encode("utf-8")]
                i += 1
        return out

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return StreamDecoder(self, skip_special).feed_all(ids)

    def token_bytes(self, tid: int, skip_special: bool = True) -> bytes:
        if tid < self.offset:
            return b"" if skip_special else self.SPECIALS[tid].encode()
        b = tid - self.offset
        return bytes([b]) if b < 256 else b"?"


class HfTokenizer:
    def __init__(self, directory: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(os.path.join(directory, "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size()
        self.eos_ids: List[int] = []
        gen = os.path.join(directory, "generation_config.json")
        if os.path.exists(gen):
            e = json.load(open(gen)).get("eos_token_id", [])
            self.eos_ids = e if isinstance(e, list) else [e]
        for name in ("<|im_end|>", "<|endoftext|>"):
            i = self.tk.token_to_id(name)
            if i is not None and i not in self.eos_ids:
                self.eos_ids.append(i)

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special)

    def token_bytes(self, tid: int, skip_special: bool = True) -> bytes:
        return self.tk.decode([tid], skip_special_tokens=skip_special).encode("utf-8", "surrogatepass")


class StreamDecoder:
    """Incremental detokenizer: holds back bytes until they form complete UTF-8 characters."""

    def __init__(self, tokenizer, skip_special: bool = True):
        self.tk = tokenizer
        self.skip = skip_special
        self.pending = b""
        self.ids: List[int] = []
        self.emitted = ""

    def feed(self, tid: int) -> str:
        if isinstance(self.tk, HfTokenizer):
            # byte-level BPE pieces are not independently decodable: re-decode the tail window
            self.ids.append(tid)
            text = self.tk.decode(self.ids, self.skip)
            if text.endswith("�"):
                return ""
            new = text[len(self.emitted):]
            self.emitted = text
            return new
        self.pending += self.tk.token_bytes(tid, self.skip)
        try:
            s = self.pending.decode("utf-8")
            self.pending = b""
            return s
        except UnicodeDecodeError as e:
            if e.start > 0:
                s = self.pending[:e.start].decode("utf-8")
                self.pending = self.pending[e.start:]
                return s
            if len(self.pending) > 4:
                s = self.pending.decode("utf-8", "replace")
                self.pending = b""
                return s
            return ""

    def feed_all(self, ids: Sequence[int]) -> str:
        return "".join(self.feed(i) for i in ids) + self.flush()

    def flush(self) -> str:
        s = self.pending.decode("utf-8", "replace") if self.pending else ""
        self.pending = b""
        return s


class ChatTemplate:
    def __init__(self, source: Optional[str] = None):
        import jinja2
        env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False)
        env.globals["raise_exception"] = self._raise
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False)
        self.template = env.from_string(source or DEFAULT_TEMPLATE)

    @staticmethod
    def _raise(msg):
        raise ValueError(msg)

    def render(self, messages: List[Dict], add_generation_prompt: bool = True, tools: Optional[list] = None,
               enable_thinking: Optional[bool] = None) -> str:
        kw = dict(messages=messages, add_generation_prompt=add_generation_prompt, tools=tools)
        if enable_thinking is not None:
            kw["enable_thinking"] = enable_thinking
        return self.template.render(**kw)


def load_tokenizer(directory: Optional[str], vocab_size: int = 4096):
    if directory and os.path.exists(os.path.join(directory, "tokenizer.json")):
        # the engine's own BPE reads byte-level and byte-fallback BPE vocabularies; anything else (Unigram, WordPiece,
        # normalisers it does not model) falls back to the `tokenizers` library
        try:
            if os.environ.get("R4DXB_TOKENIZER", "own") != "own":
                raise ValueError("library tokenizer requested")
            from .bpe import BpeTokenizer
            tk = BpeTokenizer(directory)
        except (ValueError, KeyError):
            tk = HfTokenizer(directory)
        tpl_path = os.path.join(directory, "chat_template.jinja")
        tpl = ChatTemplate(open(tpl_path).read() if os.path.exists(tpl_path) else None)
        return tk, tpl
    return ByteTokenizer(vocab_size), ChatTemplate(None)
