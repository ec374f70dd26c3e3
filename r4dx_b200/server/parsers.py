"""Stream post-processing: reasoning split (<think>...</think>) and tool-call extraction.

Both are incremental: they take text deltas and hold back only what might still turn out to be a tag
(reference: src/server/reasoning_splitter.*, *tool_call_parser.*, tool_stream_gate).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Dict, List, Optional, Tuple


class ReasoningSplitter:
    """Routes text inside <think>...</think> to ``reasoning`` and the rest to ``content``."""

    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, start_in_think: bool = False, open_tag: Optional[str] = None, close_tag: Optional[str] = None):
        self.in_think = start_in_think
        self.buf = ""
        if open_tag:
            self.OPEN = open_tag
        if close_tag:
            self.CLOSE = close_tag

    def feed(self, delta: str) -> Tuple[str, str]:
        """Returns (content_delta, reasoning_delta)."""
        self.buf += delta
        content, reasoning = "", ""
        while self.buf:
            tag = self.CLOSE if self.in_think else self.OPEN
            i = self.buf.find(tag)
            if i >= 0:
                piece, self.buf = self.buf[:i], self.buf[i + len(tag):]
                if self.in_think:
                    reasoning += piece
                else:
                    content += piece
                self.in_think = not self.in_think
                if not self.in_think:
                    self.buf = self.buf.lstrip("\n")
                continue
            # keep a possible partial tag at the end
            hold = 0
            for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-k:]):
                    hold = k
                    break
            piece = self.buf[:len(self.buf) - hold]
            self.buf = self.buf[len(self.buf) - hold:]
            if self.in_think:
                reasoning += piece
            else:
                content += piece
            break
        return content, reasoning

    def flush(self) -> Tuple[str, str]:
        piece, self.buf = self.buf, ""
        return ("", piece) if self.in_think else (piece, "")


class QwenToolCallParser:
    """Extracts <tool_call>{"name": ..., "arguments": {...}}</tool_call> blocks (also the XML-ish
    <function=name><parameter=key>value</parameter></function> form) from the content stream."""

    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self):
        self.buf = ""
        self.in_call = False
        self.calls: List[Dict] = []

    def feed(self, delta: str) -> str:
        """Returns the content delta with tool-call blocks removed; finished calls land in ``calls``."""
        self.buf += delta
        out = ""
        while self.buf:
            tag = self.CLOSE if self.in_call else self.OPEN
            i = self.buf.find(tag)
            if i >= 0:
                piece, self.buf = self.buf[:i], self.buf[i + len(tag):]
                if self.in_call:
                    self._finish(piece)
                else:
                    out += piece
                self.in_call = not self.in_call
                continue
            if self.in_call:
                break                      # wait for the closing tag
            hold = 0
            for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-k:]):
                    hold = k
                    break
            out += self.buf[:len(self.buf) - hold]
            self.buf = self.buf[len(self.buf) - hold:]
            break
        return out

    def _finish(self, body: str) -> None:
        body = body.strip()
        name, args = None, None
        try:
            obj = json.loads(body)
            name, args = obj.get("name"), obj.get("arguments", {})
        except Exception:
            m = re.search(r"<function=([^>]+)>(.*?)</function>", body, re.S)
            if m:
                name = m.group(1).strip()
                args = {k.strip(): v.strip() for k, v in re.findall(r"<parameter=([^>]+)>(.*?)</parameter>", m.group(2), re.S)}
        if name is None:
            return
        self.calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                           "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}})

    def flush(self) -> str:
        piece, self.buf = self.buf, ""
        if self.in_call:
            return ""
        return piece


class _Incomplete(Exception):
    """The span ran out of text before it was closed: wait for more."""


class _Malformed(Exception):
    """The span cannot be a tool call: it degrades to literal content."""


class _Cursor:
    def __init__(self, s: str, at: int = 0):
        self.s, self.p = s, at

    def ws(self) -> None:
        while self.p < len(self.s) and self.s[self.p].isspace():
            self.p += 1

    def peek(self) -> str:
        if self.p >= len(self.s):
            raise _Incomplete()
        return self.s[self.p]

    def startswith(self, t: str) -> bool:
        """True if ``t`` is next; raises _Incomplete if the text ends inside a possible ``t``."""
        rest = self.s[self.p:self.p + len(t)]
        if rest == t:
            return True
        if len(rest) < len(t) and t.startswith(rest):
            raise _Incomplete()
        return False

    def expect(self, t: str) -> None:
        if not self.startswith(t):
            raise _Malformed()
        self.p += len(t)

    def word(self, stop: str) -> str:
        a = self.p
        while self.p < len(self.s) and self.s[self.p] not in stop and not self.s[self.p].isspace():
            self.p += 1
        if self.p >= len(self.s):
            raise _Incomplete()
        return self.s[a:self.p]


def _bare(word: str):
    low = {"true": True, "false": False, "null": None, "True": True, "False": False, "None": None}
    if word in low:
        return low[word], True
    try:
        return (int(word) if re.fullmatch(r"[-+]?\d+", word) else float(word)), True
    except ValueError:
        return word, False


class SpanToolCallParser:
    """Streaming extraction of tool calls written between an opening and a closing marker.  The span is parsed by
    recursive descent from the opening marker (not by searching for the closing marker), so a string argument that contains
    the closing marker does not end the call early.  A span that cannot be a call is passed through as literal content,
    markers included, and ``had_malformed_call`` is set (reference: src/server/gemma_tool_call_parser.cpp:1-16,
    src/server/lfm2_tool_call_parser.cpp:1-25)."""

    OPEN = ""
    CLOSE = ""
    MAX_DEPTH = 64

    def __init__(self):
        self.buf = ""
        self.calls: List[Dict] = []
        self.had_malformed_call = False

    def parse_span(self, c: _Cursor) -> List[Tuple[str, Dict]]:
        raise NotImplementedError

    def feed(self, delta: str) -> str:
        self.buf += delta
        out = ""
        while self.buf:
            i = self.buf.find(self.OPEN)
            if i < 0:
                hold = 0
                for k in range(min(len(self.OPEN) - 1, len(self.buf)), 0, -1):
                    if self.OPEN.startswith(self.buf[-k:]):
                        hold = k
                        break
                out += self.buf[:len(self.buf) - hold]
                self.buf = self.buf[len(self.buf) - hold:]
                break
            out += self.buf[:i]
            self.buf = self.buf[i:]
            c = _Cursor(self.buf, len(self.OPEN))
            try:
                found = self.parse_span(c)
                c.ws()
                c.expect(self.CLOSE)
            except _Incomplete:
                break                                   # wait for the rest of the span
            except (_Malformed, RecursionError):
                self.had_malformed_call = True
                out += self.OPEN                        # literal content; what follows is scanned again
                self.buf = self.buf[len(self.OPEN):]
                continue
            for name, args in found:
                self.calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                                   "function": {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}})
            self.buf = self.buf[c.p:]
        return out

    def flush(self) -> str:
        piece, self.buf = self.buf, ""
        if piece.startswith(self.OPEN) and self.OPEN:
            self.had_malformed_call = True              # a generation cut off inside a call
        return piece


class GemmaToolCallParser(SpanToolCallParser):
    """``<|tool_call>call:NAME{key:value,key2:<|"|>text<|"|>,obj:{a:1},list:[1,<|"|>x<|"|>]}<tool_call|>``: bare keys
    (a key wrapped in the string delimiter is accepted too), strings between ``<|"|>`` markers with raw text inside, bare
    numbers / true / false / null, any other bare word kept as a string."""

    OPEN, CLOSE, ESC = "<|tool_call>", "<tool_call|>", '<|"|>'

    def parse_span(self, c: _Cursor):
        c.ws()
        c.expect("call:")
        name = c.word("{")
        if not name:
            raise _Malformed()
        c.ws()
        return [(name, self._object(c, 0))]

    def _string(self, c: _Cursor) -> str:
        c.expect(self.ESC)
        j = c.s.find(self.ESC, c.p)
        if j < 0:
            raise _Incomplete()
        text, c.p = c.s[c.p:j], j + len(self.ESC)
        return text

    def _value(self, c: _Cursor, depth: int):
        if depth > self.MAX_DEPTH:
            raise _Malformed()
        c.ws()
        if c.startswith(self.ESC):
            return self._string(c)
        ch = c.peek()
        if ch == "{":
            return self._object(c, depth + 1)
        if ch == "[":
            c.p += 1
            items = []
            while True:
                c.ws()
                if c.peek() == "]":
                    c.p += 1
                    return items
                items.append(self._value(c, depth + 1))
                c.ws()
                if c.peek() == ",":
                    c.p += 1
        word = c.word(",}]")
        if not word:
            raise _Malformed()
        return _bare(word)[0]

    def _object(self, c: _Cursor, depth: int) -> Dict:
        if depth > self.MAX_DEPTH:
            raise _Malformed()
        c.expect("{")
        obj: Dict = {}
        while True:
            c.ws()
            if c.peek() == "}":
                c.p += 1
                return obj
            key = self._string(c) if c.startswith(self.ESC) else c.word(":")
            if not key:
                raise _Malformed()
            c.ws()
            c.expect(":")
            obj[key] = self._value(c, depth)
            c.ws()
            if c.peek() == ",":
                c.p += 1
            elif c.peek() != "}":
                raise _Malformed()


class Lfm2ToolCallParser(SpanToolCallParser):
    """``<|tool_call_start|>[name(arg='text', n=3, flag=True, nested=[1, "two", null, {"k": "v"}]), other()]<|tool_call_end|>``:
    a Python list of keyword-only calls whose values are Python or JSON literals.  Positional arguments, other bare words,
    an empty list and unbalanced brackets make the whole span malformed; whitespace, trailing commas and call or argument
    names that are not Python identifiers (``mcp__srv__tool-1``) are accepted."""

    OPEN, CLOSE = "<|tool_call_start|>", "<|tool_call_end|>"
    _ESC = {"n": "\n", "r": "\r", "t": "\t", "b": "\b", "f": "\f", "\\": "\\", "'": "'", '"': '"', "/": "/"}

    def parse_span(self, c: _Cursor):
        c.ws()
        c.expect("[")
        calls = []
        while True:
            c.ws()
            if c.peek() == "]":
                c.p += 1
                break
            name = c.word("(,[]")
            if not name or c.peek() != "(":
                raise _Malformed()
            c.p += 1
            args: Dict = {}
            while True:
                c.ws()
                if c.peek() == ")":
                    c.p += 1
                    break
                key = c.word("=,()")
                c.ws()
                if not key or c.peek() != "=":
                    raise _Malformed()                  # positional argument
                c.p += 1
                args[key] = self._value(c, 0)
                c.ws()
                if c.peek() == ",":
                    c.p += 1
                elif c.peek() != ")":
                    raise _Malformed()
            calls.append((name, args))
            c.ws()
            if c.peek() == ",":
                c.p += 1
            elif c.peek() != "]":
                raise _Malformed()
        if not calls:
            raise _Malformed()
        return calls

    def _string(self, c: _Cursor) -> str:
        q = c.peek()
        c.p += 1
        out = []
        while True:
            ch = c.peek()
            c.p += 1
            if ch == q:
                return "".join(out)
            if ch != "\\":
                out.append(ch)
                continue
            e = c.peek()
            c.p += 1
            if e == "u":
                if c.p + 4 > len(c.s):
                    raise _Incomplete()
                try:
                    out.append(chr(int(c.s[c.p:c.p + 4], 16)))
                except ValueError:
                    raise _Malformed()
                c.p += 4
            else:
                out.append(self._ESC.get(e, "\\" + e))

    def _value(self, c: _Cursor, depth: int):
        if depth > self.MAX_DEPTH:
            raise _Malformed()
        c.ws()
        ch = c.peek()
        if ch in "'\"":
            return self._string(c)
        if ch == "[":
            c.p += 1
            items = []
            while True:
                c.ws()
                if c.peek() == "]":
                    c.p += 1
                    return items
                items.append(self._value(c, depth + 1))
                c.ws()
                if c.peek() == ",":
                    c.p += 1
                elif c.peek() != "]":
                    raise _Malformed()
        if ch == "{":
            c.p += 1
            obj: Dict = {}
            while True:
                c.ws()
                if c.peek() == "}":
                    c.p += 1
                    return obj
                if c.peek() not in "'\"":
                    raise _Malformed()
                key = self._string(c)
                c.ws()
                c.expect(":")
                obj[key] = self._value(c, depth + 1)
                c.ws()
                if c.peek() == ",":
                    c.p += 1
                elif c.peek() != "}":
                    raise _Malformed()
        word = c.word(",)]}")
        val, ok = _bare(word)
        if not word or not ok:
            raise _Malformed()
        return val


def make_tool_call_parser(dialect: str):
    """The parser of a model family's tool-call syntax (``detect_dialect`` names the family)."""
    return {"gemma": GemmaToolCallParser, "lfm2": Lfm2ToolCallParser}.get(dialect, QwenToolCallParser)()


class ModelDialect:
    """The text surface of a model family beyond what its chat template renders: how reasoning is delimited, how tool calls
    are written, and which architecture names it goes with (reference: src/server/dialect.h:1-40)."""

    TABLE = {
        # name: (reasoning open, reasoning close, architectures it is expected with)
        "qwen": ("<think>", "</think>", ("qwen_hybrid", "qwen_hybrid_moe", "qwen4_exp")),
        "gemma": ("<|channel>thought\n", "<channel|>", ("gemma",)),
        "lfm2": ("<think>", "</think>", ("lfm2_moe",)),
        "llama": ("<think>", "</think>", ("llama",)),
    }

    def __init__(self, name: str):
        if name == "qwen4_exp":
            name = "qwen"            # the 4-stream MoE family shares the hybrid family's template, markers and tool-call syntax
        if name not in self.TABLE:
            raise ValueError(f"unknown dialect {name!r}; one of {sorted(self.TABLE)}")
        self.name = name
        self.reasoning_open, self.reasoning_close, self.archs = self.TABLE[name]

    def reasoning_splitter(self, start_in_think: bool = False) -> "ReasoningSplitter":
        return ReasoningSplitter(start_in_think, self.reasoning_open, self.reasoning_close)

    def tool_call_parser(self):
        return make_tool_call_parser(self.name)

    def cross_check(self, arch: str) -> Optional[str]:
        """A warning line when the dialect was forced onto a model of another family (the server still starts: a fine-tune
        may keep its base architecture and change its surface syntax), else None."""
        if arch and arch not in self.archs:
            return f"dialect {self.name!r} is normally used with {list(self.archs)}, the model's architecture is {arch!r}"
        return None


def select_dialect(choice: str, model_id: str, arch: str = "") -> ModelDialect:
    """``choice``: "auto" (from the model id and architecture) or a dialect name."""
    return ModelDialect(detect_dialect(model_id, arch) if choice in ("", "auto", None) else choice)


def detect_dialect(model_id: str, arch: str = "") -> str:
    """Model family -> which tool-call / reasoning conventions apply (reference: src/server/dialect.*)."""
    s = (model_id + " " + arch).lower()
    if "gemma" in s:
        return "gemma"
    if "lfm" in s:
        return "lfm2"
    if "llama" in s:
        return "llama"
    return "qwen"
