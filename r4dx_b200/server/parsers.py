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

    def __init__(self, start_in_think: bool = False):
        self.in_think = start_in_think
        self.buf = ""

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
