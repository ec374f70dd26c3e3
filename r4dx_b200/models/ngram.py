"""N-gram (prompt-lookup) drafter: proposes the tokens that followed the most recent earlier occurrence of the current
suffix.  No weights and no device work; the target's verify window keeps the output exact, so the only cost of a wrong
guess is the wider window.  It pays off on text that repeats its own context (code edits, retrieval answers, long
structured output).  (reference: the n-gram speculation simulator under tools/ngram and the drafter interface of
src/model/model.h:559-632.)

The class has the interface ``runtime.text_model.LocalTextModel`` expects of a drafter (``draft``, ``after_verify``,
``prefill_hook``, ``after_prefill``, ``reset``), so ``--ngram`` can stand in for the MTP head or the block-diffusion drafter.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple


class NgramIndex:
    """Token history with, for every n in [min_n, max_n], a map from each n-gram to the position right after its latest
    occurrence.  Appending is O(max_n); a lookup tries the longest suffix first."""

    def __init__(self, min_n: int = 2, max_n: int = 4):
        if not 1 <= min_n <= max_n:
            raise ValueError("need 1 <= min_n <= max_n")
        self.min_n, self.max_n = min_n, max_n
        self.tokens: List[int] = []
        self._next: Dict[Tuple[int, ...], int] = {}
        self._prev: Dict[Tuple[int, ...], int] = {}     # the occurrence before the latest one (a suffix always matches itself)

    def clear(self) -> None:
        self.tokens, self._next, self._prev = [], {}, {}

    def append(self, tok: int) -> None:
        self.tokens.append(int(tok))
        end = len(self.tokens)
        for n in range(self.min_n, self.max_n + 1):
            if end >= n:
                key = tuple(self.tokens[end - n:end])
                if key in self._next:
                    self._prev[key] = self._next[key]
                self._next[key] = end

    def extend(self, toks: Sequence[int]) -> None:
        for t in toks:
            self.append(t)

    def propose(self, k: int) -> List[int]:
        """Up to k tokens that followed the latest earlier occurrence of the current suffix (longest n first)."""
        end = len(self.tokens)
        for n in range(min(self.max_n, end), self.min_n - 1, -1):
            key = tuple(self.tokens[end - n:end])
            at = self._next.get(key)
            if at == end:                       # the suffix itself: take the occurrence before it
                at = self._prev.get(key)
            if at is not None and at < end:
                out = self.tokens[at:at + k]
                if out:
                    return list(out)
        return []


class NgramDrafter:
    kind = "ngram"

    def __init__(self, min_n: int = 2, max_n: int = 4):
        self.index = NgramIndex(min_n, max_n)
        self.rounds = 0
        self.proposed = 0
        self.accepted = 0

    # ---- drafter interface ---------------------------------------------------------------------
    def reset(self) -> None:
        self.index.clear()

    def prefill_hook(self, ids):
        return None                             # nothing to keep in lock-step with the target's hidden states

    def after_prefill(self, ids, tok: int) -> None:
        self.index.extend(int(t) for t in (ids.tolist() if hasattr(ids, "tolist") else ids))

    def draft(self, anchor: int, k: int) -> List[int]:
        """The anchor is the token about to be fed; proposals continue the history ending with it."""
        self.index.append(anchor)
        self._anchor_fed = True
        out = self.index.propose(k)
        self.rounds += 1
        self.proposed += len(out)
        return out

    def after_verify(self, anchor: int, drafts: List[int], emitted: List[int]) -> None:
        """The target committed the anchor and the accepted drafts (all emitted tokens but the last, which is the next anchor)."""
        if not getattr(self, "_anchor_fed", False):
            self.index.append(anchor)
        self._anchor_fed = False
        a = len(emitted) - 1
        self.accepted += a
        self.index.extend(drafts[:a])

    def acceptance(self) -> float:
        return self.accepted / max(1, self.rounds)


def simulate(tokens: Sequence[int], prompt_len: int, k: int = 4, min_n: int = 2, max_n: int = 4) -> dict:
    """Replays a finished generation (``tokens`` = prompt + output) through the drafter as a lossless speculative loop would
    and reports what it would have saved: target calls, mean accepted drafts per call, mean window width.
    (reference: tools/ngram, the n-gram speculation simulator.)"""
    d = NgramDrafter(min_n, max_n)
    d.after_prefill(list(tokens[:prompt_len]), 0)
    pos, calls, accepted, width = prompt_len, 0, 0, 0
    n = len(tokens)
    while pos < n:
        anchor = tokens[pos]                     # already known: emitted by the previous call (or the prefill)
        drafts = d.draft(anchor, k)
        a = 0
        while a < len(drafts) and pos + 1 + a < n and drafts[a] == tokens[pos + 1 + a]:
            a += 1
        d.after_verify(anchor, drafts, list(drafts[:a]) + [0])
        calls += 1
        accepted += a
        width += 1 + len(drafts)
        pos += 1 + a
    out_tokens = n - prompt_len
    return {"output_tokens": out_tokens, "target_calls": calls, "accepted_per_call": accepted / max(1, calls),
            "mean_window": width / max(1, calls), "calls_saved_frac": 1.0 - calls / max(1, out_tokens)}
