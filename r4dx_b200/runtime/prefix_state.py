"""Token-exact prefix reuse between requests, with the prompt checkpoint as a fallback.

The model holds one sequence.  Given the tokens it has been fed so far and the next request's prompt,
``plan`` picks the cheapest way to get the model to "prompt consumed":
  * extend    -- the fed tokens are a prefix of the prompt: feed only the tail;
  * restore   -- the saved checkpoint (taken after a previous prompt) is a prefix: roll the recurrent
                 state back to it and feed the tail (a hybrid model cannot rewind otherwise);
  * reset     -- start over.
(reference behaviour: src/server/prefix_state.h:1-60, src/server/engine.cpp:736-780)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence


@dataclass
class PrefixPlan:
    action: str              # "extend" | "restore" | "reset"
    feed_from: int           # index into the prompt where feeding starts
    reused: int              # tokens not recomputed


class PrefixState:
    def __init__(self):
        self.fed: List[int] = []              # tokens the model state reflects
        self.checkpoint: Optional[List[int]] = None
        self.valid = True

    def invalidate(self) -> None:
        self.fed = []
        self.checkpoint = None
        self.valid = False

    def plan(self, prompt: Sequence[int], min_tail: int = 1) -> PrefixPlan:
        """At least ``min_tail`` tokens are always fed so that the call produces fresh logits."""
        prompt = list(prompt)
        n = len(prompt)
        if self.valid and self.fed and len(self.fed) <= n - min_tail and prompt[:len(self.fed)] == self.fed:
            return PrefixPlan("extend", len(self.fed), len(self.fed))
        ck = self.checkpoint
        if self.valid and ck and len(ck) <= n - min_tail and prompt[:len(ck)] == ck:
            return PrefixPlan("restore", len(ck), len(ck))
        return PrefixPlan("reset", 0, 0)

    def commit(self, fed_tokens: Sequence[int], checkpoint_len: Optional[int] = None) -> None:
        self.fed = list(fed_tokens)
        self.valid = True
        if checkpoint_len is not None:
            self.checkpoint = self.fed[:checkpoint_len]
