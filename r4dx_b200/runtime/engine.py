"""Public generation API over a model: sessions that move tokens between host and device.

``GreedySession.step`` is the end-to-end decode step a caller makes: the previous token goes from
pinned host memory to the device, one captured decode graph runs, the next token comes back through
pinned memory (the reference overlaps the same 4-byte read-back with streaming the previous
token: reference src/model/model.cpp:2186-2196).
"""
from __future__ import annotations

from typing import List

import torch


class GreedySession:
    def __init__(self, model):
        self.model = model
        self.h_in = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.h_out = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.h2d_bytes = self.h_in.numel() * 4
        self.d2h_bytes = self.h_out.numel() * 4
        model.enable_graphs((1,))
        self._begun = False

    def begin(self, first_token: int) -> None:
        self.model.decode_begin(first_token)
        self._begun = True

    def step(self, token: int) -> int:
        m = self.model
        if not self._begun:
            self.begin(token)
        self.h_in[0] = token
        m.buf.ids[:1].copy_(self.h_in, non_blocking=True)
        m.decode_step_graph()
        self.h_out.copy_(m.buf.next_ids[:1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(self.h_out[0])

    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> List[int]:
        tok = self.model.prefill(prompt)
        out = [tok]
        self.begin(tok)
        for _ in range(max_new_tokens - 1):
            tok = self.step(tok)
            out.append(tok)
        return out
