"""Opt-in JSONL request log.  Privacy by construction: counts, timings and cache savings only; token ids
are written only when explicitly asked for, text never (reference: src/server/request_log.h:1-60)."""
from __future__ import annotations

import json
import threading
import time
from typing import Optional, Sequence


class RequestLog:
    def __init__(self, path: Optional[str], log_tokens: bool = False):
        self.path = path
        self.log_tokens = log_tokens
        self._lock = threading.Lock()

    def write(self, *, request_id: str, prompt_tokens: int, completion_tokens: int, reused_tokens: int,
              prefill_ms: float, decode_ms: float, finish_reason: str, spec_rounds: int = 0,
              spec_emitted: int = 0, prompt_ids: Optional[Sequence[int]] = None,
              completion_ids: Optional[Sequence[int]] = None, error: Optional[str] = None) -> None:
        if not self.path:
            return
        rec = {"ts": time.time(), "id": request_id, "prompt_tokens": prompt_tokens,
               "completion_tokens": completion_tokens, "prefix_cache_tokens": reused_tokens,
               "prefill_ms": round(prefill_ms, 3), "decode_ms": round(decode_ms, 3), "finish_reason": finish_reason,
               "spec_rounds": spec_rounds, "spec_emitted": spec_emitted}
        if error:
            rec["error"] = error
        if self.log_tokens:
            rec["prompt_ids"] = list(prompt_ids or [])
            rec["completion_ids"] = list(completion_ids or [])
        with self._lock, open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")
