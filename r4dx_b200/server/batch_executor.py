"""``--batch N`` serving: N sequence slots decoded together by one executor thread.

Request threads enqueue jobs; the executor admits waiting jobs into free slots (prefills are serialised, one
prompt at a time), waits a short gather window so that requests arriving together start together, then advances
every active slot by one token per batched decode call.  The front door is the same as the single-sequence
``Engine`` (submit / generate / shutdown), so the HTTP layer takes either
(reference: src/server/batch_executor.h:1-50: N request threads, one executor thread, 2 ms gather window,
serialised prefill).
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Callable, Dict, List, Optional, Protocol, Sequence

from ..runtime.sampler import Rng, apply_repetition_penalty, sample_canonical
from ..runtime.tokenizer import StreamDecoder
from .engine import EngineFatal, GenRequest, GenResult, QueueFull, _Job
from .parsers import ReasoningSplitter, detect_dialect, make_tool_call_parser
from .request_log import RequestLog


class BatchBackend(Protocol):
    slots: int
    slot_ctx: int

    def import_slot(self, slot: int, ids: Sequence[int]) -> int: ...
    def decode_batch(self, slots: Sequence[int], tokens: Sequence[int]) -> List[int]: ...
    def release_slot(self, slot: int) -> None: ...


class FakeBatchBackend:
    """CPU stand-in: a slot's next token is a hash of its token history (independent of the other slots)."""

    def __init__(self, slots: int = 4, slot_ctx: int = 4096, vocab: int = 256, eos: int = 0):
        self.slots, self.slot_ctx, self.vocab, self.eos = slots, slot_ctx, vocab, eos
        self.hist: Dict[int, List[int]] = {}
        self.batch_sizes: List[int] = []
        self.last_logits = None

    @staticmethod
    def _next(h: List[int], vocab: int) -> int:
        x = 1469598103934665603
        for t in h[-8:]:
            x = ((x ^ (t + 1)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return 1 + x % (vocab - 1)

    def import_slot(self, slot: int, ids: Sequence[int]) -> int:
        self.hist[slot] = list(ids)
        return self._next(self.hist[slot], self.vocab)

    def decode_batch(self, slots: Sequence[int], tokens: Sequence[int]) -> List[int]:
        self.batch_sizes.append(len(slots))
        out = []
        for s, t in zip(slots, tokens):
            self.hist[s].append(t)
            out.append(self._next(self.hist[s], self.vocab))
        return out

    def release_slot(self, slot: int) -> None:
        self.hist.pop(slot, None)


class _Active:
    def __init__(self, job: _Job, slot: int, tk, dialect: str = "qwen"):
        from .parsers import ModelDialect
        self.job, self.slot = job, slot
        d = ModelDialect(dialect)
        self.dec = StreamDecoder(tk)
        self.splitter = d.reasoning_splitter()
        self.tools = d.tool_call_parser() if job.req.parse_tools else None
        self.rng = Rng(job.req.params.seed)
        self.text_all = ""
        self.next_token = 0
        self.t_decode = time.perf_counter()


class BatchEngine:
    def __init__(self, backend: BatchBackend, tokenizer, max_queue: int = 64, gather_ms: float = 2.0,
                 request_log: Optional[RequestLog] = None):
        self.backend, self.tk = backend, tokenizer
        self.q: "queue.Queue[_Job]" = queue.Queue(maxsize=max_queue)
        self.gather_s = gather_ms / 1e3
        self.log = request_log or RequestLog(None)
        self.fatal: Optional[str] = None
        self.stats = {"requests": 0, "errors": 0, "tokens": 0, "steps": 0}
        self._stop = False
        self.worker = threading.Thread(target=self._loop, daemon=True)
        self.worker.start()

    # ---- front door (same as Engine) ----
    def submit(self, req: GenRequest, on_delta: Optional[Callable[[str, str], None]] = None) -> _Job:
        if self.fatal:
            raise EngineFatal(self.fatal)
        job = _Job(req, on_delta)
        try:
            self.q.put_nowait(job)
        except queue.Full:
            raise QueueFull("request queue is full")
        return job

    def generate(self, req: GenRequest, on_delta=None, timeout: Optional[float] = None) -> GenResult:
        job = self.submit(req, on_delta)
        job.done.wait(timeout)
        return job.result

    def shutdown(self) -> None:
        self._stop = True
        self.q.put(None)  # type: ignore[arg-type]
        self.worker.join(timeout=5)

    # ---- executor ----
    def _loop(self) -> None:
        active: Dict[int, _Active] = {}
        free = list(range(self.backend.slots - 1, -1, -1))
        eos = set(getattr(self.tk, "eos_ids", []))
        while not self._stop:
            # admit: block when idle, otherwise only take what is already waiting (after a short gather window)
            try:
                if not active:
                    job = self.q.get()
                    if job is None:
                        break
                    waiting = [job]
                    deadline = time.perf_counter() + self.gather_s
                    while len(waiting) < len(free):
                        left = deadline - time.perf_counter()
                        if left <= 0:
                            break
                        try:
                            j = self.q.get(timeout=left)
                        except queue.Empty:
                            break
                        if j is None:
                            self._stop = True
                            break
                        waiting.append(j)
                else:
                    waiting = []
                    while len(waiting) < len(free):
                        try:
                            j = self.q.get_nowait()
                        except queue.Empty:
                            break
                        if j is None:
                            self._stop = True
                            break
                        waiting.append(j)
            except Exception as e:       # pragma: no cover - queue errors are fatal
                self.fatal = str(e)
                break
            for job in waiting:          # serialised prefill
                slot = free.pop()
                try:
                    self._admit(job, slot, active, eos)
                except Exception as e:
                    self._fail(job, e)
                    self.backend.release_slot(slot)
                    free.append(slot)
            if not active:
                continue
            # one batched step for every active slot
            order = sorted(active)
            try:
                nxt = self.backend.decode_batch(order, [active[s].next_token for s in order])
                self.stats["steps"] += 1
            except Exception as e:
                for s in order:
                    self._fail(active[s].job, e)
                    self.backend.release_slot(s)
                    free.append(s)
                active.clear()
                continue
            rows = getattr(self.backend, "last_logits", None)
            for j, (s, tok) in enumerate(zip(order, nxt)):
                a = active[s]
                try:                     # one bad request fails alone; the executor and the other slots go on
                    tok = self._pick(a, tok, None if rows is None else rows[j])
                    done = self._consume(a, tok, eos)
                except Exception as e:
                    self._fail(a.job, e)
                    done = True
                else:
                    if done:
                        self._finish(a)
                if done:
                    self.backend.release_slot(s)
                    free.append(s)
                    del active[s]
        for a in active.values():
            a.job.result.finish_reason = "cancelled"
            self._finish(a)

    def _pick(self, a: "_Active", greedy_tok: int, row) -> int:
        """The slot's next token: the backend's greedy pick, or - for a sampling request when the backend exposes the
        logits row - one draw of the request's own generator from the penalised row (same sampler as the single-sequence
        engine, one draw per emitted token)."""
        p = a.job.req.params
        if row is None or (p.greedy and p.repetition_penalty == 1.0):
            return greedy_tok
        lg = row.detach().to("cpu", dtype=__import__("torch").float32).contiguous().clone()
        if p.repetition_penalty != 1.0:
            apply_repetition_penalty(lg, list(a.job.req.prompt_ids) + list(a.job.result.token_ids), p.repetition_penalty)
        if p.greedy:
            return int(lg.argmax().item())
        return sample_canonical(lg, p, a.rng.next())

    def _admit(self, job: _Job, slot: int, active: Dict[int, "_Active"], eos) -> None:
        req, res = job.req, job.result
        self.stats["requests"] += 1
        res.prompt_tokens = len(req.prompt_ids)
        if len(req.prompt_ids) + req.max_tokens > self.backend.slot_ctx:
            raise ValueError(f"prompt ({len(req.prompt_ids)}) + max_tokens ({req.max_tokens}) exceeds the slot context "
                             f"({self.backend.slot_ctx})")
        t0 = time.perf_counter()
        first = self.backend.import_slot(slot, req.prompt_ids)
        res.prefill_ms = (time.perf_counter() - t0) * 1e3
        cfg = getattr(self.backend, "config", None)
        a = _Active(job, slot, self.tk, detect_dialect(getattr(self.backend, "model_id", ""), getattr(cfg, "arch", "")))
        prow = getattr(self.backend, "last_prefill_logits", None)      # the row the first token is picked from, if kept
        first = self._pick(a, first, prow)
        if self._consume(a, first, eos):
            self._finish(a)
            raise_slot_free = True
        else:
            raise_slot_free = False
            active[slot] = a
        if raise_slot_free:
            raise _SlotDone()

    def _consume(self, a: "_Active", tok: int, eos) -> bool:
        """Takes one generated token; True when the request is finished."""
        req, res = a.job.req, a.job.result
        if tok in eos:
            res.finish_reason = "stop"
            return True
        res.token_ids.append(tok)
        a.next_token = tok
        piece = a.dec.feed(tok)
        if piece:
            a.text_all += piece
            for s in req.stop:
                j = a.text_all.find(s)
                if j >= 0:
                    piece = piece[:max(0, len(piece) - (len(a.text_all) - j))]
                    self._emit(a, piece)
                    res.finish_reason = "stop"
                    return True
            self._emit(a, piece)
        if len(res.token_ids) >= req.max_tokens:
            res.finish_reason = "length"
            return True
        if a.job.cancelled:
            res.finish_reason = "cancelled"
            return True
        return False

    def _emit(self, a: "_Active", piece: str) -> None:
        c, r = a.splitter.feed(piece)
        if a.tools is not None and c:
            c = a.tools.feed(c)
        a.job.result.text += c
        a.job.result.reasoning += r
        if a.job.on_delta and (c or r):
            a.job.on_delta(c, r)

    def _finish(self, a: "_Active") -> None:
        res = a.job.result
        tail = a.dec.flush()
        if tail and res.finish_reason != "stop":
            self._emit(a, tail)
        c, r = a.splitter.flush()
        if a.tools is not None:
            c = a.tools.feed(c) + a.tools.flush()
            res.tool_calls = a.tools.calls
            if a.tools.calls:
                res.finish_reason = "tool_calls"
        res.text += c
        res.reasoning += r
        if a.job.on_delta and (c or r):
            a.job.on_delta(c, r)
        res.decode_ms = (time.perf_counter() - a.t_decode) * 1e3
        self.stats["tokens"] += len(res.token_ids)
        self._log(a.job)
        a.job.done.set()

    def _fail(self, job: _Job, e: Exception) -> None:
        if isinstance(e, _SlotDone):
            return
        job.result.error = f"{type(e).__name__}: {e}"
        job.result.finish_reason = "error"
        self.stats["errors"] += 1
        self._log(job)
        job.done.set()

    def _log(self, job: _Job) -> None:
        r = job.result
        self.log.write(request_id=job.req.request_id, prompt_tokens=r.prompt_tokens, completion_tokens=r.completion_tokens,
                       reused_tokens=0, prefill_ms=r.prefill_ms, decode_ms=r.decode_ms, finish_reason=r.finish_reason,
                       prompt_ids=job.req.prompt_ids, completion_ids=r.token_ids, error=r.error)


class _SlotDone(Exception):
    """The request finished during admission (first token was the end): the slot is free again."""
