"""Serving engine: a bounded request queue and one worker thread that owns the model.

One request runs at a time (the model holds one sequence); requests that arrive while the queue is
full are rejected (HTTP 429).  Per request: render + tokenize, prefix-reuse plan (extend / restore
checkpoint / reset), prefill, decode loop (greedy graph replay, sampled, or speculative), streamed
through a sink.  A failed request invalidates the prefix state and the next request's reset() runs
the model's recovery (reference: src/server/engine.h:1-120, engine.cpp:123-324, 324-1619).
"""
from __future__ import annotations

import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from ..runtime.prefix_state import PrefixState
from ..runtime.sampler import Rng, SampleParams
from ..runtime.text_model import ModelStateError, TextModel
from ..runtime.tokenizer import StreamDecoder
from .parsers import ReasoningSplitter, detect_dialect, make_tool_call_parser, select_dialect
from .request_log import RequestLog


class EngineFatal(RuntimeError):
    """The engine can no longer serve (e.g. a tensor-parallel rank was lost and recovery failed)."""


class QueueFull(RuntimeError):
    pass


@dataclass
class GenRequest:
    prompt_ids: List[int]
    max_tokens: int = 256
    params: SampleParams = field(default_factory=SampleParams)
    stop: List[str] = field(default_factory=list)
    stream: bool = False
    parse_tools: bool = False
    thinking: bool = True
    request_id: str = field(default_factory=lambda: "req_" + uuid.uuid4().hex[:16])
    spec_k: int = 0
    images: List = field(default_factory=list)          # uint8 [H, W, 3] tensors, in the order of the image placeholders
    image_token_id: int = -1
    audio_rows: List = field(default_factory=list)      # one [frames, hidden] tensor per clip, in the order of the audio placeholders
    audio_token_id: int = -1


@dataclass
class GenResult:
    text: str = ""
    reasoning: str = ""
    tool_calls: List[Dict] = field(default_factory=list)
    token_ids: List[int] = field(default_factory=list)
    finish_reason: str = "stop"
    prompt_tokens: int = 0
    reused_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    error: Optional[str] = None

    @property
    def completion_tokens(self) -> int:
        return len(self.token_ids)


class _Job:
    def __init__(self, req: GenRequest, on_delta: Optional[Callable[[str, str], None]]):
        self.req = req
        self.on_delta = on_delta
        self.done = threading.Event()
        self.result = GenResult()
        self.cancelled = False


class Engine:
    def __init__(self, model: TextModel, tokenizer, max_queue: int = 8, prompt_checkpoint: bool = True,
                 request_log: Optional[RequestLog] = None, vision=None, audio=None):
        self.model = model
        self.vision = vision               # object with encode_images(list of uint8 images) -> [tokens, hidden]
        self.audio = audio                 # object with embed_clip(wav bytes) -> [frames, hidden] (host side, once per clip)
        self.dialect = "auto"              # "auto" or a dialect name (reasoning markers and tool-call syntax of the family)
        self.tk = tokenizer
        self.q: "queue.Queue[_Job]" = queue.Queue(maxsize=max_queue)
        self.prefix = PrefixState()
        self.prompt_checkpoint = prompt_checkpoint
        self.log = request_log or RequestLog(None)
        self.fatal: Optional[str] = None
        self._stop = False
        self.worker = threading.Thread(target=self._loop, daemon=True)
        self.worker.start()
        self.stats = {"requests": 0, "errors": 0, "tokens": 0}

    # ---- front door ----
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

    # ---- worker ----
    def _loop(self) -> None:
        while not self._stop:
            job = self.q.get()
            if job is None:
                break
            try:
                self._run(job)
            except Exception as e:                      # the request fails, the server lives on
                job.result.error = f"{type(e).__name__}: {e}"
                job.result.finish_reason = "error"
                self.prefix.invalidate()
                self.stats["errors"] += 1
                lost = getattr(self.model, "fatal", None)       # a rank group that cannot be recovered ends the service
                if lost:
                    self.fatal = str(lost)
            finally:
                r = job.result
                self.log.write(request_id=job.req.request_id, prompt_tokens=r.prompt_tokens,
                               completion_tokens=r.completion_tokens, reused_tokens=r.reused_tokens,
                               prefill_ms=r.prefill_ms, decode_ms=r.decode_ms, finish_reason=r.finish_reason,
                               prompt_ids=job.req.prompt_ids, completion_ids=r.token_ids, error=r.error)
                job.done.set()

    def _run(self, job: _Job) -> None:
        req, res, m = job.req, job.result, self.model
        self.stats["requests"] += 1
        prompt = list(req.prompt_ids)
        res.prompt_tokens = len(prompt)
        if len(prompt) + req.max_tokens > m.max_ctx:
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({req.max_tokens}) exceeds the context ({m.max_ctx})")
        overrides = None
        if req.images:
            # image requests run from a clean state: a token-exact prefix says nothing about the pixels behind it
            if self.vision is None:
                raise ValueError("this model was loaded without a vision tower")
            import torch
            emb = self.vision.encode_images(req.images)
            where = torch.tensor([i for i, t in enumerate(prompt) if t == req.image_token_id], dtype=torch.long)
            if where.numel() != emb.shape[0]:
                raise ValueError(f"{where.numel()} image placeholder tokens for {emb.shape[0]} image embeddings")
            overrides = (where, emb)
            self.prefix.invalidate()
        if req.audio_rows:
            import torch
            rows = torch.cat([r for r in req.audio_rows], 0)
            where = torch.tensor([i for i, t in enumerate(prompt) if t == req.audio_token_id], dtype=torch.long)
            if where.numel() != rows.shape[0]:
                raise ValueError(f"{where.numel()} audio placeholder tokens for {rows.shape[0]} audio rows")
            if overrides is not None:      # images and audio in one prompt: one override list, ordered by position
                pos = torch.cat([overrides[0], where])
                emb_all = torch.cat([overrides[1], rows.to(overrides[1].device, overrides[1].dtype)], 0)
                order = torch.argsort(pos)
                overrides = (pos[order], emb_all[order.to(emb_all.device)])
            else:
                overrides = (where, rows)
            self.prefix.invalidate()
        plan = self.prefix.plan(prompt) if self.prefix.valid else None
        t0 = time.perf_counter()
        if plan is None or plan.action == "reset":
            m.reset()                                    # also the recovery path after a failed request
            feed_from = 0
        elif plan.action == "restore":
            m.restore_checkpoint()
            feed_from = plan.feed_from
        else:
            feed_from = plan.feed_from
        res.reused_tokens = feed_from
        if overrides is not None and req.images and getattr(self.vision, "bidirectional_blocks", False):
            # this family's image rows attend to their whole block on sliding-window layers: the prefill gets the blocks
            from ..models.gemma_vision import find_blocks
            first = m.prefill(prompt[feed_from:], embed_overrides=overrides, image_blocks=find_blocks(prompt[feed_from:], req.image_token_id))
        elif overrides is not None:
            first = m.prefill(prompt[feed_from:], embed_overrides=overrides)
        else:
            first = m.prefill(prompt[feed_from:])
        if self.prompt_checkpoint:
            m.save_checkpoint()
        rng = Rng(req.params.seed)
        if not req.params.greedy or req.params.repetition_penalty != 1.0:
            first = m.sample_from_last(req.params, rng, prompt)
        res.prefill_ms = (time.perf_counter() - t0) * 1e3

        dec = StreamDecoder(self.tk)
        dialect = select_dialect(self.dialect, getattr(m, "model_id", ""), getattr(getattr(m, "config", None), "arch", ""))
        splitter = dialect.reasoning_splitter()
        tools = dialect.tool_call_parser() if req.parse_tools else None
        eos = set(getattr(self.tk, "eos_ids", []))
        fed = list(prompt)
        text_all = ""
        t1 = time.perf_counter()
        pending = [first]
        stop_hit = False
        while pending and not stop_hit:
            tok = pending.pop(0)
            if tok in eos:
                res.finish_reason = "stop"
                break
            res.token_ids.append(tok)
            piece = dec.feed(tok)
            if piece:
                text_all += piece
                for s in req.stop:
                    j = text_all.find(s)
                    if j >= 0:
                        piece = piece[:max(0, len(piece) - (len(text_all) - j))]
                        text_all = text_all[:j]
                        stop_hit = True
                        break
                self._emit(job, splitter, tools, piece)
            if stop_hit:
                res.finish_reason = "stop"
                break
            if len(res.token_ids) >= req.max_tokens:
                res.finish_reason = "length"
                break
            if job.cancelled:
                res.finish_reason = "cancelled"
                break
            if not pending:
                fed.append(tok)
                # a speculative round stages 1 + k rows: near the end of the context or of the answer it is cut to what
                # still fits (0: a plain step), so a request admitted up to the limit never overflows in its last rounds
                max_ctx = getattr(m, "max_ctx", None)
                k = req.spec_k
                if k > 0:
                    k = min(k, req.max_tokens - len(res.token_ids) - 1)
                    if max_ctx is not None:
                        k = min(k, max_ctx - len(fed) - 1)
                    k = max(k, 0)
                if k > 0 and req.params.greedy and req.params.repetition_penalty == 1.0:
                    emitted = m.decode_step_spec_greedy(tok, k)
                    fed += emitted[:-1]
                    pending = list(emitted)
                elif k > 0:
                    emitted = m.decode_step_spec_sampled(tok, k, req.params, rng, fed)
                    fed += emitted[:-1]
                    pending = list(emitted)
                elif req.params.greedy and req.params.repetition_penalty == 1.0:
                    pending = [m.decode_step_greedy(tok)]
                else:
                    pending = [m.decode_step_sampled(tok, req.params, rng, fed)]
        tail = dec.flush()
        if tail and not stop_hit:
            self._emit(job, splitter, tools, tail)
        c, r = splitter.flush()
        if tools is not None:
            c = tools.feed(c) + tools.flush()
            res.tool_calls = tools.calls
            if tools.calls:
                res.finish_reason = "tool_calls"
        res.text += c
        res.reasoning += r
        if job.on_delta and (c or r):
            job.on_delta(c, r)
        res.decode_ms = (time.perf_counter() - t1) * 1e3
        self.stats["tokens"] += len(res.token_ids)
        # the model state reflects exactly the tokens it was fed
        if req.images or req.audio_rows:      # rows computed from one clip's / picture's embeddings must never be reused
            self.prefix.invalidate()
        else:
            self.prefix.commit(fed[:m.position_count()], checkpoint_len=len(prompt) if self.prompt_checkpoint else None)

    def _emit(self, job: _Job, splitter: ReasoningSplitter, tools, piece: str) -> None:
        c, r = splitter.feed(piece)
        if tools is not None and c:
            c = tools.feed(c)
        job.result.text += c
        job.result.reasoning += r
        if job.on_delta and (c or r):
            job.on_delta(c, r)
