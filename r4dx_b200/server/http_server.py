"""OpenAI-compatible HTTP front end: GET /health, GET /v1/models, POST /v1/chat/completions,
POST /v1/completions (JSON or SSE streaming with a final ``data: [DONE]``), 429 when the queue is full
(reference: src/server/http_server.cpp:136-285, docs/server.md:7-46)."""
from __future__ import annotations

import json
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional

from ..runtime.sampler import SampleParams
from .engine import Engine, EngineFatal, GenRequest, QueueFull


class BadRequest(ValueError):
    pass


def parse_sampling(body: Dict, defaults: Dict) -> SampleParams:
    def num(key, default, lo=None, hi=None, cast=float):
        v = body.get(key, default)
        if v is None:
            v = default
        try:
            v = cast(v)
        except (TypeError, ValueError):
            raise BadRequest(f"'{key}' must be a number")
        if (lo is not None and v < lo) or (hi is not None and v > hi):
            raise BadRequest(f"'{key}' out of range")
        return v
    return SampleParams(temperature=num("temperature", defaults.get("temperature", 1.0), 0.0, 10.0),
                        top_k=num("top_k", defaults.get("top_k", 0), 0, None, int),
                        top_p=num("top_p", defaults.get("top_p", 1.0), 0.0, 1.0),
                        min_p=num("min_p", defaults.get("min_p", 0.0), 0.0, 1.0),
                        seed=num("seed", int(time.time_ns() % (2**31)), None, None, int),
                        repetition_penalty=num("repetition_penalty", defaults.get("repetition_penalty", 1.0), 0.01, 10.0))


def message_text(m: Dict, images: Optional[list] = None, audios: Optional[list] = None) -> str:
    """Flattens OpenAI content parts; every image / audio part becomes a numbered marker and its payload is appended to
    ``images`` / ``audios``."""
    c = m.get("content", "")
    if isinstance(c, list):
        parts = []
        for p in c:
            if p.get("type") == "text":
                parts.append(p.get("text", ""))
            elif p.get("type") == "image_url":
                if images is None:
                    raise BadRequest("this model was loaded without a vision tower")
                u = p.get("image_url")
                from ..runtime.image_prompt import MARK
                parts.append(MARK % len(images))
                images.append(u.get("url", "") if isinstance(u, dict) else str(u))
            elif p.get("type") == "input_audio":
                if audios is None:
                    raise BadRequest("this model was loaded without an audio embedder")
                from ..runtime.image_prompt import AUDIO_MARK
                parts.append(AUDIO_MARK % len(audios))
                audios.append(p.get("input_audio", ""))
        c = "".join(parts)
    if not isinstance(c, str):
        raise BadRequest("message content must be a string or a list of parts")
    return c


class ApiServer:
    def __init__(self, engine: Engine, tokenizer, template, model_id: str, host: str = "127.0.0.1", port: int = 8080,
                 max_tokens_default: int = 512, defaults: Optional[Dict] = None, spec_k: int = 0, vision_config=None,
                 image_token_id: int = -1, audio_token_id: int = -1):
        self.vision_config, self.image_token_id = vision_config, image_token_id
        self.audio_token_id = audio_token_id          # >= 0 when the engine holds an audio embedder
        self.engine, self.tk, self.template, self.model_id = engine, tokenizer, template, model_id
        self.max_tokens_default = max_tokens_default
        self.defaults = defaults or {}
        self.spec_k = spec_k
        outer = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _json(self, code: int, obj: Dict):
                data = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def _error(self, code: int, msg: str, kind: str = "invalid_request_error"):
                self._json(code, {"error": {"message": msg, "type": kind, "code": code}})

            def do_GET(self):
                if self.path == "/health":
                    if outer.engine.fatal:
                        return self._json(503, {"status": "tp_fatal", "detail": outer.engine.fatal})
                    return self._json(200, {"status": "ok"})
                if self.path == "/metrics":
                    st = getattr(outer.engine, "stats", {})
                    text = "".join(f"# TYPE r4dxb_{k}_total counter\nr4dxb_{k}_total {v}\n" for k, v in st.items())
                    data = text.encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                    return
                if self.path == "/v1/models":
                    return self._json(200, {"object": "list", "data": [{"id": outer.model_id, "object": "model", "owned_by": "r4dx_b200"}]})
                self._error(404, "not found")

            def do_POST(self):
                try:
                    n = int(self.headers.get("Content-Length", "0"))
                    body = json.loads(self.rfile.read(n) or b"{}")
                    if not isinstance(body, dict):
                        raise BadRequest("body must be a JSON object")
                except BadRequest as e:
                    return self._error(400, str(e))
                except Exception:
                    return self._error(400, "body is not valid JSON")
                try:
                    if self.path == "/v1/chat/completions":
                        return outer._chat(self, body)
                    if self.path == "/v1/completions":
                        return outer._completion(self, body)
                except BadRequest as e:
                    return self._error(400, str(e))
                except QueueFull:
                    return self._error(429, "the request queue is full, retry later", "rate_limit_error")
                except EngineFatal as e:
                    return self._json(503, {"error": {"message": f"the engine is down: {e}", "type": "tp_fatal", "code": 503}})
                except BrokenPipeError:
                    return
                self._error(404, "not found")

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self.httpd.server_address[1]
        self.thread: Optional[threading.Thread] = None

    # ---- request building ----
    def _common(self, body: Dict, prompt_ids: List[int], chat: bool) -> GenRequest:
        mt = body.get("max_completion_tokens", body.get("max_tokens", self.max_tokens_default))
        if not isinstance(mt, int) or mt < 1:
            raise BadRequest("'max_tokens' must be a positive integer")
        stop = body.get("stop") or []
        if isinstance(stop, str):
            stop = [stop]
        if not isinstance(stop, list) or not all(isinstance(s, str) for s in stop):
            raise BadRequest("'stop' must be a string or a list of strings")
        params = parse_sampling(body, self.defaults)
        return GenRequest(prompt_ids=prompt_ids, max_tokens=mt, params=params, stop=stop, stream=bool(body.get("stream", False)),
                          parse_tools=chat and bool(body.get("tools")), spec_k=self.spec_k)

    def _chat(self, h, body: Dict):
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise BadRequest("'messages' must be a non-empty list")
        norm = []
        urls: list = []
        clips: list = []
        for m in msgs:
            if not isinstance(m, dict) or "role" not in m:
                raise BadRequest("every message needs a role")
            norm.append({**m, "content": message_text(m, urls if self.vision_config is not None else None,
                                                      clips if self.audio_token_id >= 0 else None)})
        thinking = body.get("enable_thinking", (body.get("chat_template_kwargs") or {}).get("enable_thinking"))
        prompt = self.template.render(norm, add_generation_prompt=True, tools=body.get("tools"), enable_thinking=thinking)
        if urls or clips:
            from ..runtime import image_prompt as IP
            try:
                imgs = [IP.decode_image(u) for u in urls]
                spans = [(IP.MARK % i, self.image_token_id, IP.image_token_count(im, self.vision_config)) for i, im in enumerate(imgs)]
                rows = [self.engine.audio.embed_clip(IP.decode_audio(c)) for c in clips]
                spans += [(IP.AUDIO_MARK % i, self.audio_token_id, int(r.shape[0])) for i, r in enumerate(rows)]
                ids = IP.assemble_media_prompt(prompt, spans, self.tk.encode)
            except ValueError as e:
                raise BadRequest(str(e))
            req = self._common(body, ids, chat=True)
            req.images, req.image_token_id = imgs, self.image_token_id
            req.audio_rows, req.audio_token_id = rows, self.audio_token_id
        else:
            req = self._common(body, self.tk.encode(prompt), chat=True)
        self._serve(h, req, chat=True)

    def _completion(self, h, body: Dict):
        prompt = body.get("prompt")
        if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            ids = prompt
        elif isinstance(prompt, str):
            ids = self.tk.encode(prompt)
        else:
            raise BadRequest("'prompt' must be a string or a list of token ids")
        if not ids:
            raise BadRequest("'prompt' is empty")
        self._serve(h, self._common(body, ids, chat=False), chat=False)

    # ---- response ----
    def _serve(self, h, req: GenRequest, chat: bool):
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        created = int(time.time())
        obj = "chat.completion" if chat else "text_completion"
        if not req.stream:
            job = self.engine.submit(req)
            job.done.wait()
            r = job.result
            if r.error:
                return h._error(500, r.error, "server_error")
            if chat:
                msg = {"role": "assistant", "content": r.text}
                if r.reasoning:
                    msg["reasoning_content"] = r.reasoning
                if r.tool_calls:
                    msg["tool_calls"] = r.tool_calls
                choice = {"index": 0, "message": msg, "finish_reason": r.finish_reason}
            else:
                choice = {"index": 0, "text": r.text, "finish_reason": r.finish_reason}
            return h._json(200, {"id": rid, "object": obj, "created": created, "model": self.model_id, "choices": [choice],
                                 "usage": self._usage(r), "timings": self._timings(r)})
        # streaming
        q: "queue.Queue" = queue.Queue()
        job = self.engine.submit(req, on_delta=lambda c, r: q.put((c, r)))
        h.send_response(200)
        h.send_header("Content-Type", "text/event-stream")
        h.send_header("Cache-Control", "no-cache")
        h.send_header("Connection", "close")
        h.end_headers()

        def send(payload: Dict):
            h.wfile.write(b"data: " + json.dumps(payload).encode() + b"\n\n")
            h.wfile.flush()

        def chunk(delta: Dict, finish=None, extra=None):
            ch = {"index": 0, "finish_reason": finish}
            if chat:
                ch["delta"] = delta
            else:
                ch["text"] = delta.get("content", "")
            d = {"id": rid, "object": obj + ".chunk" if chat else obj, "created": created, "model": self.model_id, "choices": [ch]}
            if extra:
                d.update(extra)
            send(d)
        try:
            if chat:
                chunk({"role": "assistant", "content": ""})
            while not (job.done.is_set() and q.empty()):
                try:
                    c, r = q.get(timeout=0.05)
                except queue.Empty:
                    continue
                if r:
                    chunk({"reasoning_content": r})
                if c:
                    chunk({"content": c})
            res = job.result
            if res.error:
                send({"error": {"message": res.error, "type": "server_error"}})
            else:
                if res.tool_calls:
                    chunk({"tool_calls": [{**tc, "index": i} for i, tc in enumerate(res.tool_calls)]})
                chunk({}, finish=res.finish_reason, extra={"usage": self._usage(res), "timings": self._timings(res)})
            h.wfile.write(b"data: [DONE]\n\n")
            h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError):
            job.cancelled = True

    @staticmethod
    def _usage(r) -> Dict:
        return {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
                "total_tokens": r.prompt_tokens + r.completion_tokens,
                "prompt_tokens_details": {"cached_tokens": r.reused_tokens}}

    @staticmethod
    def _timings(r) -> Dict:
        return {"prefill_ms": round(r.prefill_ms, 3), "decode_ms": round(r.decode_ms, 3),
                "decode_tok_per_s": round(r.completion_tokens / (r.decode_ms / 1e3), 2) if r.decode_ms > 0 else None}

    def start(self) -> None:
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.thread.start()

    def serve_forever(self) -> None:
        self.httpd.serve_forever()

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
