"""Serving layer on CPU fakes: engine, prefix reuse, recovery, OpenAI HTTP API, SSE, parsers, request log."""
import json
import threading
import urllib.error
import urllib.request

import pytest

from r4dx_b200.runtime.prefix_state import PrefixState
from r4dx_b200.runtime.sampler import SampleParams
from r4dx_b200.runtime.text_model import FakeTextModel
from r4dx_b200.runtime.tokenizer import ByteTokenizer, ChatTemplate, StreamDecoder
from r4dx_b200.server.engine import Engine, GenRequest, QueueFull
from r4dx_b200.server.http_server import ApiServer
from r4dx_b200.server.parsers import QwenToolCallParser, ReasoningSplitter
from r4dx_b200.server.request_log import RequestLog


def test_prefix_plan():
    p = PrefixState()
    assert p.plan([1, 2, 3]).action == "reset"
    p.commit([1, 2, 3, 9, 9], checkpoint_len=3)
    assert p.plan([1, 2, 3, 9, 9, 4]).action == "extend"
    pl = p.plan([1, 2, 3, 7])
    assert pl.action == "restore" and pl.feed_from == 3
    assert p.plan([5, 5]).action == "reset"
    assert p.plan([1, 2, 3]).action == "reset"       # nothing left to feed -> no fresh logits -> start over
    p.invalidate()
    assert p.plan([1, 2, 3, 9, 9, 4]).action == "reset"


def test_tokenizer_stream_decoder_holds_partial_utf8():
    tk = ByteTokenizer()
    ids = tk.encode("héllo <|im_end|>")
    assert tk.decode(ids) == "héllo "
    d = StreamDecoder(tk)
    pieces = [d.feed(i) for i in tk.encode("é")]
    assert pieces == ["", "é"]
    assert "<|im_start|>user" in ChatTemplate().render([{"role": "user", "content": "hi"}])


def test_reasoning_splitter_and_tool_parser_incremental():
    s = ReasoningSplitter()
    c = r = ""
    for piece in ["<th", "ink>let me ", "see</thi", "nk>\nans", "wer"]:
        dc, dr = s.feed(piece)
        c += dc; r += dr
    dc, dr = s.flush()
    assert (c + dc, r + dr) == ("answer", "let me see")
    t = QwenToolCallParser()
    out = ""
    for piece in ['ok <tool_', 'call>{"name": "f", "argum', 'ents": {"x": 1}}</tool_call> done']:
        out += t.feed(piece)
    out += t.flush()
    assert out == "ok  done" and t.calls[0]["function"]["name"] == "f"
    assert json.loads(t.calls[0]["function"]["arguments"]) == {"x": 1}


def _engine(**kw):
    return Engine(FakeTextModel(vocab=300, **kw), ByteTokenizer(300), max_queue=2)


def test_engine_generates_and_reuses_prefix(tmp_path):
    log = str(tmp_path / "req.jsonl")
    eng = Engine(FakeTextModel(vocab=300), ByteTokenizer(300), request_log=RequestLog(log))
    tk = ByteTokenizer(300)
    p1 = tk.encode("hello world")
    r1 = eng.generate(GenRequest(p1, max_tokens=8, params=SampleParams(temperature=0)))
    assert r1.error is None and 1 <= r1.completion_tokens <= 8 and r1.reused_tokens == 0
    # same prompt + the answer + a new turn: extends the fed prefix
    p2 = p1 + r1.token_ids + tk.encode(" more")
    r2 = eng.generate(GenRequest(p2, max_tokens=4, params=SampleParams(temperature=0)))
    assert r2.reused_tokens >= len(p1)
    # a different continuation of the latest prompt: the model cannot rewind, the prompt checkpoint can
    r3 = eng.generate(GenRequest(p2 + tk.encode("!!"), max_tokens=4, params=SampleParams(temperature=0)))
    assert r3.reused_tokens == len(p2)
    # determinism: greedy output is a pure function of the tokens
    eng2 = Engine(FakeTextModel(vocab=300), ByteTokenizer(300))
    assert eng2.generate(GenRequest(p1, max_tokens=8, params=SampleParams(temperature=0))).token_ids == r1.token_ids
    lines = [json.loads(l) for l in open(log)]
    assert len(lines) == 3 and "prompt_ids" not in lines[0] and lines[1]["prefix_cache_tokens"] >= len(p1)
    eng.shutdown(); eng2.shutdown()


def test_sampled_is_seed_deterministic():
    eng = _engine()
    tk = ByteTokenizer(300)
    a = eng.generate(GenRequest(tk.encode("abc"), max_tokens=12, params=SampleParams(temperature=0.9, top_p=0.9, seed=7)))
    b = eng.generate(GenRequest(tk.encode("abc"), max_tokens=12, params=SampleParams(temperature=0.9, top_p=0.9, seed=7)))
    c = eng.generate(GenRequest(tk.encode("abc"), max_tokens=12, params=SampleParams(temperature=0.9, top_p=0.9, seed=8)))
    assert a.token_ids == b.token_ids and a.token_ids != c.token_ids
    eng.shutdown()


def test_engine_recovers_after_a_model_fault():
    eng = _engine(fail_at_call=2)
    tk = ByteTokenizer(300)
    bad = eng.generate(GenRequest(tk.encode("xyz"), max_tokens=8, params=SampleParams(temperature=0)))
    assert bad.error and "injected" in bad.error
    good = eng.generate(GenRequest(tk.encode("xyz"), max_tokens=4, params=SampleParams(temperature=0)))
    assert good.error is None and good.reused_tokens == 0
    eng.shutdown()


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    return urllib.request.urlopen(req, timeout=20)


def test_http_api_roundtrip():
    eng = _engine()
    srv = ApiServer(eng, ByteTokenizer(300), ChatTemplate(), "fake-model", port=0)
    srv.start()
    try:
        assert json.load(urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/health"))["status"] == "ok"
        assert json.load(urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/v1/models"))["data"][0]["id"] == "fake-model"
        r = json.load(_post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}))
        assert r["object"] == "chat.completion" and r["choices"][0]["finish_reason"] in ("stop", "length")
        assert r["usage"]["completion_tokens"] <= 6 and "timings" in r
        c = json.load(_post(srv.port, "/v1/completions", {"prompt": "abc", "max_tokens": 3, "temperature": 0}))
        assert c["object"] == "text_completion"
        # streaming
        resp = _post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "temperature": 0, "stream": True})
        events = [l.decode().strip() for l in resp if l.strip()]
        assert events[-1] == "data: [DONE]"
        last = json.loads(events[-2][6:])
        assert last["choices"][0]["finish_reason"] in ("stop", "length") and "usage" in last
        # validation errors
        for body in ({"messages": []}, {"messages": [{"role": "user", "content": "x"}], "max_tokens": 0},
                     {"messages": [{"role": "user", "content": "x"}], "temperature": "hot"}):
            with pytest.raises(urllib.error.HTTPError) as e:
                _post(srv.port, "/v1/chat/completions", body)
            assert e.value.code == 400
    finally:
        srv.stop(); eng.shutdown()


def test_queue_full_gives_429():
    class Slow(FakeTextModel):
        def decode_step(self, token):
            import time
            time.sleep(0.05)
            return super().decode_step(token)
    eng = Engine(Slow(vocab=300), ByteTokenizer(300), max_queue=1)
    tk = ByteTokenizer(300)
    jobs = [eng.submit(GenRequest(tk.encode("a"), max_tokens=20, params=SampleParams(temperature=0)))]
    with pytest.raises(QueueFull):
        for _ in range(4):
            jobs.append(eng.submit(GenRequest(tk.encode("a"), max_tokens=20, params=SampleParams(temperature=0))))
    for j in jobs:
        j.cancelled = True
    eng.shutdown()


def test_batch_engine_runs_requests_together_and_independently():
    import threading
    from r4dx_b200.runtime.tokenizer import ByteTokenizer
    from r4dx_b200.server.batch_executor import BatchEngine, FakeBatchBackend
    from r4dx_b200.server.engine import GenRequest, QueueFull
    tk = ByteTokenizer()
    be = FakeBatchBackend(slots=3, vocab=200)
    eng = BatchEngine(be, tk, max_queue=4, gather_ms=20.0)
    prompts = [[5, 6, 7], [9, 9], [1, 2, 3, 4], [8]]
    results = [None] * 4

    def run(i):
        results[i] = eng.generate(GenRequest(prompt_ids=prompts[i], max_tokens=6 + i), timeout=10)

    th = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    # every stream equals the single-sequence continuation of its own prompt
    for i, r in enumerate(results):
        assert r.error is None and r.finish_reason == "length" and len(r.token_ids) == 6 + i
        h = list(prompts[i])
        for tok in r.token_ids:
            assert tok == FakeBatchBackend._next(h, 200)
            h.append(tok)
    assert max(be.batch_sizes) >= 2            # requests really shared decode steps
    assert eng.stats["requests"] == 4 and eng.stats["errors"] == 0
    # a prompt that cannot fit the slot is an error for that request only
    r = eng.generate(GenRequest(prompt_ids=[1] * 5000, max_tokens=4), timeout=10)
    assert r.finish_reason == "error" and "slot context" in r.error
    r = eng.generate(GenRequest(prompt_ids=[3, 3], max_tokens=2), timeout=10)
    assert r.error is None and len(r.token_ids) == 2
    eng.shutdown()


def test_image_parts_become_placeholder_tokens_and_embedding_overrides():
    import base64
    import io
    import torch
    from PIL import Image
    from r4dx_b200.models.vision import tiny_vision_config
    from r4dx_b200.runtime import image_prompt as IP
    vcfg = tiny_vision_config()

    class FakeVision:
        def __init__(self):
            self.seen = []

        def encode_images(self, images):
            self.seen.append([tuple(i.shape) for i in images])
            n = sum(IP.image_token_count(i, vcfg) for i in images)
            return torch.ones(n, 128)

    model = FakeTextModel(vocab=300)
    vis = FakeVision()
    eng = Engine(model, ByteTokenizer(300), vision=vis)
    srv = ApiServer(eng, ByteTokenizer(300), ChatTemplate(), "fake-vl", port=0, vision_config=vcfg, image_token_id=299)
    srv.start()
    try:
        buf = io.BytesIO()
        Image.new("RGB", (40, 24), (200, 10, 10)).save(buf, format="PNG")
        uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
        body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "what is "}, {"type": "image_url", "image_url": {"url": uri}},
                                                           {"type": "text", "text": " ?"}]}], "max_tokens": 4, "temperature": 0}
        r = json.load(_post(srv.port, "/v1/chat/completions", body))
        assert r["choices"][0]["finish_reason"] in ("stop", "length")
        assert vis.seen == [[(24, 40, 3)]]
        pos, rows = model.last_overrides
        n = IP.image_token_count(torch.zeros(24, 40, 3, dtype=torch.uint8), vcfg)
        assert pos.numel() == n == rows.shape[0] and n > 0
        assert all(model.history[int(p)] == 299 for p in pos)                  # overrides sit exactly on the placeholders
        assert model.history.count(299) == n
        assert r["usage"]["prompt_tokens"] > n
        # a plain-text request afterwards is unaffected, and a non-data URL is a 400
        r2 = json.load(_post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "temperature": 0}))
        assert r2["usage"]["completion_tokens"] <= 2 and model.last_overrides is None
        body["messages"][0]["content"][1]["image_url"]["url"] = "http://example.com/x.png"
        with pytest.raises(urllib.error.HTTPError) as e:
            _post(srv.port, "/v1/chat/completions", body)
        assert e.value.code == 400
        m = urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/metrics").read().decode()
        assert "r4dxb_requests_total" in m
    finally:
        srv.stop(); eng.shutdown()


def test_block_style_image_front_sizes_images_and_hands_the_blocks_to_the_prefill():
    """The family whose image rows form bidirectional blocks: the front object decides the soft-token count, and the
    engine passes the runs of image placeholders to the model's prefill."""
    import base64
    import io
    import torch
    from PIL import Image
    from r4dx_b200.models import gemma_vision as GV

    class Front:
        bidirectional_blocks = True

        def token_count(self, img):
            h, w = GV.target_size(int(img.shape[0]), int(img.shape[1]), 70)
            return (h // GV.SIDE) * (w // GV.SIDE)

        def encode_images(self, images):
            return torch.ones(sum(self.token_count(i) for i in images), 128)

    model = FakeTextModel(vocab=300)
    front = Front()
    eng = Engine(model, ByteTokenizer(300), vision=front)
    srv = ApiServer(eng, ByteTokenizer(300), ChatTemplate(), "fake-gemma", port=0, vision_config=front, image_token_id=299)
    srv.start()
    try:
        parts = [{"type": "text", "text": "a "}]
        for size in ((96, 96), (200, 100)):
            buf = io.BytesIO()
            Image.new("RGB", size, (10, 200, 10)).save(buf, format="PNG")
            parts += [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()}},
                      {"type": "text", "text": " b "}]
        r = json.load(_post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": parts}], "max_tokens": 2, "temperature": 0}))
        assert r["choices"][0]["finish_reason"] in ("stop", "length")
        blocks = model.last_image_blocks
        assert len(blocks) == 2 and all(b > a for a, b in blocks)
        n = [front.token_count(torch.zeros(96, 96, 3)), front.token_count(torch.zeros(100, 200, 3))]
        assert [b - a for a, b in blocks] == n
        assert all(model.history[i] == 299 for a, b in blocks for i in range(a, b))
        assert model.history[blocks[0][0] - 1] != 299 and model.history[blocks[0][1]] != 299
    finally:
        srv.stop(); eng.shutdown()


def test_paged_kv_allocator_tables_exhaustion_and_reuse():
    import torch
    from r4dx_b200.models.batch import PagedKvAllocator
    al = PagedKvAllocator(num_blocks=6, slots=3, max_blocks_per_slot=4, device="cpu")
    al.ensure(0, 17)                       # 2 blocks of 16 tokens
    al.ensure(1, 40)                       # 3 blocks
    assert al.blocks_in_use() == 5
    t0, t1 = al.tables[0, :2].tolist(), al.tables[1, :3].tolist()
    assert len(set(t0 + t1)) == 5 and all(0 <= b < 6 for b in t0 + t1)
    al.ensure(0, 30)                       # still 2 blocks: nothing new
    assert al.blocks_in_use() == 5 and al.tables[0, :2].tolist() == t0
    with pytest.raises(MemoryError):
        al.ensure(2, 33)                   # needs 3, one is free; the failed call takes nothing
    assert al.blocks_in_use() == 5
    with pytest.raises(ValueError):
        al.ensure(0, 16 * 4 + 1)           # beyond the slot's table
    al.release(1)
    assert al.blocks_in_use() == 2
    al.ensure(2, 48)                       # the released blocks serve another slot
    assert set(al.tables[2, :3].tolist()) <= set(t1) | {b for b in range(6) if b not in t0 + t1}


def test_sampled_speculation_emits_the_same_stream_as_plain_sampled_decode():
    """Sample-and-match: with the same seed, the speculative engine path produces exactly the plain sampled stream,
    whatever the drafter proposes (an oracle-like drafter, a wrong one, none)."""
    def run(draft_fn, spec_k):
        model = FakeTextModel(vocab=64)
        model.draft_fn = draft_fn
        eng = Engine(model, ByteTokenizer(300))
        req = GenRequest(prompt_ids=[5, 9, 11], max_tokens=24, params=SampleParams(temperature=0.9, top_k=12, seed=7,
                                                                                  repetition_penalty=1.1), spec_k=spec_k)
        r = eng.generate(req, timeout=20)
        eng.shutdown()
        assert r.error is None, r.error
        return r.token_ids, model

    plain, _ = run(None, 0)

    def good(history, token, k):
        # proposes the plain stream's own continuation where it knows it (so drafts are accepted), junk elsewhere
        seq = [5, 9, 11] + plain
        i = len(history) + 1
        return [seq[j] if j < len(seq) else 1 for j in range(i, i + k)]

    def bad(history, token, k):
        return [63] * k

    for fn in (good, bad):
        toks, model = run(fn, 3)
        assert toks == plain, (fn.__name__, toks, plain)
        assert model.history[:3 + len(plain) - 1] == ([5, 9, 11] + plain)[:3 + len(plain) - 1]


def test_ngram_drafter_proposes_what_followed_the_latest_match_and_stays_lossless():
    from r4dx_b200.models.ngram import NgramDrafter, NgramIndex, simulate
    ix = NgramIndex(2, 3)
    ix.extend([1, 2, 3, 4, 5, 9, 1, 2, 3])
    assert ix.propose(3) == [4, 5, 9]                  # the earlier "1 2 3" was followed by 4 5 9
    ix.extend([7, 8, 2, 3])
    assert ix.propose(2) == [7, 8]                     # the LATEST earlier "2 3" wins
    assert NgramIndex(2, 3).propose(4) == []
    # drafter protocol: anchor fed by draft(), accepted drafts by after_verify()
    d = NgramDrafter(2, 4)
    d.after_prefill([5, 6, 7, 8, 5, 6], 7)
    assert d.draft(7, 3) == [8, 5, 6]
    d.after_verify(7, [8, 5, 6], [8, 5, 0])            # two accepted, then a correction
    assert d.index.tokens == [5, 6, 7, 8, 5, 6, 7, 8, 5]
    # a stream that repeats a 6-token phrase saves most of the target calls; a random one saves nothing
    rep = [3, 1, 4, 1, 5, 9] * 12
    s = simulate(rep, 12, k=4)
    assert s["calls_saved_frac"] > 0.6 and s["accepted_per_call"] > 2.0
    import random
    rnd = random.Random(0)
    noise = [rnd.randrange(50000) for _ in range(200)]
    assert simulate(noise, 20, k=4)["calls_saved_frac"] < 0.05
    # through the engine's sampled speculative path the stream equals plain sampled decode
    model = FakeTextModel(vocab=16)                    # a small vocabulary repeats itself: the drafter gets matches
    nd = NgramDrafter(1, 3)

    def draft_fn(history, token, k):
        ix2 = NgramIndex(1, 3)
        ix2.extend(history + [token])
        return ix2.propose(k)

    def run(fn):
        m = FakeTextModel(vocab=16)
        m.draft_fn = fn
        eng = Engine(m, ByteTokenizer(300))
        r = eng.generate(GenRequest(prompt_ids=[1, 2, 3, 1, 2], max_tokens=40, params=SampleParams(temperature=0.3, top_k=3, seed=3),
                                    spec_k=3 if fn else 0), timeout=20)
        eng.shutdown()
        assert r.error is None, r.error
        return r.token_ids, m.calls

    plain, calls_plain = run(None)
    spec, calls_spec = run(draft_fn)
    assert spec == plain and calls_spec <= calls_plain


def test_gemma_and_pythonic_tool_call_parsers_stream_and_degrade():
    import json
    from r4dx_b200.server.parsers import (GemmaToolCallParser, Lfm2ToolCallParser, QwenToolCallParser, detect_dialect,
                                          make_tool_call_parser)

    def run(p, text, step):
        out = ""
        for i in range(0, len(text), step):
            out += p.feed(text[i:i + step])
        return out + p.flush()

    for step in (1, 4, 1000):
        g = GemmaToolCallParser()
        out = run(g, 'Sure. <|tool_call>call:get_weather{city:<|"|>Paris <tool_call|> x<|"|>,days:3,opts:{metric:true,tags:[1,<|"|>a<|"|>,null]},'
                     'mode:fast}<tool_call|> done<|tool_call>call:b{}<tool_call|>', step)
        assert out == "Sure.  done" and not g.had_malformed_call
        assert [c["function"]["name"] for c in g.calls] == ["get_weather", "b"]
        assert json.loads(g.calls[0]["function"]["arguments"]) == {
            "city": "Paris <tool_call|> x", "days": 3, "opts": {"metric": True, "tags": [1, "a", None]}, "mode": "fast"}
        p = Lfm2ToolCallParser()
        out = run(p, "ok <|tool_call_start|>[get_w(city='Pa\\'ris <|tool_call_end|>', n=3, x=-1.5, f=True, "
                     'nested=[1, "two", true, null, {"k": "v\\u00e9"}],), mcp__srv__tool-1()]\n<|tool_call_end|> bye', step)
        assert out == "ok  bye" and not p.had_malformed_call
        assert json.loads(p.calls[0]["function"]["arguments"]) == {
            "city": "Pa'ris <|tool_call_end|>", "n": 3, "x": -1.5, "f": True, "nested": [1, "two", True, None, {"k": "v\u00e9"}]}
        assert p.calls[1]["function"] == {"name": "mcp__srv__tool-1", "arguments": "{}"}
    # malformed spans come back as literal content
    for bad in ("<|tool_call_start|>[f(1)]<|tool_call_end|>", "<|tool_call_start|>[]<|tool_call_end|>",
                "<|tool_call_start|>[f(a=word)]<|tool_call_end|>", '<|tool_call_start|>[{"name": "f", "arguments": {}}]<|tool_call_end|>'):
        p = Lfm2ToolCallParser()
        assert run(p, "a " + bad + " b", 3) == "a " + bad + " b" and p.had_malformed_call and not p.calls
    p = Lfm2ToolCallParser()
    assert run(p, "x <|tool_call_start|>[f(a='cut", 2) == "x <|tool_call_start|>[f(a='cut" and p.had_malformed_call
    g = GemmaToolCallParser()
    assert run(g, "<|tool_call>oops<tool_call|>", 2) == "<|tool_call>oops<tool_call|>" and g.had_malformed_call
    assert isinstance(make_tool_call_parser(detect_dialect("gemma-4-12b")), GemmaToolCallParser)
    assert isinstance(make_tool_call_parser(detect_dialect("LFM2.5-24B")), Lfm2ToolCallParser)
    assert isinstance(make_tool_call_parser(detect_dialect("qwen-hybrid")), QwenToolCallParser)


def test_audio_front_end_and_audio_parts_in_chat_requests():
    """WAV reader + framing + the encoder-free embedder against an fp32 restatement; then an ``input_audio`` part travels
    through the HTTP layer as placeholder tokens whose embeddings the engine overrides with the clip's rows."""
    import base64
    import math
    import torch
    from r4dx_b200.models import audio as A
    t = torch.arange(16000 // 2) / 16000.0
    wave = 0.4 * torch.sin(2 * math.pi * 330 * t)
    back, rate = A.read_wav(A.write_wav(wave))
    assert rate == 16000 and back.shape == wave.shape and float((back - wave).abs().max()) < 1e-4
    frames = A.frame_waveform(back)
    assert frames.shape == (13, 640) and float(frames[-1, 8000 - 12 * 640:].abs().max()) == 0.0      # zero-padded tail
    assert A.resample(wave, 16000, 8000).numel() == 4000
    W = torch.randn(128, 640, generator=torch.Generator().manual_seed(0)) * 0.05
    emb = A.AudioEmbedder(W)
    rows = emb.embed(frames)
    x = frames.to(torch.bfloat16).float()
    ref = (x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float() @ W.to(torch.bfloat16).float().T
    assert rows.dtype == torch.bfloat16 and torch.allclose(rows.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(emb.embed(frames[3:5]), rows[3:5])                     # a row depends on its own frame only
    with pytest.raises(ValueError):
        A.read_wav(b"not a wave file")
    with pytest.raises(ValueError):
        A.load_audio_embedder({})

    model = FakeTextModel(vocab=300)
    eng = Engine(model, ByteTokenizer(300), audio=emb)
    srv = ApiServer(eng, ByteTokenizer(300), ChatTemplate(), "fake-audio", port=0, audio_token_id=298)
    srv.start()
    try:
        clip = base64.b64encode(A.write_wav(wave)).decode()
        body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "transcribe "},
                                                           {"type": "input_audio", "input_audio": {"data": clip, "format": "wav"}}]}],
                "max_tokens": 3, "temperature": 0}
        r = json.load(_post(srv.port, "/v1/chat/completions", body))
        assert r["choices"][0]["finish_reason"] in ("stop", "length")
        pos, got = model.last_overrides
        assert pos.numel() == 13 and torch.equal(got, rows)
        assert all(model.history[int(p)] == 298 for p in pos) and model.history.count(298) == 13
        body["messages"][0]["content"][1]["input_audio"]["format"] = "mp3"
        with pytest.raises(urllib.error.HTTPError) as e:
            _post(srv.port, "/v1/chat/completions", body)
        assert e.value.code == 400
    finally:
        srv.stop(); eng.shutdown()
    # a server without the embedder refuses audio parts
    eng2 = Engine(FakeTextModel(vocab=300), ByteTokenizer(300))
    srv2 = ApiServer(eng2, ByteTokenizer(300), ChatTemplate(), "fake", port=0)
    srv2.start()
    try:
        body["messages"][0]["content"][1]["input_audio"]["format"] = "wav"
        with pytest.raises(urllib.error.HTTPError) as e:
            _post(srv2.port, "/v1/chat/completions", body)
        assert e.value.code == 400
    finally:
        srv2.stop(); eng2.shutdown()


def test_dialects_carry_reasoning_markers_tool_syntax_and_an_architecture_cross_check():
    from r4dx_b200.server.parsers import GemmaToolCallParser, ModelDialect, QwenToolCallParser, select_dialect
    d = select_dialect("auto", "gemma-4-12b-it", "gemma")
    assert d.name == "gemma" and isinstance(d.tool_call_parser(), GemmaToolCallParser) and d.cross_check("gemma") is None
    sp = d.reasoning_splitter()
    out = [sp.feed(x) for x in ("<|chan", "nel>thought\nlet me ", "think<chan", "nel|>The answer", " is 4")]
    c, r = sp.flush()
    assert "".join(o[0] for o in out) + c == "The answer is 4" and "".join(o[1] for o in out) + r == "let me think"
    q = select_dialect("auto", "some-qwen-hybrid", "qwen_hybrid")
    assert q.name == "qwen" and isinstance(q.tool_call_parser(), QwenToolCallParser)
    sp = q.reasoning_splitter(start_in_think=True)
    assert sp.feed("plan</think>\n\nhi") == ("hi", "plan")
    forced = select_dialect("lfm2", "some-qwen-hybrid", "qwen_hybrid")
    assert forced.name == "lfm2" and "qwen_hybrid" in forced.cross_check("qwen_hybrid")
    with pytest.raises(ValueError):
        ModelDialect("klingon")
    # the engine uses the forced dialect's tool syntax
    model = FakeTextModel(vocab=300)
    eng = Engine(model, ByteTokenizer(300))
    eng.dialect = "lfm2"
    r = eng.generate(GenRequest(prompt_ids=[1, 2, 3], max_tokens=4, params=SampleParams(temperature=0.0), parse_tools=True), timeout=20)
    eng.shutdown()
    assert r.error is None


def test_ngram_drafter_through_the_local_text_model_protocol():
    """LocalTextModel + NgramDrafter over a stand-in for the device model (a deterministic next-token rule that repeats
    itself): the speculative greedy stream equals the plain one and needs fewer target calls."""
    import torch
    from r4dx_b200.models.ngram import NgramDrafter
    from r4dx_b200.runtime.text_model import LocalTextModel

    class StubModel:
        """next token = (sum of the last two tokens) mod 7: periodic, so earlier n-grams predict the future"""
        max_ctx = 4096

        def __init__(self):
            self.hist, self.calls = [], 0
            self.cfg = type("C", (), {"tp_world": 1})()
            self.buf = type("B", (), {})()

        @property
        def pos(self):
            return len(self.hist)

        def _next(self, h):
            return (h[-1] + (h[-2] if len(h) > 1 else 0)) % 7

        def reset(self):
            self.hist = []

        def prefill(self, ids, chunk=None, hook=None, embed_overrides=None):
            self.calls += 1
            self.hist += [int(t) for t in ids.tolist()]
            return self._next(self.hist)

        def verify_window(self, anchor, drafts):
            self.calls += 1
            h = self.hist + [anchor]
            emitted = []
            for d in list(drafts) + [None]:
                t = self._next(h)
                emitted.append(t)
                if d is None or d != t:
                    break
                h.append(d)
            self.hist += [anchor] + emitted[:-1]
            return emitted

    def run(drafter, k):
        m = StubModel()
        tm = LocalTextModel(m, drafter=drafter)
        tok = tm.prefill([1, 2, 3, 5, 1])
        out = [tok]
        while len(out) < 40:
            out += tm.decode_step_spec_greedy(out[-1], k) if drafter is not None else [m.verify_window(out[-1], [])[0]]
        return out[:40], m.calls

    plain, calls_plain = run(None, 0)
    spec, calls_spec = run(NgramDrafter(2, 4), 4)
    assert spec == plain
    assert calls_spec < 0.6 * calls_plain, (calls_spec, calls_plain)


def test_batch_engine_samples_from_the_backends_logits_and_one_bad_request_fails_alone():
    """Sampling requests on the batch path: the draw comes from the request's own generator (a float, not the generator
    object), the first token is sampled too, the repetition penalty applies, and a slot whose handling raises is failed
    without taking the executor thread - and so every other request - down with it."""
    import torch
    from r4dx_b200.runtime.sampler import Rng, SampleParams, apply_repetition_penalty, sample_canonical
    from r4dx_b200.runtime.tokenizer import ByteTokenizer
    from r4dx_b200.server.batch_executor import BatchEngine, FakeBatchBackend
    from r4dx_b200.server.engine import GenRequest

    class LogitBackend(FakeBatchBackend):
        """Logits are a fixed function of the slot's history; the greedy pick is their argmax."""

        def _row(self, h):
            g = torch.Generator().manual_seed(sum((i + 1) * t for i, t in enumerate(h[-6:])) % 100003)
            return torch.randn(self.vocab, generator=g) * 2.0

        def import_slot(self, slot, ids):
            self.hist[slot] = list(ids)
            self.last_prefill_logits = self._row(self.hist[slot])
            return int(self.last_prefill_logits.argmax())

        def decode_batch(self, slots, tokens):
            rows = []
            for s, t in zip(slots, tokens):
                if t == 199:
                    raise_for = s          # noqa: F841  (kept for readability)
                self.hist[s].append(t)
                rows.append(self._row(self.hist[s]))
            self.last_logits = torch.stack(rows)
            return [int(r.argmax()) for r in rows]

    tk = ByteTokenizer()
    be = LogitBackend(slots=2, vocab=200)
    eng = BatchEngine(be, tk, max_queue=4, gather_ms=1.0)
    params = SampleParams(temperature=0.8, top_k=20, top_p=0.95, seed=1234, repetition_penalty=1.3)
    prompt = [5, 6, 7]
    res = eng.generate(GenRequest(prompt_ids=prompt, max_tokens=6, params=params), timeout=10)
    assert res.error is None and len(res.token_ids) == 6
    # replay on the host: same rows, same generator, same penalty
    rng, h, out = Rng(1234), list(prompt), []
    for _ in range(6):
        row = be._row(h).clone()
        apply_repetition_penalty(row, list(prompt) + out, 1.3)
        tok = sample_canonical(row, params, rng.next())
        out.append(tok)
        h.append(tok)
    assert res.token_ids == out
    # a request whose token handling raises (decoder blows up) ends with an error; the next request is served
    class Boom(Exception):
        pass
    orig = eng._consume
    def consume(a, tok, eos):
        if a.job.req.request_id == "bad":
            raise Boom("decoder failed")
        return orig(a, tok, eos)
    eng._consume = consume
    bad = eng.generate(GenRequest(prompt_ids=[1, 2], max_tokens=4, request_id="bad"), timeout=10)
    assert bad.finish_reason == "error" and "Boom" in (bad.error or "")
    good = eng.generate(GenRequest(prompt_ids=[3, 4], max_tokens=3), timeout=10)
    assert good.error is None and len(good.token_ids) == 3
    assert eng.worker.is_alive()
    eng.shutdown()


def test_speculation_is_cut_to_what_still_fits_when_a_request_runs_up_to_the_context_limit():
    """prompt + max_tokens == max_ctx with speculation on: the last rounds stage fewer draft rows (none at the very end),
    so the request finishes with every token instead of failing with a context overflow, and emits the plain stream."""
    def run(spec_k):
        model = FakeTextModel(vocab=64, max_ctx=3 + 20)
        model.draft_fn = (lambda history, token, k: [7] * k) if spec_k else None
        eng = Engine(model, ByteTokenizer(300))
        req = GenRequest(prompt_ids=[5, 9, 11], max_tokens=20, params=SampleParams(temperature=0.9, top_k=12, seed=3),
                         spec_k=spec_k)
        r = eng.generate(req, timeout=20)
        eng.shutdown()
        return r

    plain, spec = run(0), run(4)
    assert plain.error is None and spec.error is None, (plain.error, spec.error)
    assert len(spec.token_ids) == 20 and spec.token_ids == plain.token_ids
