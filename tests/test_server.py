"""HTTP plane over the scheduler + device mock: real ASGI app, streaming and non-streaming."""
import json

import pytest
from starlette.testclient import TestClient

from saber_engine_b200.sched.mock import NullExecutor, reference_generation
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve.parse import ReasoningParser, StopStrings, parse_tool_calls
from saber_engine_b200.serve.server import ServerState, create_app
from saber_engine_b200.serve.tokenizer import ByteCodec, IncrementalDetok, render_chat


class CountingEngine:
    """Wraps the scheduler and counts the events each request was sent (= engine steps it took)."""

    def __init__(self, inner):
        self.inner, self.events = inner, {}

    def submit(self, req):
        sub = self.inner.submit(req)
        put = sub.events.put
        def counted(ev, sid=sub.seq_id):
            self.events[sid] = self.events.get(sid, 0) + 1
            put(ev)
        # the scheduler holds the same StepStream object: patch its put
        sub.events.put = counted
        self.last = sub.seq_id
        return sub

    def __getattr__(self, k):
        return getattr(self.inner, k)


@pytest.fixture()
def client():
    sched = Scheduler(NullExecutor(seed=2, vocab=300), SchedulerConfig(max_seqs=8, max_ctx=4096, model_name="mock"))
    sched.spawn_step_loop()
    eng = CountingEngine(sched)
    app = create_app(ServerState(eng, ByteCodec(300), model_name="mock", api_keys=["sk-test"]))
    c = TestClient(app)
    c.headers.update({"Authorization": "Bearer sk-test"})
    c.engine = eng
    yield c
    sched.shutdown()


def test_models_health_auth(client):
    assert client.get("/health").text == "ok"
    assert client.get("/v1/models").json()["data"][0]["id"] == "mock"
    assert client.get("/v1/models", headers={"Authorization": "Bearer nope"}).status_code == 401


def test_completion_matches_engine_ids(client):
    prompt = [1, 2, 3, 4, 5]
    r = client.post("/v1/completions", json={"model": "mock", "prompt": prompt, "max_tokens": 10, "temperature": 0,
                                               "ignore_eos": True})
    assert r.status_code == 200
    body = r.json()
    want = ByteCodec(300).decode(reference_generation(prompt, 10, 300))
    assert body["choices"][0]["text"] == want
    assert body["usage"] == {"prompt_tokens": 5, "completion_tokens": 10, "total_tokens": 15,
                             "prompt_tokens_details": {"cached_tokens": 0}}
    assert body["choices"][0]["finish_reason"] == "length"


def test_stream_has_exactly_one_chunk_per_engine_step(client):
    with client.stream("POST", "/v1/chat/completions", json={
            "messages": [{"role": "user", "content": "hello"}], "max_tokens": 24, "temperature": 0, "ignore_eos": True,
            "stream": True, "stream_options": {"include_usage": True}}) as r:
        assert r.status_code == 200
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    usage = chunks[-1]
    assert usage["choices"] == [] and usage["usage"]["completion_tokens"] == 24
    content_chunks = chunks[:-1]
    assert len(content_chunks) == client.engine.events[client.engine.last]
    assert content_chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert content_chunks[-1]["choices"][0]["finish_reason"] == "length"
    assert len(content_chunks) < 24          # speculation: several tokens per step, still one chunk each


def test_request_validation_lists_every_problem(client):
    r = client.post("/v1/chat/completions", json={"model": "other", "messages": [], "n": 2, "temperature": "hot"})
    assert r.status_code == 400
    msg = r.json()["error"]["message"]
    assert "not served" in msg and "n > 1" in msg and "temperature" in msg and "messages" in msg
    assert client.post("/v1/completions", json={"prompt": "x", "max_tokens": 100000}).status_code == 400
    assert client.post("/v1/completions", content=b"not json").status_code == 400


def test_metrics_stats_requests(client):
    client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5, "temperature": 0, "ignore_eos": True})
    m = client.get("/metrics").text
    for fam in ("saber:num_requests_running", "saber:prompt_tokens_total", "saber:generation_tokens_total",
                "saber:time_to_first_token_seconds_bucket", "saber:inter_token_latency_seconds_count",
                "saber:spec_decode_num_draft_tokens_total", "saber:request_success_total",
                'engine="0",model_name="mock"'):
        assert fam in m, fam
    s = client.get("/v1/stats").json()
    assert s["generation_tokens"] >= 5 and "ttft_p50_s" in s
    ring = client.get("/v1/requests").json()["data"]
    assert ring and "prompt" not in ring[-1] and ring[-1]["status"] == "length"


def test_fatal_turns_into_503(client):
    client.engine.inner.set_fatal("rank 1 exited with code 86")
    r = client.post("/v1/completions", json={"prompt": "abc"})
    assert r.status_code == 503 and "rank 1" in r.json()["error"]["message"]
    assert client.get("/health").status_code == 503


def test_parsers_and_detok():
    p = ReasoningParser()
    out = [p.push(t) for t in ["<thi", "nk>plan", " it</th", "ink>\nThe ", "answer"]]
    assert "".join(o["reasoning"] for o in out) == "plan it"
    assert "".join(o["content"] for o in out) == "The answer"
    assert ReasoningParser().push("plain text", final=True)["content"] == "plain text"
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}}}}]
    text = "ok <tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>"
    content, calls = parse_tool_calls(text, tools)
    assert content == "ok" and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris", "days": 3}
    st = StopStrings(["END"])
    assert st.push("abcE") == "abc" and st.push("ND tail") == "" and st.hit
    tok = ByteCodec()
    d = IncrementalDetok(tok)
    ids = tok.encode("héllo")
    assert d.push(ids[:2]) == "h" and d.push(ids[2:]) == "éllo"       # never splits a UTF-8 sequence
    assert "<|im_start|>user\nhi<|im_end|>" in render_chat([{"role": "user", "content": "hi"}])


def test_chat_request_with_an_image_part_reaches_the_engine_with_image_rows():
    """An image_url part (data URL) goes through the processor and the request builder: placeholders
    become rows of the image arena, three-axis positions ride with the request, the rows are freed
    when the request ends; a server without a tower answers 400."""
    import base64
    import io
    from types import SimpleNamespace

    import numpy as np
    import torch
    from PIL import Image

    from saber_engine_b200.vision import processor as VP
    from saber_engine_b200.vision.engine import VisionFrontend
    tok = ByteCodec(300)
    ex = NullExecutor(seed=2, vocab=1000)
    ex.model = SimpleNamespace(cfg=SimpleNamespace(vocab=300), image_rows=128, stream=None,
                               embed_table=torch.zeros(428, 8, dtype=torch.bfloat16))
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096, model_name="mock"))
    sched.spawn_step_loop()
    seen = []
    sub0 = sched.submit
    sched.submit = lambda req: (seen.append(req), sub0(req))[1]
    vis = VisionFrontend(ex, SimpleNamespace(max_patches=512), tok.special_ids["<|image_pad|>"],
                         VP.ProcessorConfig(min_pixels=0), encode=lambda px, grids, rows: rows.fill_(0.5))
    img = (np.arange(64 * 64 * 3) % 255).astype(np.uint8).reshape(64, 64, 3)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    body = {"model": "mock", "max_tokens": 5, "messages": [{"role": "user", "content": [
        {"type": "text", "text": "what is this?"}, {"type": "image_url", "image_url": {"url": url}}]}]}
    try:
        c = TestClient(create_app(ServerState(sched, tok, model_name="mock", vision=vis)))
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        req = seen[-1]
        rows = [t for t in req.prompt_token_ids if t >= 300]
        assert rows == list(range(300, 304)) and req.mm["grids"] == [(1, 4, 4)]      # 64 x 64 -> 16 patches -> 4 tokens
        assert r.json()["usage"]["prompt_tokens"] == len(req.prompt_token_ids)
        assert vis.arena.free_rows == 128 and vis.counters["images"] == 1
        c2 = TestClient(create_app(ServerState(sched, tok, model_name="mock")))
        r2 = c2.post("/v1/chat/completions", json=body)
        assert r2.status_code == 400 and "vision" in r2.json()["error"]["message"]
        body["messages"][0]["content"][1]["image_url"]["url"] = "https://example.com/cat.png"
        assert c.post("/v1/chat/completions", json=body).status_code == 400
    finally:
        sched.shutdown()


def test_logprobs_come_from_the_engine_candidate_rows(client):
    body = {"model": "mock", "prompt": "abc", "max_tokens": 6, "temperature": 0, "logprobs": 3}
    r = client.post("/v1/completions", json=body).json()
    lp = r["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == 6 and len(lp["token_logprobs"]) == 6 and all(1 <= len(t) <= 3 for t in lp["top_logprobs"])   # (byte tokens that are not text alone share one key)
    import math
    want = -math.log(sum(math.exp(-i) for i in range(8)))         # the mock's pick sits at logit 0
    assert all(abs(x - want) < 1e-6 for x in lp["token_logprobs"])
    chat = {"model": "mock", "max_tokens": 4, "temperature": 0, "logprobs": True, "top_logprobs": 2,
            "messages": [{"role": "user", "content": "hi"}]}
    c = client.post("/v1/chat/completions", json=chat).json()["choices"][0]["logprobs"]["content"]
    assert len(c) == 4 and all(len(x["top_logprobs"]) == 2 and x["top_logprobs"][0]["logprob"] == x["logprob"] for x in c)
    # streaming: every chunk carries the entries of its own tokens
    n = 0
    with client.stream("POST", "/v1/completions", json={**body, "stream": True}) as s:
        for line in s.iter_lines():
            if line.startswith("data: {"):
                ch = json.loads(line[6:])["choices"]
                if ch and ch[0].get("logprobs"):
                    n += len(ch[0]["logprobs"]["tokens"])
    assert n == 6
    # without the field nothing is attached (and the engine is not asked for candidate rows)
    assert "logprobs" not in client.post("/v1/completions", json={"model": "mock", "prompt": "abc", "max_tokens": 2}).json()["choices"][0]


def test_prompt_logprobs_cover_every_prompt_token_but_the_first(client):
    body = {"model": "mock", "prompt": [5, 6, 7, 8, 9, 10, 11], "max_tokens": 2, "prompt_logprobs": 2}
    ch = client.post("/v1/completions", json=body).json()["choices"][0]
    plp = ch["prompt_logprobs"]
    assert len(plp) == 7 and plp[0] is None
    for tok, entry in zip(body["prompt"][1:], plp[1:]):
        assert str(tok) in entry and entry[str(tok)]["logprob"] == -1.0 - (tok % 7) * 0.125 and len(entry) == 2
    # a long prompt is prefilled in chunks: the entries of all chunks arrive together with the first token
    long = {"model": "mock", "prompt": [(i * 7) % 250 for i in range(700)], "max_tokens": 1, "prompt_logprobs": 0}
    plp = client.post("/v1/completions", json=long).json()["choices"][0]["prompt_logprobs"]
    assert len(plp) == 700 and plp[0] is None and all(len(e) == 1 for e in plp[1:])
