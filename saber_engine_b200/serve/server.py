"""OpenAI-compatible HTTP plane: /v1/chat/completions, /v1/completions, /v1/models, /health,
/metrics, /v1/stats, /v1/requests.  Streaming responses carry EXACTLY ONE SSE chunk per engine step
of the request (then a usage chunk when asked, then [DONE]).

Parity: `crates/saber-serve/src/server.rs:51-60` (the seven routes), `:1-10` (one chunk per step),
`reqcheck.rs:1-20` (request-shape validation answers 400 with every problem), `auth.rs` (API keys),
`requests.rs:1-12` (a ring of recent requests without bodies), `fatal.rs` (503 with the reason).
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from collections import deque
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .engine_api import EngineRefused, EngineRequest, SamplingParams
from .metrics import Metrics
from .parse import ReasoningParser, StopStrings, parse_tool_calls
from .tokenizer import ByteCodec, IncrementalDetok, normalise_messages, render_chat


def _err(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": message, "type": kind, "code": status}}, status_code=status)


def sampling_from_body(body: dict, default_max: int) -> SamplingParams:
    def num(k, d, cast=float):
        v = body.get(k, d)
        if v is None:
            return d
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ValueError(f"{k} must be a number")
        return cast(v)
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens"))
    lp = body.get("logprobs")
    top_lp = body.get("top_logprobs")
    if isinstance(lp, bool):
        lp = (top_lp or 0) if lp else None
    return SamplingParams(
        temperature=num("temperature", 1.0), top_p=num("top_p", 1.0), top_k=num("top_k", 0, int),
        min_p=num("min_p", 0.0), presence_penalty=num("presence_penalty", 0.0),
        frequency_penalty=num("frequency_penalty", 0.0), repetition_penalty=num("repetition_penalty", 1.0),
        seed=body.get("seed"), max_tokens=int(max_tokens) if max_tokens is not None else default_max,
        stop_token_ids=tuple(body.get("stop_token_ids") or ()), ignore_eos=bool(body.get("ignore_eos", False)),
        logprobs=lp, prompt_logprobs=body.get("prompt_logprobs"))


def _collect_images(msgs: list, have_vision: bool) -> list:
    """RGB arrays of every image part of a conversation, in order (`data:` URLs only).  Parity:
    `crates/saber-vision-input/src/url.rs`, `src/decode.rs`."""
    urls = []
    for m in msgs:
        if isinstance(m.get("content"), list):
            for part in m["content"]:
                if not isinstance(part, dict) or part.get("type") not in ("text", "image", "image_url"):
                    raise ValueError("content parts must be of type text or image_url")
                if part["type"] in ("image", "image_url"):
                    u = part.get("image_url")
                    u = u.get("url") if isinstance(u, dict) else (u or part.get("image"))
                    if not isinstance(u, str):
                        raise ValueError("image_url part needs a url")
                    urls.append(u)
    if urls and not have_vision:
        raise ValueError("this server was started without a vision tower: image parts are not accepted")
    if not urls:
        return []
    from ..vision import processor as VP
    return [VP.decode_image(VP.fetch_image_url(u)) for u in urls]


class ServerState:
    def __init__(self, engine, tokenizer=None, model_name: str = "saber", api_keys=(), chat_template=None,
                 default_max_tokens: int = 256, reasoning_parser: Optional[str] = "qwen3",
                 tool_parser: Optional[str] = "qwen3_coder", census_fn=None, vision=None):
        self.engine, self.tok = engine, tokenizer or ByteCodec()
        self.model_name, self.api_keys = model_name, set(api_keys)
        self.chat_template, self.default_max_tokens = chat_template, default_max_tokens
        self.reasoning_parser, self.tool_parser = reasoning_parser, tool_parser
        self.metrics = Metrics(model_name)
        self.requests = deque(maxlen=256)       # ring: no bodies are stored
        self.started = time.time()
        self.census_fn = census_fn
        self.vision = vision                     # vision.engine.VisionFrontend, or None: a text-only plane


def create_app(state: ServerState) -> FastAPI:
    app = FastAPI(title="saber-b200", docs_url=None, redoc_url=None)
    app.state.saber = state

    def authorised(request: Request) -> bool:
        if not state.api_keys:
            return True
        h = request.headers.get("authorization", "")
        return h.startswith("Bearer ") and h[7:] in state.api_keys

    def fatal_reason() -> Optional[str]:
        return getattr(state.engine, "fatal", None)

    @app.get("/health")
    async def health():
        if fatal_reason():
            return _err(503, f"engine is down: {fatal_reason()}", "service_unavailable")
        return PlainTextResponse("ok")

    @app.get("/v1/models")
    async def models(request: Request):
        if not authorised(request):
            return _err(401, "invalid API key", "authentication_error")
        m = state.engine.model()
        return {"object": "list", "data": [{"id": state.model_name, "object": "model", "created": int(state.started),
                                            "owned_by": "saber", "max_model_len": m.get("max_model_len")}]}

    @app.get("/metrics")
    async def metrics():
        census = state.census_fn() if state.census_fn else None
        return PlainTextResponse(state.metrics.render(state.engine.stats(), census),
                                 media_type="text/plain; version=0.0.4")

    @app.get("/v1/stats")
    async def stats(request: Request):
        if not authorised(request):
            return _err(401, "invalid API key", "authentication_error")
        s = dict(state.engine.stats())
        s["uptime_s"] = time.time() - state.started
        s["ttft_p50_s"] = state.metrics.h["time_to_first_token_seconds"].quantile(0.5)
        s["itl_p99_s"] = state.metrics.h["inter_token_latency_seconds"].quantile(0.99)
        return s

    @app.get("/v1/requests")
    async def requests_ring(request: Request):
        if not authorised(request):
            return _err(401, "invalid API key", "authentication_error")
        return {"object": "list", "data": list(state.requests)}

    async def run_request(request: Request, body: dict, chat: bool):
        if not authorised(request):
            return _err(401, "invalid API key", "authentication_error")
        if fatal_reason():
            return _err(503, f"engine is down: {fatal_reason()}", "service_unavailable")
        problems = []
        if body.get("model") not in (None, state.model_name):
            problems.append(f"model {body.get('model')!r} is not served (serving {state.model_name!r})")
        if body.get("n", 1) != 1:
            problems.append("n > 1 is not supported")
        try:
            params = sampling_from_body(body, state.default_max_tokens)
        except (ValueError, TypeError) as exc:
            problems.append(str(exc))
            params = SamplingParams()
        stops = body.get("stop") or []
        if isinstance(stops, str):
            stops = [stops]
        if not isinstance(stops, list) or not all(isinstance(s, str) for s in stops) or len(stops) > 4:
            problems.append("stop must be a string or a list of at most 4 strings")
            stops = []
        tools = body.get("tools") if chat else None
        starts_in_reasoning = False
        images = []
        try:
            if chat:
                msgs = normalise_messages(body.get("messages"))
                images = _collect_images(msgs, state.vision is not None)
                kw = body.get("chat_template_kwargs") or {}
                text = render_chat(msgs, state.chat_template, True, tools, **kw)
                starts_in_reasoning = text.rstrip().endswith("<think>")
                prompt_ids = state.tok.encode(text)
            else:
                p = body.get("prompt")
                if isinstance(p, list) and p and all(isinstance(x, int) for x in p):
                    prompt_ids = list(p)
                elif isinstance(p, str):
                    prompt_ids = state.tok.encode(p)
                else:
                    raise ValueError("prompt must be a string or a list of token ids")
        except ValueError as exc:
            problems.append(str(exc))
            prompt_ids = []
        if problems:
            return _err(400, "; ".join(problems))
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        ereq = None
        try:
            eos = getattr(state.tok, "eos_token_id", None)
            if images:      # tower forward into the image arena, placeholders -> arena rows, three-axis positions
                ereq = await asyncio.get_running_loop().run_in_executor(
                    None, lambda: state.vision.build_request(prompt_ids, images, params, request_id=rid, eos_token_id=eos))
                prompt_ids = ereq.prompt_token_ids
            else:
                ereq = EngineRequest(prompt_ids, params, rid, eos)
            sub = state.engine.submit(ereq)
        except ValueError as exc:             # an image the processor refuses (aspect ratio, placeholders)
            return _err(400, str(exc))
        except EngineRefused as exc:
            if ereq is not None and ereq.mm and callable(ereq.mm.get("release")):
                ereq.mm["release"]()
            state.metrics.inc("request_refused_total")
            return _err(exc.status, exc.reason, "service_unavailable" if exc.status == 503 else "invalid_request_error")
        loop = asyncio.get_running_loop()
        wake = asyncio.Event()
        sub.events.set_notifier(lambda: loop.call_soon_threadsafe(wake.set))
        t_submit = time.monotonic()
        created = int(time.time())
        rec = {"id": rid, "created": created, "prompt_tokens": len(prompt_ids), "completion_tokens": 0,
               "stream": bool(body.get("stream")), "status": "running", "kind": "chat" if chat else "completion"}
        if request.headers.get("x-saber-console-ref"):     # the console proxy's row id: its usage poll merges on it
            rec["client_ref"] = request.headers["x-saber-console-ref"][:64]
        state.requests.append(rec)
        detok = IncrementalDetok(state.tok, skip_ids=[getattr(state.tok, "eos_token_id", -1)])
        stopper = StopStrings(stops)
        reason = ReasoningParser(starts_in_reasoning) if (chat and state.reasoning_parser) else None

        async def events():
            """Yields (event, text_delta) once per engine step of this request."""
            t_last = None
            while True:
                ev = sub.events.get_nowait()
                if ev is None:
                    wake.clear()
                    ev = sub.events.get_nowait()
                    if ev is None:
                        try:
                            await asyncio.wait_for(wake.wait(), timeout=1.0)
                        except asyncio.TimeoutError:
                            if await request.is_disconnected():
                                state.engine.abort(sub.seq_id)
                        continue
                now = time.monotonic()
                if ev.first_token:
                    state.metrics.observe("time_to_first_token_seconds", now - t_submit)
                elif t_last is not None and ev.new_token_ids:
                    state.metrics.observe("inter_token_latency_seconds", (now - t_last) / max(1, len(ev.new_token_ids)))
                if ev.step_time_s:
                    state.metrics.observe("step_time_seconds", ev.step_time_s)
                t_last = now
                rec["completion_tokens"] += len(ev.new_token_ids)
                text = detok.push(ev.new_token_ids)
                if ev.finished:
                    text += detok.flush()
                text = stopper.push(text, final=ev.finished)
                if stopper.hit and not ev.finished:
                    state.engine.abort(sub.seq_id)
                    ev.finished, ev.finish_reason = True, "stop"
                yield ev, text
                if ev.finished:
                    rec["status"] = ev.finish_reason or "stop"
                    state.metrics.observe("e2e_request_latency_seconds", time.monotonic() - t_submit)
                    state.metrics.inc("request_success_total" if ev.finish_reason in ("stop", "length") else "request_refused_total")
                    return

        plp_items = []
        lp_items = []     # per generated token: {"token_id", "logprob", "top"} from the engine's candidate rows

        def lp_chat(items):
            def one(tid, lp):
                bs = state.tok.token_bytes(tid)
                return {"token": bs.decode("utf-8", errors="replace"), "logprob": lp, "bytes": list(bs)}
            return {"content": [{**one(it["token_id"], it["logprob"]),
                                 "top_logprobs": [one(i, v) for i, v in it["top"][: (params.logprobs or 0)]]} for it in items]}

        def lp_text(items):
            tk = lambda t: state.tok.token_bytes(t).decode("utf-8", errors="replace")   # noqa: E731
            return {"tokens": [tk(it["token_id"]) for it in items], "token_logprobs": [it["logprob"] for it in items],
                    "top_logprobs": [{tk(i): v for i, v in it["top"][: (params.logprobs or 0)]} for it in items]}

        def plp_vllm(items):
            """vLLM's shape: one entry per prompt token, None for the first, else {token id: {logprob, rank, decoded_token}}."""
            out = [None]
            for it in items:
                d = {}
                for rank, (i, v) in enumerate(it["top"], 1):
                    d[str(i)] = {"logprob": v, "rank": rank, "decoded_token": state.tok.token_bytes(i).decode("utf-8", errors="replace")}
                if str(it["token_id"]) not in d:
                    d[str(it["token_id"])] = {"logprob": it["logprob"], "rank": None,
                                              "decoded_token": state.tok.token_bytes(it["token_id"]).decode("utf-8", errors="replace")}
                out.append(d)
            return out

        def usage(ev):
            return {"prompt_tokens": len(prompt_ids), "completion_tokens": rec["completion_tokens"],
                    "total_tokens": len(prompt_ids) + rec["completion_tokens"],
                    "prompt_tokens_details": {"cached_tokens": ev.cached_tokens if ev else 0}}

        obj = "chat.completion" if chat else "text_completion"
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

            async def sse():
                last = None
                first = True
                async for ev, text in events():
                    last = ev
                    if ev.finish_reason == "error":
                        yield "data: " + json.dumps({"error": {"message": ev.error, "type": "service_unavailable", "code": 503}}) + "\n\n"
                        break
                    if chat:
                        delta = {}
                        if first:
                            delta["role"] = "assistant"
                        if reason is not None:
                            parts = reason.push(text, final=ev.finished)
                            if parts["reasoning"]:
                                delta["reasoning"] = parts["reasoning"]
                            delta["content"] = parts["content"]
                        else:
                            delta["content"] = text
                        choice = {"index": 0, "delta": delta, "finish_reason": ev.finish_reason if ev.finished else None}
                    else:
                        choice = {"index": 0, "text": text, "finish_reason": ev.finish_reason if ev.finished else None}
                    if ev.logprobs:
                        choice["logprobs"] = lp_chat(ev.logprobs) if chat else lp_text(ev.logprobs)
                    if ev.prompt_logprobs is not None:
                        choice["prompt_logprobs"] = plp_vllm(ev.prompt_logprobs)
                    first = False
                    yield "data: " + json.dumps({"id": rid, "object": obj + ".chunk" if chat else obj, "created": created,
                                                 "model": state.model_name, "choices": [choice]}) + "\n\n"
                if include_usage and last is not None and last.finish_reason != "error":
                    yield "data: " + json.dumps({"id": rid, "object": obj + ".chunk" if chat else obj, "created": created,
                                                 "model": state.model_name, "choices": [], "usage": usage(last)}) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        full, last = "", None
        async for ev, text in events():
            full += text
            last = ev
            if ev.logprobs:
                lp_items.extend(ev.logprobs)
            if ev.prompt_logprobs is not None:
                plp_items.extend(ev.prompt_logprobs)
        if last is not None and last.finish_reason == "error":
            return _err(503, last.error or "engine error", "service_unavailable")
        if chat:
            msg = {"role": "assistant"}
            content = full
            if reason is not None:
                parts = reason.push(full, final=True)
                content = parts["content"]
                if parts["reasoning"]:
                    msg["reasoning"] = parts["reasoning"]
            finish = last.finish_reason
            if tools and state.tool_parser:
                content, calls = parse_tool_calls(content, tools)
                if calls:
                    msg["tool_calls"] = calls
                    finish = "tool_calls"
            msg["content"] = content
            choice = {"index": 0, "message": msg, "finish_reason": finish}
        else:
            choice = {"index": 0, "text": full, "finish_reason": last.finish_reason}
        if params.logprobs is not None:
            choice["logprobs"] = lp_chat(lp_items) if chat else lp_text(lp_items)
        if params.prompt_logprobs is not None:
            choice["prompt_logprobs"] = plp_vllm(plp_items)
        return {"id": rid, "object": obj, "created": created, "model": state.model_name,
                "choices": [choice], "usage": usage(last)}

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        try:
            body = await request.json()
            assert isinstance(body, dict)
        except Exception:
            return _err(400, "request body must be a JSON object")
        return await run_request(request, body, chat=True)

    @app.post("/v1/completions")
    async def completions(request: Request):
        try:
            body = await request.json()
            assert isinstance(body, dict)
        except Exception:
            return _err(400, "request body must be a JSON object")
        return await run_request(request, body, chat=False)

    return app
