"""The console's `/v1/*` reverse proxy.

Every request is forwarded to the engine on the loopback; the response's chunks are passed to the
client AS THEY ARRIVE (a streamed reply's SSE events reach the client when the engine writes them).
On the way through the proxy watches the frames of `/v1/chat/completions` and `/v1/completions` to
record one usage row per request: TTFT at the first SSE event that carries a token, the `usage`
block's token counts, the finish reason, the status (499 when the client went away first).  The row
is queued to the usage store's writer thread, never written on the request path.  The engine request
carries `x-saber-console-ref: <the row's uid>`, which the engine keeps in its `/v1/requests` ring, so
the fallback poll merges the engine's view into the same row.

Auth: with proxy keys configured a client presents one of them (its label rides the row; a revoked
key is refused); otherwise the admin token when the console has one; otherwise the proxy is open.
Wrong keys count toward the address's lockout.  The engine sees the console's own engine key when one
is configured, else (open mode) the client's `Authorization` unchanged.

Parity: `crates/saber-console/src/proxy.rs:1-22`.
"""
from __future__ import annotations

import itertools
import json
import time
from typing import Optional

import aiohttp
from starlette.requests import Request
from starlette.responses import JSONResponse, Response, StreamingResponse

from .auth import KeyRing, Limiter
from .usage import SRC_PROXY, UsageRow, UsageStore

REF_HEADER = "x-saber-console-ref"
MAX_REQUEST_BYTES = 256 * 1024 * 1024
MAX_COPY = 8 * 1024 * 1024          # bytes of a non-streamed reply kept to read its usage block
MAX_LINE = 1024 * 1024              # a longer SSE line is passed through unparsed
RECORDED = ("/v1/chat/completions", "/v1/completions")
HOP_BY_HOP = {"connection", "keep-alive", "proxy-connection", "proxy-authenticate", "proxy-authorization", "te",
              "trailer", "transfer-encoding", "upgrade", "host", "content-length"}


class SseWatcher:
    """Reads the usage facts out of a reply as its bytes go by (never alters them)."""

    def __init__(self, t0: float, stream: bool):
        self.t0, self.stream = t0, stream
        self.ttft_ms: Optional[float] = None
        self.prompt_tokens = self.completion_tokens = 0
        self.finish, self.model = "", ""
        self._buf = b""
        self._copy = bytearray()

    def _event(self, obj: dict) -> None:
        self.model = obj.get("model", self.model) or self.model
        for ch in obj.get("choices") or []:
            delta = ch.get("delta") or {}
            has_tok = bool(ch.get("text") or delta.get("content") or delta.get("reasoning_content") or delta.get("tool_calls"))
            if has_tok and self.ttft_ms is None:
                self.ttft_ms = (time.monotonic() - self.t0) * 1000.0
            if ch.get("finish_reason"):
                self.finish = ch["finish_reason"]
        u = obj.get("usage")
        if isinstance(u, dict):
            self.prompt_tokens = int(u.get("prompt_tokens", self.prompt_tokens) or 0)
            self.completion_tokens = int(u.get("completion_tokens", self.completion_tokens) or 0)

    def feed(self, chunk: bytes) -> None:
        if not self.stream:
            if len(self._copy) < MAX_COPY:
                self._copy += chunk[:MAX_COPY - len(self._copy)]
            return
        self._buf += chunk
        while b"\n" in self._buf:
            line, self._buf = self._buf.split(b"\n", 1)
            if len(line) > MAX_LINE or not line.startswith(b"data:"):
                continue
            data = line[5:].strip()
            if data == b"[DONE]":
                continue
            try:
                self._event(json.loads(data))
            except (ValueError, TypeError):
                pass
        if len(self._buf) > MAX_LINE:
            self._buf = b""

    def end(self) -> None:
        if not self.stream and self._copy:
            try:
                obj = json.loads(bytes(self._copy))
                if self.ttft_ms is None and obj.get("choices"):
                    self.ttft_ms = (time.monotonic() - self.t0) * 1000.0
                self._event(obj)
            except (ValueError, TypeError):
                pass


class Proxy:
    def __init__(self, engine_url: str, usage: Optional[UsageStore] = None, keys: Optional[KeyRing] = None,
                 admin_token: Optional[str] = None, engine_bearer: Optional[str] = None, limiter: Optional[Limiter] = None):
        self.engine_url = engine_url.rstrip("/")
        self.usage, self.keys, self.admin_token, self.engine_bearer = usage, keys, admin_token, engine_bearer
        self.limiter = limiter or Limiter()
        self._seq = itertools.count(1)
        self._prefix = f"c{int(time.time() * 1000):x}"      # unique across console restarts
        self._session: Optional[aiohttp.ClientSession] = None

    def next_uid(self) -> str:
        return f"{self._prefix}-{next(self._seq)}"

    def caller(self, request: Request):
        """(label | None for open mode, refusal response | None)."""
        addr = request.client.host if request.client else "?"
        if self.limiter.locked(addr):
            return None, JSONResponse({"error": {"message": "too many failed attempts", "type": "authentication_error"}}, 429)
        auth = request.headers.get("authorization", "")
        token = auth[7:] if auth.lower().startswith("bearer ") else ""
        if self.keys is not None and self.keys.keys:
            label = self.keys.check(token) if token else None
            if label is None and self.admin_token and token == self.admin_token:
                label = "admin"
        elif self.admin_token:
            label = "admin" if token == self.admin_token else None
        else:
            return None, None                                  # open mode
        if label is None:
            self.limiter.fail(addr)
            return None, JSONResponse({"error": {"message": "invalid API key", "type": "authentication_error"}}, 401)
        self.limiter.ok(addr)
        return label, None

    async def _client(self) -> aiohttp.ClientSession:
        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None, sock_connect=10),
                                                  auto_decompress=False)
        return self._session

    async def close(self) -> None:
        if self._session is not None and not self._session.closed:
            await self._session.close()

    async def handle(self, request: Request) -> Response:
        label, refusal = self.caller(request)
        if refusal is not None:
            return refusal
        cl = request.headers.get("content-length")
        if cl and cl.isdigit() and int(cl) > MAX_REQUEST_BYTES:
            return JSONResponse({"error": {"message": "request body too large", "type": "invalid_request_error"}}, 413)
        body = await request.body()
        path = request.url.path
        recorded = request.method == "POST" and path in RECORDED
        uid = self.next_uid()
        headers = {k: v for k, v in request.headers.items() if k.lower() not in HOP_BY_HOP}
        headers[REF_HEADER] = uid
        if self.engine_bearer:
            headers["authorization"] = f"Bearer {self.engine_bearer}"
        elif label is not None:
            headers.pop("authorization", None)              # a console credential is not the engine's
        stream, model = False, ""
        if recorded:
            try:
                req_obj = json.loads(body)
                stream, model = bool(req_obj.get("stream")), str(req_obj.get("model") or "")
            except (ValueError, TypeError, AttributeError):
                pass
        t0 = time.monotonic()
        ts_ms = int(time.time() * 1000)
        url = self.engine_url + path + (("?" + request.url.query) if request.url.query else "")
        watcher = SseWatcher(t0, stream) if recorded else None
        session = await self._client()
        try:
            up = await session.request(request.method, url, data=body, headers=headers)
        except aiohttp.ClientError as exc:
            if recorded and self.usage:
                self.usage.record(UsageRow(uid, ts_ms, model, label or "", path, 502, stream=stream, src=SRC_PROXY,
                                           total_ms=(time.monotonic() - t0) * 1000.0, finish="upstream_unreachable"))
            return JSONResponse({"error": {"message": f"engine unreachable: {exc}", "type": "bad_gateway"}}, 502)

        state = {"done": False}

        def finish(status: int) -> None:
            if state["done"]:
                return
            state["done"] = True
            if watcher is not None:
                watcher.end()
                if self.usage:
                    self.usage.record(UsageRow(uid, ts_ms, watcher.model or model, label or "", path, status,
                                               watcher.prompt_tokens, watcher.completion_tokens, watcher.ttft_ms,
                                               (time.monotonic() - t0) * 1000.0, watcher.finish, stream, SRC_PROXY))

        async def chunks():
            try:
                async for chunk in up.content.iter_any():
                    if watcher is not None:
                        watcher.feed(chunk)
                    yield chunk
                finish(up.status)
            finally:
                up.release() if state["done"] else up.close()   # a client that left: the upstream stream is dropped with it
                finish(499)

        out_headers = {k: v for k, v in up.headers.items() if k.lower() not in HOP_BY_HOP}
        return StreamingResponse(chunks(), status_code=up.status, headers=out_headers)
