"""The recording mirror: a reverse proxy that forwards every request to the upstream byte for byte
and, for the two generation routes, records the exchange on the side.

* transparent: the request body is forwarded unchanged, status and headers are forwarded (hop-by-hop
  headers excepted), a streamed body is forwarded chunk by chunk AS EACH CHUNK ARRIVES and copied on
  the side; the bytes forwarded and the bytes received are both hashed into the record;
* a failure to log never fails the client: records go to a writer thread over a queue, a write
  error is counted on `/shadow/health` and nothing else happens;
* a client that leaves is a client that left: the upstream stream is dropped with it;
* `/shadow/health` is the mirror's own, answered without touching the upstream.

Recorded: `POST /v1/chat/completions` and `POST /v1/completions`; everything else is forwarded only.

Parity: `crates/saber-shadow/src/mirror.rs:1-20`.
"""
from __future__ import annotations

import contextlib
import itertools
import queue
import threading
import time
from typing import Optional

import aiohttp
from starlette.applications import Starlette
from starlette.requests import Request
from starlette.responses import JSONResponse, StreamingResponse
from starlette.routing import Route

from .record import Fnv, append_line, blob_of, unix_ms, utc_date

RECORDED = ("/v1/chat/completions", "/v1/completions")
HOP_BY_HOP = {"connection", "keep-alive", "proxy-connection", "proxy-authenticate", "proxy-authorization", "te", "trailer",
              "transfer-encoding", "upgrade", "host", "content-length"}
KEPT_REQUEST_HEADERS = ("content-type", "accept", "user-agent", "x-request-id")


class Mirror:
    def __init__(self, upstream: str, log_dir: str):
        self.upstream, self.log_dir = upstream.rstrip("/"), log_dir
        self._ids = itertools.count(1)
        self._boot = f"{unix_ms():x}"
        self.recorded = self.forwarded = self.write_errors = 0
        self._q: "queue.Queue[Optional[dict]]" = queue.Queue()
        self._idle = threading.Event()
        self._idle.set()
        self._session: Optional[aiohttp.ClientSession] = None
        self._t0 = time.monotonic()
        self._writer = threading.Thread(target=self._write_loop, daemon=True)
        self._writer.start()
        self._log({"kind": "start", "ts_ms": unix_ms(), "upstream": self.upstream, "boot": self._boot})

    def log_path(self, ms: Optional[int] = None) -> str:
        return f"{self.log_dir}/{utc_date(ms)}.jsonl"

    def _log(self, obj: dict) -> None:
        self._idle.clear()
        self._q.put(obj)

    def _write_loop(self) -> None:
        while True:
            obj = self._q.get()
            if obj is None:
                return
            try:
                append_line(self.log_path(obj.get("ts_ms")), obj)
            except OSError:
                self.write_errors += 1
            if self._q.empty():
                self._idle.set()

    def flush(self, timeout: float = 5.0) -> bool:
        return self._idle.wait(timeout)

    def close(self) -> None:
        self._q.put(None)
        self._writer.join(timeout=5)

    async def health(self, request: Request):
        return JSONResponse({"ok": True, "recorded": self.recorded, "forwarded": self.forwarded,
                             "write_errors": self.write_errors, "upstream": self.upstream})

    async def handle(self, request: Request):
        body = await request.body()
        path = request.url.path
        record = request.method == "POST" and path in RECORDED
        headers = {k: v for k, v in request.headers.items() if k.lower() not in HOP_BY_HOP}
        url = self.upstream + path + (("?" + request.url.query) if request.url.query else "")
        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None, sock_connect=10), auto_decompress=False)
        t0, ts = time.monotonic(), unix_ms()
        try:
            up = await self._session.request(request.method, url, data=body, headers=headers)
        except aiohttp.ClientError as exc:
            return JSONResponse({"error": {"message": f"upstream unreachable: {exc}", "type": "bad_gateway"}}, 502)
        self.forwarded += 1
        ex = None
        if record:
            ex = {"kind": "exchange", "id": f"{self._boot}-{next(self._ids)}", "ts_ms": ts, "offset_ms": int((t0 - self._t0) * 1000),
                  "method": request.method, "path": path,
                  "headers": {k: request.headers[k] for k in KEPT_REQUEST_HEADERS if k in request.headers},
                  "request": blob_of(body),
                  "response": {"status": up.status, "headers": {k: v for k, v in up.headers.items() if k.lower() == "content-type"},
                               "chunks": [], "complete": False}}
        rx, tx = Fnv(), Fnv()
        done = {"v": False}

        def finish(complete: bool) -> None:
            if done["v"]:
                return
            done["v"] = True
            if ex is not None:
                ex["response"].update(complete=complete, rx_fnv=rx.hex(), tx_fnv=tx.hex(), total_ms=int((time.monotonic() - t0) * 1000))
                self.recorded += 1
                self._log(ex)

        async def chunks():
            try:
                async for chunk in up.content.iter_any():
                    rx.update(chunk)
                    if ex is not None:
                        ex["response"]["chunks"].append({"at_ms": int((time.monotonic() - t0) * 1000), "data": blob_of(chunk)})
                    yield chunk
                    tx.update(chunk)
                finish(True)
            finally:
                up.release() if done["v"] else up.close()
                finish(False)

        out_headers = {k: v for k, v in up.headers.items() if k.lower() not in HOP_BY_HOP}
        return StreamingResponse(chunks(), status_code=up.status, headers=out_headers)

    def app(self) -> Starlette:
        @contextlib.asynccontextmanager
        async def lifespan(app):
            yield
            if self._session is not None and not self._session.closed:
                await self._session.close()
        return Starlette(lifespan=lifespan, routes=[Route("/shadow/health", self.health),
                                                    Route("/{rest:path}", self.handle, methods=["GET", "POST", "PUT", "DELETE", "PATCH"])])
