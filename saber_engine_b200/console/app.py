"""The console's HTTP application: admin API over the supervisor (engine start / stop / restart, config
apply with auto-rollback, history and rollback), the audit log, the usage history, the `/v1/*`
reverse proxy, and one page of HTML that shows state, config history and usage.

    GET  /api/state                     supervisor state, last fatal reason, restarts
    POST /api/engine/start|stop|restart
    GET  /api/config/history            applied configs (argv, when, whether they reached ready)
    POST /api/config/apply              {"argv": [...], "note": "..."}  (auto-rollback when never ready)
    POST /api/config/rollback           {"version": N}   re-apply an earlier config
    GET  /api/usage/summary?hours=24&by=model|key ;  GET /api/usage/recent ;  GET /api/usage/metrics
    GET  /api/audit?n=100
    POST /api/keys  {"label": ...} -> the secret, once ;  DELETE /api/keys/{label}
    ANY  /v1/*                          proxied to the engine (console/proxy.py)

Every mutating admin call lands in the audit log with the caller's label.  With an admin token
configured the admin API wants it as a bearer; without one the console is open and is meant to be
bound to the loopback.

Parity: `crates/saber-console/src/http.rs` (routes), `history.rs` (config history + rollback),
`audit.rs`, `usage.rs`, `proxy.rs`, `docs/CONSOLE.md:28-31,165-177`.
"""
from __future__ import annotations

import contextlib
import html
import time
from typing import Optional

from starlette.applications import Starlette
from starlette.requests import Request
from starlette.responses import HTMLResponse, JSONResponse, PlainTextResponse
from starlette.routing import Route

from .audit import Audit
from .auth import KeyRing
from .proxy import Proxy
from .supervisor import Supervisor
from .usage import UsageStore


class Console:
    def __init__(self, supervisor: Supervisor, data_dir: str, engine_url: str, admin_token: Optional[str] = None,
                 engine_bearer: Optional[str] = None, usage: Optional[UsageStore] = None):
        self.sup, self.admin_token = supervisor, admin_token
        self.audit = Audit(data_dir)
        self.usage = usage if usage is not None else UsageStore(f"{data_dir}/usage.db")
        self.keys = KeyRing()
        self.proxy = Proxy(engine_url, self.usage, self.keys, admin_token, engine_bearer)

    # ---- helpers
    def _who(self, request: Request) -> Optional[str]:
        if not self.admin_token:
            return "local"
        auth = request.headers.get("authorization", "")
        return "admin" if auth == f"Bearer {self.admin_token}" else None

    def _audited(self, request: Request, who: str, action: str, status: int, detail: str = "") -> None:
        self.audit.log(who, action, f"{request.method} {request.url.path}", status,
                       request.client.host if request.client else None, detail)

    def _current_argv(self) -> Optional[list]:
        good = next((c for c in reversed(self.sup.history) if c.reached_ready), None)
        return list(good.argv) if good else None

    # ---- routes
    async def state(self, request: Request):
        if self._who(request) is None:
            return JSONResponse({"error": "admin token required"}, 401)
        return JSONResponse({"state": self.sup.poll(), "last_fatal": self.sup.last_fatal, "restarts": self.sup.restarts,
                             "events": [list(e) for e in self.sup.events[-20:]]})

    async def engine_action(self, request: Request):
        who = self._who(request)
        if who is None:
            return JSONResponse({"error": "admin token required"}, 401)
        action = request.path_params["action"]
        status, detail = 200, ""
        if action == "stop":
            self.sup.stop()
        elif action in ("start", "restart"):
            argv = self._current_argv()
            if argv is None:
                status, detail = 409, "no config has reached ready yet: apply one first"
            else:
                ok = self.sup.apply(argv, note=f"{action} by {who}")
                status, detail = (200, "") if ok else (502, "the engine never reached ready")
        else:
            status, detail = 404, "unknown action"
        self._audited(request, who, f"engine.{action}", status, detail)
        return JSONResponse({"state": self.sup.state, "detail": detail}, status)

    async def history(self, request: Request):
        if self._who(request) is None:
            return JSONResponse({"error": "admin token required"}, 401)
        return JSONResponse([dict(version=c.version, argv=c.argv, applied_at=c.applied_at, reached_ready=c.reached_ready,
                                  note=c.note) for c in self.sup.history])

    async def apply(self, request: Request):
        who = self._who(request)
        if who is None:
            return JSONResponse({"error": "admin token required"}, 401)
        body = await request.json()
        argv = body.get("argv")
        if not isinstance(argv, list) or not argv or not all(isinstance(a, str) for a in argv):
            self._audited(request, who, "config.apply", 400, "argv must be a non-empty list of strings")
            return JSONResponse({"error": "argv must be a non-empty list of strings"}, 400)
        ok = self.sup.apply(argv, note=str(body.get("note", "")))
        if not ok:
            self.audit.log("console", "config.auto_rollback", detail=f"version {len(self.sup.history)} never reached ready")
        self._audited(request, who, "config.apply", 200 if ok else 502, f"version {len(self.sup.history)}")
        return JSONResponse({"applied": ok, "version": len(self.sup.history), "state": self.sup.state}, 200 if ok else 502)

    async def rollback(self, request: Request):
        who = self._who(request)
        if who is None:
            return JSONResponse({"error": "admin token required"}, 401)
        body = await request.json()
        rec = next((c for c in self.sup.history if c.version == body.get("version")), None)
        if rec is None or not rec.reached_ready:
            self._audited(request, who, "config.rollback", 404, f"version {body.get('version')}")
            return JSONResponse({"error": "no such version that reached ready"}, 404)
        ok = self.sup.apply(rec.argv, note=f"rollback to version {rec.version}")
        self._audited(request, who, "config.rollback", 200 if ok else 502, f"to version {rec.version}")
        return JSONResponse({"applied": ok, "state": self.sup.state}, 200 if ok else 502)

    async def usage_summary(self, request: Request):
        if self._who(request) is None:
            return JSONResponse({"error": "admin token required"}, 401)
        hours = float(request.query_params.get("hours", "24"))
        by = request.query_params.get("by", "model")
        now = int(time.time() * 1000)
        grain = "m" if hours <= 2 else ("h" if hours <= 72 else "d")
        return JSONResponse(self.usage.summary(now - int(hours * 3_600_000), now + 1, grain, "key" if by == "key" else "model"))

    async def usage_recent(self, request: Request):
        if self._who(request) is None:
            return JSONResponse({"error": "admin token required"}, 401)
        return JSONResponse(self.usage.recent(int(request.query_params.get("n", "50"))))

    async def usage_metrics(self, request: Request):
        return PlainTextResponse(self.usage.prometheus(), media_type="text/plain; version=0.0.4")

    async def audit_tail(self, request: Request):
        if self._who(request) is None:
            return JSONResponse({"error": "admin token required"}, 401)
        return JSONResponse(self.audit.tail(int(request.query_params.get("n", "100"))))

    async def key_issue(self, request: Request):
        who = self._who(request)
        if who is None:
            return JSONResponse({"error": "admin token required"}, 401)
        label = str((await request.json()).get("label", "")).strip()
        try:
            if not label:
                raise ValueError("label is required")
            secret = self.keys.issue(label)
        except ValueError as exc:
            self._audited(request, who, "auth.key.issue", 400, str(exc))
            return JSONResponse({"error": str(exc)}, 400)
        self._audited(request, who, "auth.key.issue", 200, label)       # the label, never the secret
        return JSONResponse({"label": label, "key": secret})

    async def key_revoke(self, request: Request):
        who = self._who(request)
        if who is None:
            return JSONResponse({"error": "admin token required"}, 401)
        label = request.path_params["label"]
        ok = self.keys.revoke(label)
        self._audited(request, who, "auth.key.revoke", 200 if ok else 404, label)
        return JSONResponse({"revoked": ok}, 200 if ok else 404)

    async def page(self, request: Request):
        if self._who(request) is None:
            return HTMLResponse("<p>admin token required</p>", 401)
        rows = "".join(f"<tr><td>{c.version}</td><td>{html.escape(' '.join(c.argv))}</td><td>{'yes' if c.reached_ready else 'no'}</td>"
                       f"<td>{html.escape(c.note)}</td></tr>" for c in reversed(self.sup.history))
        now = int(time.time() * 1000)
        use = "".join(f"<tr><td>{html.escape(str(u['model']))}</td><td>{u['requests']}</td><td>{u['errors']}</td>"
                      f"<td>{u['prompt_tokens']}</td><td>{u['completion_tokens']}</td><td>{u['ttft_ms_p50']}</td></tr>"
                      for u in self.usage.summary(now - 86_400_000, now + 1, "h"))
        return HTMLResponse(
            f"<html><body><h1>saber console</h1><p>engine: <b>{self.sup.state}</b>"
            f"{' &mdash; ' + html.escape(self.sup.last_fatal) if self.sup.last_fatal else ''}</p>"
            f"<h2>config history</h2><table border=1><tr><th>v</th><th>argv</th><th>ready</th><th>note</th></tr>{rows}</table>"
            f"<h2>usage, last 24 h</h2><table border=1><tr><th>model</th><th>requests</th><th>errors</th><th>prompt tok</th>"
            f"<th>completion tok</th><th>TTFT p50 ms</th></tr>{use}</table></body></html>")

    async def v1(self, request: Request):
        return await self.proxy.handle(request)

    def app(self) -> Starlette:
        methods = ["GET", "POST", "PUT", "DELETE", "PATCH"]

        @contextlib.asynccontextmanager
        async def lifespan(app):
            yield
            await self.proxy.close()
        return Starlette(lifespan=lifespan, routes=[
            Route("/", self.page), Route("/api/state", self.state),
            Route("/api/engine/{action}", self.engine_action, methods=["POST"]),
            Route("/api/config/history", self.history), Route("/api/config/apply", self.apply, methods=["POST"]),
            Route("/api/config/rollback", self.rollback, methods=["POST"]),
            Route("/api/usage/summary", self.usage_summary), Route("/api/usage/recent", self.usage_recent),
            Route("/api/usage/metrics", self.usage_metrics), Route("/api/audit", self.audit_tail),
            Route("/api/keys", self.key_issue, methods=["POST"]), Route("/api/keys/{label}", self.key_revoke, methods=["DELETE"]),
            Route("/v1/{rest:path}", self.v1, methods=methods), Route("/health", self.v1), Route("/metrics", self.v1),
        ])
