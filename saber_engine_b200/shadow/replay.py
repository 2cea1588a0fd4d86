"""The replay: the recorded requests sent to a Saber endpoint, byte for byte, with the answers
stored beside them.  The body is the recorded body unchanged (same messages, tools, sampling
parameters, seed), and so are the headers the record kept.  Two paces: `recorded` (each exchange at
its recorded arrival offset divided by `speed`, concurrency uncapped) and `sequential` (one at a
time in recorded order; deterministic, for a gate).  The target's `/metrics` is scraped before and
after the whole replay so the reader can check the census without a person looking at a log.

Parity: `crates/saber-shadow/src/replay.rs:1-20`.
"""
from __future__ import annotations

import asyncio
import time
from typing import Optional

import aiohttp

from .record import append_line, blob_bytes, blob_of, read_lines, unix_ms


def parse_metrics(text: str) -> dict:
    out = {}
    for line in text.splitlines():
        if not line or line.startswith("#"):
            continue
        name, _, val = line.rpartition(" ")
        try:
            out[name.strip()] = float(val)
        except ValueError:
            continue
    return out


async def _scrape(session: aiohttp.ClientSession, target: str, bearer: Optional[str]) -> Optional[dict]:
    try:
        async with session.get(target + "/metrics", headers={"authorization": f"Bearer {bearer}"} if bearer else {}) as r:
            return parse_metrics(await r.text()) if r.status == 200 else None
    except aiohttp.ClientError:
        return None


async def _one(session, target, ex, bearer, out_path, t_base):
    headers = dict(ex.get("headers") or {})
    if bearer:
        headers["authorization"] = f"Bearer {bearer}"
    t0 = time.monotonic()
    ans = {"kind": "answer", "id": ex["id"], "sent_at_ms": int((t0 - t_base) * 1000),
           "response": {"status": 0, "chunks": [], "complete": False}}
    try:
        async with session.post(target + ex["path"], data=blob_bytes(ex["request"]), headers=headers) as r:
            ans["response"]["status"] = r.status
            async for chunk in r.content.iter_any():
                if "first_byte_ms" not in ans:
                    ans["first_byte_ms"] = int((time.monotonic() - t0) * 1000)
                ans["response"]["chunks"].append({"at_ms": int((time.monotonic() - t0) * 1000), "data": blob_of(chunk)})
            ans["response"]["complete"] = True
    except aiohttp.ClientError as exc:
        ans["error"] = str(exc)
    ans["total_ms"] = int((time.monotonic() - t0) * 1000)
    append_line(out_path, ans)
    return ans


async def replay(log_path: str, target: str, out_path: str, pace: str = "sequential", speed: float = 1.0,
                 bearer: Optional[str] = None) -> dict:
    target = target.rstrip("/")
    exchanges = [e for e in read_lines(log_path) if e.get("kind") == "exchange"]
    exchanges.sort(key=lambda e: e.get("offset_ms", 0))
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None, sock_connect=10)) as session:
        before = await _scrape(session, target, bearer)
        append_line(out_path, {"kind": "replay_meta", "ts_ms": unix_ms(), "target": target, "source": log_path, "pace": pace,
                               "speed": speed, "exchanges": len(exchanges), "metrics_before": before})
        t_base = time.monotonic()
        if pace == "sequential":
            for ex in exchanges:
                await _one(session, target, ex, bearer, out_path, t_base)
        else:
            first = exchanges[0].get("offset_ms", 0) if exchanges else 0
            async def timed(ex):
                due = (ex.get("offset_ms", 0) - first) / 1000.0 / max(speed, 1e-6)
                await asyncio.sleep(max(0.0, due - (time.monotonic() - t_base)))
                return await _one(session, target, ex, bearer, out_path, t_base)
            await asyncio.gather(*(timed(ex) for ex in exchanges))
        after = await _scrape(session, target, bearer)
        append_line(out_path, {"kind": "replay_end", "ts_ms": unix_ms(), "metrics_after": after,
                               "wall_s": time.monotonic() - t_base})
    return {"exchanges": len(exchanges), "out": out_path}
