"""What the mirror writes and what the replay writes beside it: one JSON object per line.

A mirror log (`<dir>/<UTC date>.jsonl`) holds three kinds of line: `start` (one per mirror
process), `exchange` (one per recorded request, written when its response has ended) and `metrics`
(the upstream's serving counters, polled on a timer).  A replay file holds one `replay_meta` line
and one `answer` per replayed exchange.  Bytes are kept as text when they are UTF-8 and as hex when
they are not (a chunk boundary can split a multi-byte character, so this is decided per blob).

Parity: `crates/saber-shadow/src/record.rs:1-40`.
"""
from __future__ import annotations

import json
import os
import time
from typing import Iterator, Optional


def blob_of(data: bytes) -> dict:
    try:
        return {"text": data.decode("utf-8")}
    except UnicodeDecodeError:
        return {"hex": data.hex()}


def blob_bytes(blob: dict) -> bytes:
    return blob["text"].encode("utf-8") if "text" in blob else bytes.fromhex(blob["hex"])


class Fnv:
    """64-bit FNV-1a over a byte stream: the forwarded bytes and the received bytes are both hashed
    into the record, so a reader can prove the client got exactly what the upstream sent."""

    def __init__(self):
        self.h = 0xCBF29CE484222325

    def update(self, data: bytes) -> None:
        h = self.h
        for b in data:
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        self.h = h

    def hex(self) -> str:
        return f"{self.h:016x}"


def unix_ms() -> int:
    return int(time.time() * 1000)


def utc_date(ms: Optional[int] = None) -> str:
    return time.strftime("%Y-%m-%d", time.gmtime((ms if ms is not None else unix_ms()) / 1000))


def append_line(path: str, obj: dict) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "a", encoding="utf-8") as f:
        f.write(json.dumps(obj, separators=(",", ":")) + "\n")


def read_lines(path: str) -> Iterator[dict]:
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                yield json.loads(line)
            except json.JSONDecodeError:
                continue               # a torn last line is skipped


def response_body(resp: dict) -> bytes:
    return b"".join(blob_bytes(c["data"]) for c in resp.get("chunks", []))


def parse_response(resp: dict) -> dict:
    """The facts the reader compares, out of a recorded response (streamed or not): served or not,
    text, reasoning, tool calls, finish reasons, usage, token ids when the reply carried them."""
    body = response_body(resp)
    out = {"status": resp.get("status", 0), "complete": bool(resp.get("complete")), "error_event": False, "content": "",
           "reasoning": "", "tool_calls": [], "finish": [], "usage": None, "token_ids": None}
    def take(obj):
        if "error" in obj:
            out["error_event"] = True
        if obj.get("usage"):
            out["usage"] = obj["usage"]
        for ch in obj.get("choices") or []:
            d = ch.get("delta") or ch.get("message") or {}
            out["content"] += ch.get("text") or d.get("content") or ""
            out["reasoning"] += d.get("reasoning_content") or ""
            for tc in d.get("tool_calls") or []:
                out["tool_calls"].append(tc)
            if ch.get("finish_reason"):
                out["finish"].append(ch["finish_reason"])
            if ch.get("token_ids") is not None:
                out["token_ids"] = (out["token_ids"] or []) + list(ch["token_ids"])
    if body.lstrip().startswith(b"data:") or b"\ndata:" in body:
        for line in body.split(b"\n"):
            if line.startswith(b"data:"):
                data = line[5:].strip()
                if data and data != b"[DONE]":
                    try:
                        take(json.loads(data))
                    except (ValueError, TypeError):
                        pass
    else:
        try:
            take(json.loads(body))
        except (ValueError, TypeError):
            pass
    out["served"] = 200 <= out["status"] < 300 and out["complete"] and not out["error_event"] and "abort" not in out["finish"]
    return out
