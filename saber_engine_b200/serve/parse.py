"""Output parsers: the `reasoning` split (qwen3: text inside <think>...</think>) and the qwen3_coder
tool-call format.  Both are streaming: they take text deltas and return typed deltas.

Parity: `crates/saber-serve/src/parse/mod.rs` (parsers qwen3 / qwen3_coder, selected per request).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Optional


class ReasoningParser:
    """Routes text into `reasoning` until </think>, then into `content`. A response that starts
    without <think> is content from the first character."""
    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, starts_in_reasoning: bool = False):
        self.in_reasoning = starts_in_reasoning
        self.decided = starts_in_reasoning
        self._buf = ""

    def push(self, text: str, final: bool = False) -> dict:
        self._buf += text
        out = {"reasoning": "", "content": ""}
        while self._buf:
            if not self.decided:
                s = self._buf.lstrip()
                if s.startswith(self.OPEN):
                    self._buf = s[len(self.OPEN):]
                    self.in_reasoning = self.decided = True
                    continue
                if self.OPEN.startswith(s) and not final:
                    break                              # could still become <think>
                self.decided = True
                continue
            if self.in_reasoning:
                k = self._buf.find(self.CLOSE)
                if k >= 0:
                    out["reasoning"] += self._buf[:k]
                    self._buf = self._buf[k + len(self.CLOSE):].lstrip("\n")
                    self.in_reasoning = False
                    continue
                hold = _partial_suffix(self._buf, self.CLOSE) if not final else 0
                out["reasoning"] += self._buf[: len(self._buf) - hold]
                self._buf = self._buf[len(self._buf) - hold:]
                break
            out["content"] += self._buf
            self._buf = ""
        return out


def _partial_suffix(text: str, marker: str) -> int:
    for n in range(min(len(marker) - 1, len(text)), 0, -1):
        if marker.startswith(text[-n:]):
            return n
    return 0


_TOOL_RE = re.compile(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def _coerce(value: str, schema: Optional[dict]):
    t = (schema or {}).get("type")
    v = value.strip()
    try:
        if t in ("integer", "int"):
            return int(v)
        if t in ("number", "float"):
            return float(v)
        if t == "boolean":
            return v.lower() == "true"
        if t in ("object", "array"):
            return json.loads(v)
    except (ValueError, json.JSONDecodeError):
        return value
    if t is None:
        try:
            return json.loads(v)
        except json.JSONDecodeError:
            return value
    return value


def parse_tool_calls(text: str, tools: Optional[list] = None):
    """qwen3_coder: <tool_call><function=NAME><parameter=K>V</parameter>...</function></tool_call>.
    Returns (content without the calls, [OpenAI tool_call dicts])."""
    schemas = {}
    for t in tools or []:
        fn = t.get("function", {})
        schemas[fn.get("name")] = (fn.get("parameters") or {}).get("properties", {})
    calls = []
    for m in _TOOL_RE.finditer(text):
        name, body = m.group(1), m.group(2)
        args = {k: _coerce(v, schemas.get(name, {}).get(k)) for k, v in _PARAM_RE.findall(body)}
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": json.dumps(args)}})
    return _TOOL_RE.sub("", text).strip(), calls


class StopStrings:
    """Stop sequences on text: holds back a tail that could still become a stop string."""

    def __init__(self, stops):
        self.stops = [s for s in (stops or []) if s]
        self._held = ""
        self.hit = False

    def push(self, text: str, final: bool = False) -> str:
        if not self.stops:
            return text
        self._held += text
        for s in self.stops:
            k = self._held.find(s)
            if k >= 0:
                self.hit = True
                out, self._held = self._held[:k], ""
                return out
        hold = 0 if final else max(_partial_suffix(self._held, s) for s in self.stops)
        out = self._held[: len(self._held) - hold]
        self._held = self._held[len(self._held) - hold:]
        return out
