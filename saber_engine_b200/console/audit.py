"""The console's audit log: every mutating admin call (config saves and applies, rollbacks, engine
start / stop / restart, key changes) and the console's own actions (auto-rollback), one JSON line
each in `<data dir>/audit.jsonl`, owner-only (0600).  `who` is the credential's LABEL (`admin`,
`local` for an open loopback console, `console` for its own actions), never a secret.  Past
MAX_LINES the file is cut to its newer half.

Parity: `crates/saber-console/src/audit.rs:1-50`.
"""
from __future__ import annotations

import json
import os
import threading
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Optional

MAX_LINES = 20_000


@dataclass
class AuditEntry:
    ts_ms: int
    who: str
    action: str                 # engine.start, config.apply, auth.key.revoke, ...
    route: str = ""             # POST /api/engine/start
    status: int = 0             # the reply's status; 0 for an action the console took itself
    ip: Optional[str] = None
    detail: str = ""


class Audit:
    def __init__(self, data_dir: str, max_lines: int = MAX_LINES):
        self.path = Path(data_dir) / "audit.jsonl"
        self.max_lines = max_lines
        self._lock = threading.Lock()
        self._lines = None

    def log(self, who: str, action: str, route: str = "", status: int = 0, ip: Optional[str] = None, detail: str = "") -> AuditEntry:
        e = AuditEntry(int(time.time() * 1000), who, action, route, status, ip, detail)
        line = json.dumps({k: v for k, v in asdict(e).items() if v not in (None, "")})
        with self._lock:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            fd = os.open(self.path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o600)
            try:
                os.write(fd, (line + "\n").encode())
            finally:
                os.close(fd)
            if self._lines is None:
                self._lines = sum(1 for _ in open(self.path, "rb"))
            else:
                self._lines += 1
            if self._lines > self.max_lines:
                self._cut()
        return e

    def _cut(self) -> None:
        lines = self.path.read_text().splitlines()
        keep = lines[len(lines) // 2:]
        tmp = self.path.with_suffix(".tmp")
        fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
        try:
            os.write(fd, ("\n".join(keep) + "\n").encode())
        finally:
            os.close(fd)
        os.replace(tmp, self.path)
        self._lines = len(keep)

    def tail(self, n: int = 100) -> list:
        if not self.path.exists():
            return []
        out = []
        for line in self.path.read_text().splitlines()[-n:]:
            try:
                out.append(json.loads(line))
            except json.JSONDecodeError:
                continue           # a torn last line (crash in mid-write) is skipped, not fatal
        return out
