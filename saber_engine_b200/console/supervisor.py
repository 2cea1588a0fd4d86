"""Engine supervisor: runs the engine as a child process, tracks its state, restarts it after a
crash, keeps the history of applied configs and rolls back a config that never reaches ready.

States: stopped -> loading -> ready -> draining -> stopping -> stopped, plus crashed (the child
died with any other code; restarted with back-off) and fatal-86 (the child obeyed the teardown law:
it reported `saber: FATAL rank R: reason` and exited 86; the reason is kept, the restart is the
supervisor's recovery).  Readiness is a probe the caller supplies (the served engine answers
`/health`; tests use a file).

Parity: `crates/saber-console/src/supervisor.rs:1-40` (state machine, auto-rollback of a config that
never reaches ready), `docs/CONSOLE.md:28-31,165-177` (config history + rollback).  The HTTP application, the `/v1` proxy, the usage
store and the audit log are in `app.py`, `proxy.py`, `usage.py` and `audit.py` of this package.
"""
from __future__ import annotations

import json
import subprocess
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Optional

EXIT_FATAL = 86
STATES = ("stopped", "loading", "ready", "draining", "stopping", "crashed", "fatal-86")


@dataclass
class ConfigRecord:
    version: int
    argv: list
    applied_at: float
    reached_ready: bool = False
    note: str = ""


@dataclass
class Supervisor:
    ready_probe: Callable[[], bool]
    ready_timeout_s: float = 120.0
    max_restarts: int = 3
    backoff_s: float = 0.5
    history_path: Optional[str] = None
    state: str = "stopped"
    history: list = field(default_factory=list)
    last_fatal: Optional[str] = None
    restarts: int = 0
    events: list = field(default_factory=list)
    _proc: Optional[subprocess.Popen] = None
    _lock: threading.Lock = field(default_factory=threading.Lock)

    # ------------------------------------------------------------------ helpers
    def _set(self, state: str, why: str = "") -> None:
        assert state in STATES
        self.state = state
        self.events.append((time.time(), state, why))

    def _save(self) -> None:
        if self.history_path:
            Path(self.history_path).write_text(json.dumps(
                [dict(version=c.version, argv=c.argv, applied_at=c.applied_at, reached_ready=c.reached_ready, note=c.note)
                 for c in self.history], indent=1))

    def _spawn(self, argv: list) -> None:
        self._proc = subprocess.Popen(argv, stderr=subprocess.PIPE, text=True)
        self._set("loading", " ".join(argv[:3]))

    def _wait_ready(self) -> bool:
        t0 = time.monotonic()
        while time.monotonic() - t0 < self.ready_timeout_s:
            if self._proc.poll() is not None:
                return False
            if self.ready_probe():
                self._set("ready")
                return True
            time.sleep(0.02)
        return False

    def _reap(self) -> int:
        """Classifies the child's exit; returns its code."""
        code = self._proc.wait()
        err = self._proc.stderr.read() if self._proc.stderr else ""
        if code == EXIT_FATAL:
            line = next((ln for ln in err.splitlines() if "saber: FATAL" in ln), f"exit {code}")
            self.last_fatal = line.strip()
            self._set("fatal-86", self.last_fatal)
        elif code != 0:
            self._set("crashed", f"exit {code}")
        else:
            self._set("stopped")
        return code

    # ------------------------------------------------------------------ API
    def apply(self, argv: list, note: str = "") -> bool:
        """Starts the engine with a new config.  If it never reaches ready the last config that did
        is started again (auto-rollback) and False is returned."""
        with self._lock:
            self.stop()
            rec = ConfigRecord(len(self.history) + 1, list(argv), time.time(), note=note)
            self.history.append(rec)
            self._spawn(argv)
            if self._wait_ready():
                rec.reached_ready = True
                self._save()
                return True
            self._kill()
            rec.note = (rec.note + " " if rec.note else "") + "never reached ready: rolled back"
            good = next((c for c in reversed(self.history[:-1]) if c.reached_ready), None)
            self._save()
            if good is not None:
                self._spawn(good.argv)
                self._wait_ready()
            return False

    def poll(self) -> str:
        """Call periodically: notices a dead child and restarts it (crashed and fatal-86 alike) with
        back-off, up to max_restarts in a row."""
        with self._lock:
            if self._proc is not None and self.state in ("ready", "loading") and self._proc.poll() is not None:
                self._reap()
                cur = next((c for c in reversed(self.history) if c.reached_ready), None)
                if cur is not None and self.restarts < self.max_restarts:
                    self.restarts += 1
                    time.sleep(self.backoff_s * self.restarts)
                    self._spawn(cur.argv)
                    if self._wait_ready():
                        self.restarts = 0
            return self.state

    def drain_and_stop(self, drained: Callable[[], bool], timeout_s: float = 30.0) -> None:
        with self._lock:
            if self._proc is None:
                return
            self._set("draining")
            t0 = time.monotonic()
            while not drained() and time.monotonic() - t0 < timeout_s:
                time.sleep(0.02)
            self.stop()

    def _kill(self) -> None:
        if self._proc is not None and self._proc.poll() is None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
                self._proc.wait()
        self._proc = None

    def stop(self) -> None:
        if self._proc is None:
            return
        self._set("stopping")
        self._kill()
        self._set("stopped")
