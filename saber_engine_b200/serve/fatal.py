"""Teardown law: a failed rank sets a process-wide fatal, every blocking wait observes it, queued and
in-flight requests get 503 with the reason, and the process exits 86 with
`saber: FATAL rank R: <reason>`; a watchdog forces the exit if teardown itself wedges.

Parity: `crates/saber-serve/src/fatal.rs:1-30` (fatal::set, exit code 86, --fatal-watchdog-s) and the
RankWatch that watches a child rank's exit and stderr (`README.md:602`).
"""
from __future__ import annotations

import os
import subprocess
import sys
import threading
import time
from typing import Callable, Optional

EXIT_FATAL = 86
_state = {"reason": None, "rank": None}
_lock = threading.Lock()
_event = threading.Event()
_hooks: list = []


def on_fatal(fn: Callable) -> None:
    _hooks.append(fn)


def set_fatal(rank: int, reason: str, exit_process: bool = True, watchdog_s: float = 10.0) -> None:
    with _lock:
        if _state["reason"] is not None:
            return
        _state.update(reason=reason, rank=rank)
    _event.set()
    msg = f"saber: FATAL rank {rank}: {reason}"
    print(msg, file=sys.stderr, flush=True)
    for fn in list(_hooks):
        try:
            fn(msg)
        except Exception:
            pass
    if exit_process:
        t = threading.Timer(watchdog_s, lambda: os._exit(EXIT_FATAL))
        t.daemon = True
        t.start()
        threading.Thread(target=lambda: (time.sleep(0.2), os._exit(EXIT_FATAL)), daemon=True).start()


def is_fatal() -> Optional[str]:
    return _state["reason"]


def wait_fatal(timeout: float) -> bool:
    return _event.wait(timeout)


def reset_for_tests() -> None:
    with _lock:
        _state.update(reason=None, rank=None)
    _event.clear()
    _hooks.clear()


class RankWatch:
    """Watches a child rank process: its exit (any code) or a FATAL line on stderr is fatal here."""

    def __init__(self, proc: subprocess.Popen, rank: int, on_death: Callable, tee=None):
        """tee: a text stream that gets every stderr line of the child (its log is not swallowed)."""
        self.proc, self.rank, self.on_death, self.tee = proc, rank, on_death, tee
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self) -> None:
        reason = None
        if self.proc.stderr is not None:
            for line in self.proc.stderr:
                line = line.decode(errors="replace") if isinstance(line, bytes) else line
                if self.tee is not None:
                    try:
                        self.tee.write(line)
                        self.tee.flush()
                    except (OSError, ValueError):
                        pass
                if "saber: FATAL" in line and reason is None:
                    reason = line.strip()
                    if self.tee is None:
                        break
        code = self.proc.wait()
        self.on_death(self.rank, reason or f"rank {self.rank} exited with code {code}")
