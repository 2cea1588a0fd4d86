"""HostTrace: a fixed list of named host phases per engine step, off by default.

Off, a phase boundary costs one attribute load; on, two `perf_counter_ns()` reads and a list append.
A number taken with the trace on is an attribution, never a published step time.

Parity: `crates/saber-engine/src/host_trace.rs:1-30` (named phases Index / SeamIn / Lead / Paged /
SeamOut / Accept / Step / Idle, flag `--engine-host-trace`) and the nested startup-phase ledger of
`crates/saber-engine/src/startup.rs:1-25`.
"""
from __future__ import annotations

import json
import time
from collections import defaultdict
from contextlib import contextmanager

PHASES = ("Plan", "Index", "H2D", "Launch", "D2H", "Accept", "Sample", "Emit", "Idle")


class HostTrace:
    def __init__(self, enabled: bool = False, keep_steps: int = 4096):
        self.enabled = enabled
        self.keep_steps = keep_steps
        self.steps: list = []            # one dict phase -> ns per step
        self._cur: dict = {}

    @contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if name not in PHASES:
            raise KeyError(f"unknown host phase {name!r}: phases are declared up front ({PHASES})")
        t0 = time.perf_counter_ns()
        try:
            yield
        finally:
            self._cur[name] = self._cur.get(name, 0) + time.perf_counter_ns() - t0

    def end_step(self) -> None:
        if not self.enabled:
            return
        self.steps.append(self._cur)
        self._cur = {}
        if len(self.steps) > self.keep_steps:
            del self.steps[: len(self.steps) - self.keep_steps]

    def summary(self) -> dict:
        tot = defaultdict(int)
        for s in self.steps:
            for k, v in s.items():
                tot[k] += v
        n = max(1, len(self.steps))
        return {"steps": len(self.steps), "mean_us": {k: tot[k] / n / 1e3 for k in PHASES if k in tot}}


class StartupLedger:
    """Nested, named boot phases with wall time; printed by `saber serve` when it reaches ready."""

    def __init__(self):
        self.rows: list = []
        self._stack: list = []

    @contextmanager
    def phase(self, name: str):
        t0 = time.perf_counter()
        self._stack.append(name)
        path = "/".join(self._stack)
        try:
            yield
        finally:
            self._stack.pop()
            self.rows.append((path, time.perf_counter() - t0))

    def render(self) -> str:
        return "\n".join(f"  {p:40s} {s * 1e3:10.1f} ms" for p, s in sorted(self.rows))


class StepLedger:
    """Joins the scheduler's per-step timing with the executor's device span and (optionally) writes
    one JSON line per step.  Parity: `crates/saber-cli/src/flashnext/stepledger.rs:1-15`
    (`--fn-step-trace PATH`, `saber_fn_step_*` on /metrics)."""

    def __init__(self, path=None, keep: int = 1024):
        self.path, self.keep = path, keep
        self.rows: list = []
        self._fh = open(path, "a") if path else None

    def record(self, kind: str, live: int, host_s: float, device_ms=None, **extra) -> None:
        row = {"t": time.time(), "kind": kind, "live": live, "host_ms": host_s * 1e3, "device_ms": device_ms, **extra}
        self.rows.append(row)
        if len(self.rows) > self.keep:
            del self.rows[0]
        if self._fh:
            self._fh.write(json.dumps(row) + "\n")
            self._fh.flush()

    def percentiles(self, key: str = "host_ms") -> dict:
        v = sorted(r[key] for r in self.rows if r.get(key) is not None)
        if not v:
            return {}
        pick = lambda q: v[min(len(v) - 1, int(q * len(v)))]     # noqa: E731
        return {"p50": pick(0.5), "p90": pick(0.9), "p99": pick(0.99), "n": len(v)}

    def close(self) -> None:
        if self._fh:
            self._fh.close()
            self._fh = None
