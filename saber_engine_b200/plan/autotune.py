"""Autotune table and sweeper: measured kernel-variant selection keyed on (op, shape incl. M, dtype,
device, kernel build hash).

Parity: `crates/saber-plan/src/autotune.rs:28-50` (key fields), `:562-720` (warm-up discard, medians,
ties go to the reference variant, two-pass disagreement = unstable), `crates/saber-exec/src/tune.rs:14-40`
(the sweep enumerates legal variants and times them INTERLEAVED so drift hits all variants alike).
There is no cost model: a route that was not measured falls back to the declared default, loudly
(`lookup` returns None and the caller counts a "default used" event).
"""
from __future__ import annotations

import hashlib
import json
import statistics
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Optional


def build_hash() -> str:
    """Hash of the native library binary: a table measured on another build does not apply."""
    from .. import build as b
    p = b.lib_path()
    if not p.exists():
        return "nobuild"
    return hashlib.sha256(p.read_bytes()).hexdigest()[:16]


def make_key(op: str, **shape) -> str:
    return op + "|" + ",".join(f"{k}={shape[k]}" for k in sorted(shape))


@dataclass
class TuneRecord:
    key: str
    variant: dict
    measured_us: float
    runner_up_us: Optional[float] = None
    samples: int = 0
    stable: bool = True


@dataclass
class TuneTable:
    device: str = "unknown"
    build: str = "nobuild"
    records: dict = field(default_factory=dict)
    defaults_used: int = 0

    def lookup(self, op: str, **shape) -> Optional[dict]:
        r = self.records.get(make_key(op, **shape))
        if r is None:
            self.defaults_used += 1
            return None
        return r.variant

    def put(self, rec: TuneRecord) -> None:
        self.records[rec.key] = rec

    def to_json(self) -> str:
        return json.dumps({"device": self.device, "build": self.build,
                           "records": [vars(r) for r in self.records.values()]}, indent=1)

    def save(self, path) -> None:
        Path(path).write_text(self.to_json())

    @staticmethod
    def load(path, check_build: bool = False) -> "TuneTable":
        d = json.loads(Path(path).read_text())
        t = TuneTable(d.get("device", "unknown"), d.get("build", "nobuild"))
        for r in d.get("records", []):
            t.put(TuneRecord(**r))
        if check_build and t.build != build_hash():
            raise ValueError(f"autotune table {path} was measured on build {t.build}, not {build_hash()}")
        return t


def choose(samples: dict, reference: str, tie_rel: float = 0.01):
    """samples: variant name -> list of times. The first sample of each variant is a warm-up and is
    discarded; medians are compared; a winner within `tie_rel` of the reference variant loses to it."""
    med = {k: statistics.median(v[1:] if len(v) > 1 else v) for k, v in samples.items()}
    best = min(med, key=med.get)
    if reference in med and med[reference] <= med[best] * (1.0 + tie_rel):
        best = reference
    others = sorted(v for k, v in med.items() if k != best)
    return best, med[best], (others[0] if others else None)


class Sweeper:
    """Times candidate variants interleaved. `make_runner(variant)` returns a zero-arg callable that
    enqueues one launch on the current stream; timing is by CUDA events."""

    def __init__(self, warmup: int = 2, samples: int = 9, passes: int = 2, batch: int = 8):
        # `batch` launches are enqueued back to back between the two events of one sample, so that
        # the host's per-launch overhead does not sit inside the measured interval
        self.warmup, self.samples, self.passes, self.batch = warmup, samples, passes, batch

    def time_variants(self, runners: dict) -> dict:
        import torch
        out = {k: [] for k in runners}
        for _ in range(self.warmup):
            for r in runners.values():
                r()
        torch.cuda.synchronize()
        for _ in range(self.samples + 1):
            for k, r in runners.items():       # interleaved: one sample of each variant per round
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                r()                              # absorbs the host gap after the previous sync
                e0.record()
                for _ in range(self.batch):
                    r()
                e1.record()
                e1.synchronize()
                out[k].append(e0.elapsed_time(e1) * 1e3 / self.batch)
        return out

    def sweep(self, key: str, variants: dict, make_runner: Callable, reference: str) -> TuneRecord:
        runners = {name: make_runner(v) for name, v in variants.items()}
        winners = []
        last = None
        for _ in range(self.passes):
            samples = self.time_variants(runners)
            best, us, second = choose(samples, reference)
            winners.append(best)
            last = (best, us, second, samples)
        best, us, second, samples = last
        stable = len(set(winners)) == 1
        if not stable:
            best = reference if reference in variants else best
            us = statistics.median(samples[best][1:])
        return TuneRecord(key, dict(variants[best], name=best), us, second, self.samples, stable)
