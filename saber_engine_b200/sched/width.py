"""Verify-width policy: how many rows a sequence gets in a speculative decode step.

Parity: `crates/saber-sched/src/width.rs:9-30` (a batch -> width table, default `1:8,4:5`, rounded
up to a captured width) and the acceptance EMA of `crates/saber-model/src/draft.rs:302-307`.
On B200 a decode step is bound by weight bytes, not by rows, so the measured-best table keeps the
widest captured width at every batch size; the reference's table is kept as `WidthByBatch.reference()`.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class WidthByBatch:
    table: dict                      # min batch -> width
    captured: tuple = (1, 5, 8)

    @staticmethod
    def parse(spec: str, captured=(1, 5, 8)) -> "WidthByBatch":
        t = {}
        for part in spec.split(","):
            b, w = part.split(":")
            t[int(b)] = int(w)
        if 1 not in t:
            raise ValueError("width table needs an entry for batch 1")
        return WidthByBatch(t, tuple(sorted(captured)))

    @staticmethod
    def reference() -> "WidthByBatch":
        return WidthByBatch.parse("1:8,4:5", captured=(1, 5, 8))

    @staticmethod
    def b200(max_width: int = 8) -> "WidthByBatch":
        return WidthByBatch({1: max_width}, captured=tuple(sorted({1, 5, max_width})))

    def width_for(self, batch: int) -> int:
        want = 1
        for b in sorted(self.table):
            if batch >= b:
                want = self.table[b]
        for w in self.captured:               # round UP to a captured width
            if w >= want:
                return w
        return self.captured[-1]


@dataclass
class WidthEma:
    """Per-sequence EMA of accepted drafts; proposes the narrowest captured width that would have
    covered the recent acceptance (an opt-in policy, the table above is the default)."""
    alpha: float = 0.25
    value: float = 4.0

    def update(self, accepted: int) -> None:
        self.value = (1 - self.alpha) * self.value + self.alpha * accepted

    def width(self, captured) -> int:
        want = int(self.value + 1.5)
        for w in sorted(captured):
            if w >= want:
                return w
        return max(captured)
