"""Bucket selection: the smallest planned shape that covers the live work; extra slots are padding.

Parity: `crates/saber-sched/src/buckets.rs:1-18` (smallest captured (batch, width) >= live) and the
prefill rung law of `crates/saber-sched/src/prefill_law.rs` (smallest planned rung >= rows, prompts
cut at the largest rung).
"""
from __future__ import annotations

from dataclasses import dataclass

DEFAULT_DECODE_BATCHES = (1, 2, 3, 4, 8)
DEFAULT_PREFILL_RUNGS = (96, 128, 192, 256, 320, 384, 512, 768, 1024, 1536, 2048)


class NoBucket(Exception):
    pass


def select_batch(live: int, batches=DEFAULT_DECODE_BATCHES) -> int:
    for b in sorted(batches):
        if b >= live:
            return b
    raise NoBucket(f"{live} live sequences exceed the largest captured batch {max(batches)}")


def select_rung(rows: int, rungs=DEFAULT_PREFILL_RUNGS) -> int:
    for r in sorted(rungs):
        if r >= rows:
            return r
    return max(rungs)


def cut_prompt(n_tokens: int, start: int, rungs=DEFAULT_PREFILL_RUNGS, cuts=()) -> list:
    """Chunk boundaries for prompt tokens [start, n_tokens): at most the largest rung per chunk and
    additionally cut at every position in `cuts` (prefix-cache snapshot points)."""
    out, pos, top = [], start, max(rungs)
    marks = sorted(c for c in cuts if start < c < n_tokens) + [n_tokens]
    for m in marks:
        while pos < m:
            n = min(top, m - pos)
            out.append((pos, n))
            pos += n
    return out
