"""Prompt-lookup drafting: propose the continuation of the most recent earlier occurrence of the
current n-gram suffix.  Parity: `crates/saber-engine/src/lookup.rs:1-30` (a drafter that needs no
model; useful when the output repeats its context: code edits, counting, quoting)."""
from __future__ import annotations


def lookup_draft(history: list, k: int, max_ngram: int = 4, min_ngram: int = 1) -> list:
    n_hist = len(history)
    for n in range(min(max_ngram, n_hist - 1), min_ngram - 1, -1):
        suffix = history[n_hist - n:]
        for start in range(n_hist - n - 1, -1, -1):           # most recent earlier match first
            if history[start:start + n] == suffix:
                cont = history[start + n:start + n + k]
                if cont:
                    return cont + [0] * (k - len(cont))
    return [0] * k
