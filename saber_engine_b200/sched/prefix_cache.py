"""Prefix cache for the hybrid model (default on): KV pages are kept alive in place by refcount and
the Gated DeltaNet recurrent state is snapshotted at cut points, so a later prompt that starts with
the same tokens skips that part of its prefill.

Parity: `crates/saber-sched/src/prefix_cache.rs:1-60`: block-chained keys plus full token-id
equality (a hash match alone is never trusted), the snapshot sits at a whole-block boundary strictly
before the prompt end (the last prompt token must still run to produce logits), LRU under a byte
budget, a minimum prompt length.  Differences: cut points are also taken every `interval` tokens so
prompts that share only a prefix of a cached prompt still hit, and snapshots live in device memory
(180 GB HBM3e) instead of host RAM.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Optional


def chain_hashes(tokens, page: int) -> list:
    """hash[i] covers tokens [0, (i + 1) * page)."""
    out, h = [], b"saber-prefix-v1"
    for i in range(len(tokens) // page):
        blk = tokens[i * page:(i + 1) * page]
        h = hashlib.blake2b(h + struct.pack(f"<{page}i", *blk), digest_size=16).digest()
        out.append(h)
    return out


@dataclass
class PrefixEntry:
    n_tokens: int
    tokens: tuple
    blocks: tuple             # physical KV blocks covering [0, n_tokens)
    snapshot: object          # executor-owned recurrent-state snapshot
    nbytes: int
    hits: int = 0


@dataclass
class PrefixCacheStats:
    lookups: int = 0
    hits: int = 0
    hit_tokens: int = 0
    inserts: int = 0
    evictions: int = 0
    refused_hash_collisions: int = 0


class PrefixCache:
    def __init__(self, kv_alloc, page: int = 16, budget_bytes: int = 6 << 30, min_tokens: int = 512,
                 interval: int = 1024, enabled: bool = True,
                 free_snapshot: Optional[Callable] = None):
        self.kv, self.page = kv_alloc, page
        self.budget, self.min_tokens, self.interval = budget_bytes, min_tokens, interval
        self.enabled = enabled
        self.free_snapshot = free_snapshot or (lambda s: None)
        self._entries: "OrderedDict[bytes, PrefixEntry]" = OrderedDict()
        self.bytes_used = 0
        self.stats = PrefixCacheStats()

    # ---- planning --------------------------------------------------------------------------
    def cut_points(self, n_prompt: int, start: int = 0) -> list:
        """Positions where a prefilling prompt should end a chunk and snapshot its state."""
        if not self.enabled or n_prompt < self.min_tokens:
            return []
        last = ((n_prompt - 1) // self.page) * self.page      # strictly before the prompt end
        cuts = set(range(self.interval, last + 1, self.interval))
        if last > 0:
            cuts.add(last)
        return sorted(c for c in cuts if c > start)

    # ---- lookup ----------------------------------------------------------------------------
    def lookup(self, tokens, count: bool = True) -> Optional[PrefixEntry]:
        """Longest cached prefix of `tokens` that ends strictly before the last token.  count=False
        is a peek: neither the statistics nor the LRU order change."""
        if not count:
            if not self.enabled or len(tokens) < self.min_tokens or not self._entries:
                return None
            hashes = chain_hashes(tokens[: len(tokens) - 1], self.page)
            for i in range(len(hashes) - 1, -1, -1):
                e = self._entries.get(hashes[i])
                if e is not None and e.tokens == tuple(tokens[: e.n_tokens]):
                    return e
            return None
        self.stats.lookups += 1
        if not self.enabled or len(tokens) < self.min_tokens or not self._entries:
            return None
        hashes = chain_hashes(tokens[: len(tokens) - 1], self.page)
        for i in range(len(hashes) - 1, -1, -1):
            e = self._entries.get(hashes[i])
            if e is None:
                continue
            if e.tokens != tuple(tokens[: e.n_tokens]):
                self.stats.refused_hash_collisions += 1
                continue
            self._entries.move_to_end(hashes[i])
            e.hits += 1
            self.stats.hits += 1
            self.stats.hit_tokens += e.n_tokens
            return e
        return None

    # ---- insert / evict --------------------------------------------------------------------
    def insert(self, tokens, n_tokens: int, blocks, snapshot, nbytes: int) -> bool:
        if not self.enabled or n_tokens % self.page or n_tokens <= 0:
            self.free_snapshot(snapshot)
            return False
        key = chain_hashes(tokens[:n_tokens], self.page)[-1]
        if key in self._entries:
            self._entries.move_to_end(key)
            self.free_snapshot(snapshot)
            return False
        while self.bytes_used + nbytes > self.budget and self._entries:
            self._evict_one()
        if self.bytes_used + nbytes > self.budget:
            self.free_snapshot(snapshot)
            return False
        blk = tuple(blocks[: n_tokens // self.page])
        self.kv.share(blk)                    # the cache is now an owner of these pages
        self._entries[key] = PrefixEntry(n_tokens, tuple(tokens[:n_tokens]), blk, snapshot, nbytes)
        self.bytes_used += nbytes
        self.stats.inserts += 1
        return True

    def _evict_one(self) -> None:
        _, e = self._entries.popitem(last=False)
        self.kv.release(e.blocks)
        self.free_snapshot(e.snapshot)
        self.bytes_used -= e.nbytes
        self.stats.evictions += 1

    def evict_for_blocks(self, need: int) -> None:
        """Give pages back to the allocator until `need` blocks are free (admission pressure)."""
        while self.kv.free_blocks < need and self._entries:
            self._evict_one()

    def clear(self) -> None:
        while self._entries:
            self._evict_one()

    def __len__(self) -> int:
        return len(self._entries)
