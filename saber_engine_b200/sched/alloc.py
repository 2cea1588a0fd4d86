"""The two admission allocators: paged KV blocks and GDN state slots.

Parity: `crates/saber-sched/src/alloc.rs:7-24,77-250,256` (blocks for prompt + max_tokens are taken
up front together with one recurrent-state slot; both free lists hand out the LOWEST free index so
runs are reproducible; block 0 and slot 0 are the null block / null slot that padding rows use),
and the refcounts that let the prefix cache keep pages alive (`prefix_cache.rs:20-27`).
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field


class OutOfBlocks(Exception):
    pass


class PagedKvAllocator:
    def __init__(self, n_blocks: int, page_tokens: int = 16):
        assert n_blocks >= 2
        self.n_blocks, self.page = n_blocks, page_tokens
        self._free = list(range(1, n_blocks))       # block 0 is the null block
        heapq.heapify(self._free)
        self._ref = [0] * n_blocks

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.page - 1) // self.page

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> list:
        if n > len(self._free):
            raise OutOfBlocks(f"need {n} blocks, {len(self._free)} free")
        out = [heapq.heappop(self._free) for _ in range(n)]
        for b in out:
            self._ref[b] = 1
        return out

    def share(self, blocks) -> None:
        """Another owner (a sequence reusing cached prefix pages, or the cache itself)."""
        for b in blocks:
            assert self._ref[b] > 0, f"block {b} is not live"
            self._ref[b] += 1

    def release(self, blocks) -> None:
        for b in blocks:
            assert self._ref[b] > 0, f"double free of block {b}"
            self._ref[b] -= 1
            if self._ref[b] == 0:
                heapq.heappush(self._free, b)

    def refcount(self, b: int) -> int:
        return self._ref[b]


class GdnStateAllocator:
    """Recurrent-state slot sets: one slot per running sequence, slot 0 reserved (null)."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(1, n_slots))
        heapq.heapify(self._free)

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfBlocks("no free GDN state slot")
        return heapq.heappop(self._free)

    def release(self, slot: int) -> None:
        assert 1 <= slot < self.n_slots and slot not in self._free
        heapq.heappush(self._free, slot)


@dataclass
class Arenas:
    """Both allocators behind one admission call (all or nothing)."""
    kv: PagedKvAllocator
    gdn: GdnStateAllocator

    def can_admit(self, tokens: int, shared_blocks: int = 0) -> bool:
        return self.gdn.free_slots > 0 and self.kv.can_allocate(max(0, self.kv.blocks_for(tokens) - shared_blocks))

    def admit(self, tokens: int, shared: list = ()) -> tuple:
        """Returns (blocks, slot). `shared` are cached prefix blocks reused in place."""
        need = max(0, self.kv.blocks_for(tokens) - len(shared))
        if self.gdn.free_slots == 0 or not self.kv.can_allocate(need):
            raise OutOfBlocks("admission refused")
        self.kv.share(shared)
        blocks = list(shared) + self.kv.allocate(need)
        return blocks, self.gdn.allocate()

    def release(self, blocks, slot: int) -> None:
        self.kv.release(blocks)
        self.gdn.release(slot)
