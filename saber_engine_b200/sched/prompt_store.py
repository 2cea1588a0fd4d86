"""Prompt cache on a drive: prefixes that were prefilled once (system prompts, long documents)
survive an engine restart.  An entry is the same verified image a parked session uses (KV pages of
the prefix + the state slot at the cut); entries are found by the page-chain hash of their tokens
and checked by token equality, like the in-memory prefix cache.

Crash law: the image is written to a temporary name, fsynced, renamed, the directory fsynced, and
only then a checksummed record is appended to the index (and fsynced).  A crash at any point leaves
either no record or a complete file; at boot records whose file is missing or has another length are
dropped.

Parity: `crates/saber-mem/src/kv_ssd.rs:12-21` (tmp -> fsync -> rename -> dir fsync -> append
checksummed record), `crates/saber-cli/src/flashnext/pcache.rs:1-20`.
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
from typing import Optional

from .park import ParkError, ParkImage
from .prefix_cache import chain_hashes


class PromptStore:
    def __init__(self, directory: str, page: int = 16, min_tokens: int = 512):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.page, self.min_tokens = page, min_tokens
        self.index_path = self.dir / "index.jsonl"
        self.records: dict = {}            # key hex -> record
        self.counters = dict(puts=0, hits=0, misses=0, dropped_at_boot=0, corrupt=0)
        self.load()

    # ---- index
    @staticmethod
    def _line(rec: dict) -> str:
        body = json.dumps(rec, sort_keys=True)
        return json.dumps({"rec": rec, "sum": hashlib.sha256(body.encode()).hexdigest()}) + "\n"

    def load(self) -> None:
        self.records.clear()
        if not self.index_path.exists():
            return
        for raw in self.index_path.read_text().splitlines():
            try:
                obj = json.loads(raw)
                rec = obj["rec"]
                if hashlib.sha256(json.dumps(rec, sort_keys=True).encode()).hexdigest() != obj["sum"]:
                    raise ValueError("record checksum")
            except Exception:
                self.counters["dropped_at_boot"] += 1      # a torn last line
                continue
            f = self.dir / rec["file"]
            if not f.exists() or f.stat().st_size != rec["length"]:
                self.counters["dropped_at_boot"] += 1
                continue
            self.records[rec["key"]] = rec

    def _fsync_dir(self) -> None:
        fd = os.open(self.dir, os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)

    # ---- put / get
    def has(self, tokens, n_tokens: int) -> bool:
        return chain_hashes(tokens[:n_tokens], self.page)[-1].hex() in self.records

    def put(self, tokens, n_tokens: int, image: ParkImage) -> bool:
        if n_tokens < self.min_tokens or n_tokens % self.page:
            return False
        key = chain_hashes(tokens[:n_tokens], self.page)[-1].hex()
        if key in self.records:
            return False
        image.header["prompt_tokens"] = list(tokens[:n_tokens])
        raw = image.to_bytes()
        name = f"{key}.prompt"
        tmp = self.dir / f".{name}.tmp"
        with open(tmp, "wb") as fh:
            fh.write(raw)
            fh.flush()
            os.fsync(fh.fileno())
        os.rename(tmp, self.dir / name)
        self._fsync_dir()
        rec = {"key": key, "n_tokens": n_tokens, "file": name, "length": len(raw)}
        with open(self.index_path, "a") as fh:
            fh.write(self._line(rec))
            fh.flush()
            os.fsync(fh.fileno())
        self.records[key] = rec
        self.counters["puts"] += 1
        return True

    def get(self, tokens) -> Optional[ParkImage]:
        """The longest stored prefix that ends strictly before the last token, verified."""
        if len(tokens) < self.min_tokens or not self.records:
            self.counters["misses"] += 1
            return None
        hashes = chain_hashes(tokens[: len(tokens) - 1], self.page)
        for i in range(len(hashes) - 1, -1, -1):
            rec = self.records.get(hashes[i].hex())
            if rec is None:
                continue
            try:
                img = ParkImage.from_bytes((self.dir / rec["file"]).read_bytes())
                img.verify()
            except (ParkError, OSError):
                self.counters["corrupt"] += 1
                self.records.pop(rec["key"], None)
                continue
            if img.header.get("prompt_tokens") != list(tokens[: rec["n_tokens"]]):
                continue                                    # hash collision: ids decide
            self.counters["hits"] += 1
            return img
        self.counters["misses"] += 1
        return None
