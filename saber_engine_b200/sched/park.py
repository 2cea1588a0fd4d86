"""Session parking: a live sequence's KV pages and recurrent-state slot leave the device as ONE
image (layout header + payload, sha256 per 4 MiB chunk), first into pinned host memory, then --
when the RAM tier is over budget -- to a file; a restore verifies every chunk before anything
reaches device memory and resumes byte-identically.

Parity: `crates/saber-mem/src/park.rs:1-35`, `crates/saber-engine/src/park.rs:1-30`,
`crates/saber-sched/src/park.rs:1-20`; crash law of the drive tier (tmp -> fsync -> rename -> dir
fsync) as in `crates/saber-mem/src/kv_ssd.rs:12-21`.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

CHUNK = 4 << 20
MAGIC = b"SBRPARK1"


class ParkError(Exception):
    pass


@dataclass
class ParkImage:
    header: dict                    # layout: tensors [(name, dtype, shape, offset, nbytes)], tokens, pos, ...
    payload: bytes
    digests: list = field(default_factory=list)

    @staticmethod
    def build(header: dict, payload: bytes) -> "ParkImage":
        dig = [hashlib.sha256(payload[i:i + CHUNK]).hexdigest() for i in range(0, max(1, len(payload)), CHUNK)]
        return ParkImage(header, payload, dig)

    def verify(self) -> None:
        want = [hashlib.sha256(self.payload[i:i + CHUNK]).hexdigest() for i in range(0, max(1, len(self.payload)), CHUNK)]
        if want != self.digests:
            bad = [i for i, (a, b) in enumerate(zip(want, self.digests)) if a != b]
            raise ParkError(f"parked image is corrupt: chunk(s) {bad or 'count'} fail their sha256")

    def to_bytes(self) -> bytes:
        head = json.dumps({"header": self.header, "digests": self.digests, "length": len(self.payload)}).encode()
        return MAGIC + struct.pack("<Q", len(head)) + head + self.payload

    @staticmethod
    def from_bytes(raw: bytes) -> "ParkImage":
        if raw[:8] != MAGIC:
            raise ParkError("not a parked-session image")
        (n,) = struct.unpack("<Q", raw[8:16])
        meta = json.loads(raw[16:16 + n])
        payload = raw[16 + n:]
        if len(payload) != meta["length"]:
            raise ParkError(f"parked image is truncated: {len(payload)} of {meta['length']} bytes")
        return ParkImage(meta["header"], payload, meta["digests"])


class ParkTier:
    """RAM tier (budgeted) backed by a directory tier."""

    def __init__(self, ram_budget: int = 8 << 30, directory: Optional[str] = None):
        self.ram_budget = ram_budget
        self.dir = Path(directory) if directory else None
        if self.dir:
            self.dir.mkdir(parents=True, exist_ok=True)
        self.ram: dict = {}                 # key -> ParkImage (insertion order = age)
        self.ram_bytes = 0
        self.counters = dict(parked=0, restored=0, demoted_to_drive=0, restore_failures=0)

    def put(self, key: str, img: ParkImage) -> str:
        self.ram[key] = img
        self.ram_bytes += len(img.payload)
        self.counters["parked"] += 1
        while self.ram_bytes > self.ram_budget and len(self.ram) > 0:
            old_key = next(iter(self.ram))
            if self.dir is None:
                if old_key == key and len(self.ram) == 1:
                    break                       # nothing else to demote: keep it, over budget
                raise ParkError("RAM tier over budget and no drive tier configured")
            self._demote(old_key)
        return "ram" if key in self.ram else "drive"

    def _demote(self, key: str) -> None:
        img = self.ram.pop(key)
        self.ram_bytes -= len(img.payload)
        final = self.dir / f"{key}.park"
        tmp = self.dir / f".{key}.park.tmp"
        with open(tmp, "wb") as fh:
            fh.write(img.to_bytes())
            fh.flush()
            os.fsync(fh.fileno())
        os.rename(tmp, final)
        dfd = os.open(self.dir, os.O_RDONLY)
        try:
            os.fsync(dfd)
        finally:
            os.close(dfd)
        self.counters["demoted_to_drive"] += 1

    def take(self, key: str) -> ParkImage:
        """Returns the verified image and forgets it."""
        if key in self.ram:
            img = self.ram.pop(key)
            self.ram_bytes -= len(img.payload)
        elif self.dir and (self.dir / f"{key}.park").exists():
            path = self.dir / f"{key}.park"
            img = ParkImage.from_bytes(path.read_bytes())
            path.unlink()
        else:
            raise ParkError(f"no parked session {key!r}")
        try:
            img.verify()
        except ParkError:
            self.counters["restore_failures"] += 1
            raise
        self.counters["restored"] += 1
        return img

    def __contains__(self, key: str) -> bool:
        return key in self.ram or bool(self.dir and (self.dir / f"{key}.park").exists())
