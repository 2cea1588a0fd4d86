"""SBRPACK1 (format version 2): one pack file per rank, byte-compatible header / table / name blob /
chunk-digest blob / 4096-aligned payloads, plus the `manifest.json` sidecar.

Parity: struct offsets of `include/saber_abi.h:658-727` (256-byte header), `:825-863` (160-byte
records), `:898-917` (chunk-digest entries), dtype tags `:599-621`, shard kinds `:628-635`; the
refusal rules of `crates/saber-abi/src/lib.rs:866` (check_pack_header) and `crates/saber-mem/src/pack`
(a loader refuses on ANY mismatch and never re-derives).  Layout ids 0..19 belong to the reference;
this build appends the device-final layouts its sm_100a kernels consume (>= 20).
"""
from __future__ import annotations

import hashlib
import json
import struct
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import numpy as np

MAGIC = b"SBRPACK1"
FORMAT_VERSION = 2
FORMAT_VERSION_MIN = 1
HEADER_BYTES = 256
RECORD_BYTES = 160
ALIGN = 4096
MAX_DIMS = 8
CHUNK_BYTES = 4 << 20
REC_FLAG_CHUNK_DIGESTS = 1

DTYPES = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "u64": 6, "i64": 7, "f16": 8,
          "bf16": 9, "f32": 10, "f64": 11, "f8e4m3": 12, "f8e5m2": 13, "fp4e2m1x2": 14, "bool": 15, "e8m0": 16}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}
DTYPE_BITS = {0: 8, 1: 8, 2: 16, 3: 16, 4: 32, 5: 32, 6: 64, 7: 64, 8: 16, 9: 16, 10: 32, 11: 64, 12: 8,
              13: 8, 14: 4, 15: 8, 16: 8}
SHARD_REPLICATED, SHARD_DIM0, SHARD_DIM1, SHARD_DIM0_SEGMENTS = 0, 1, 2, 3
SHARD_NAMES = {0: "replicated", 1: "dim0", 2: "dim1", 3: "dim0_segments"}

LAYOUT_RAW = 0
# B200 device-final layouts
LAYOUT_W4_TILE256 = 20       # int4 nibbles, 256 x 128 tiles (ops.layouts.tile_weight_int4)
LAYOUT_W8_TILE256 = 21       # int8, 256 x 128 swizzled tiles
LAYOUT_ROW_SCALE_F32 = 22    # fp32 per output feature, padded to the tile grid
LAYOUT_MXFP4_TILE = 23       # e2m1 values, K-major 128 x 64-byte tiles
LAYOUT_MX_SCALE_UE8M0 = 24   # e8m0 block scales (per 32) in the tensor-core scale-factor order
LAYOUT_NVFP4_TILE = 25       # e2m1 values for the nvf4 path
LAYOUT_NV_SCALE_UE4M3 = 26   # e4m3 block scales (per 16) in the tensor-core scale-factor order
LAYOUT_NAMES = {0: "raw", 20: "w4_tile256", 21: "w8_tile256", 22: "row_scale_f32", 23: "mxfp4_tile",
                24: "mx_scale_ue8m0", 25: "nvfp4_tile", 26: "nv_scale_ue4m3"}

_HDR = struct.Struct("<8sIIIIQQQQQIIQ32s32s32sQQ32sI28s")
_REC = struct.Struct("<IIIIHBBIQQ8Q32s24s")
assert _HDR.size == HEADER_BYTES and _REC.size == RECORD_BYTES


class PackError(Exception):
    pass


def canonical_json(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()


def sha256(b) -> bytes:
    return hashlib.sha256(b).digest()


def align_up(x: int, a: int = ALIGN) -> int:
    return (x + a - 1) // a * a


@dataclass
class Record:
    name: str
    dtype: int
    shape: tuple
    layout_id: int = LAYOUT_RAW
    shard_kind: int = SHARD_REPLICATED
    rank: int = 0
    flags: int = REC_FLAG_CHUNK_DIGESTS
    data_off: int = 0
    length: int = 0
    sha256: bytes = b""
    chunks: list = field(default_factory=list)
    sources: list = field(default_factory=list)

    def describe(self) -> dict:
        d = {"name": self.name, "dtype": DTYPE_NAMES[self.dtype], "shape": list(self.shape),
             "shard_kind": SHARD_NAMES[self.shard_kind], "layout_id": self.layout_id,
             "layout": LAYOUT_NAMES.get(self.layout_id, f"private_{self.layout_id}"),
             "data_off": self.data_off, "length": self.length, "sha256": self.sha256.hex()}
        if self.chunks:
            d["chunks"] = len(self.chunks)
        if self.sources:
            d["sources"] = self.sources
        return d


def expected_length(dtype: int, shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return (n * DTYPE_BITS[dtype] + 7) // 8


class PackWriter:
    """Writes `rank<r>.pack`. Records are added as (name, numpy array, metadata); payloads land
    4096-aligned in insertion order."""

    def __init__(self, path, tp_size: int, rank: int, plan_descriptor: dict, tier_descriptor: dict,
                 build_unix: Optional[int] = None):
        self.path = Path(path)
        self.tp_size, self.rank = tp_size, rank
        self.plan_descriptor, self.tier_descriptor = plan_descriptor, tier_descriptor
        self.plan_hash = sha256(canonical_json(plan_descriptor))
        self.tier_id = sha256(canonical_json(tier_descriptor))
        self.build_unix = int(time.time()) if build_unix is None else build_unix
        self._records: list = []
        self._payloads: list = []

    def add(self, name: str, data: np.ndarray, dtype: str, shape=None, layout_id: int = LAYOUT_RAW,
            shard_kind: int = SHARD_REPLICATED, sources=()) -> None:
        if any(r.name == name for r in self._records):
            raise PackError(f"duplicate record {name!r}")
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes()
        shape = tuple(int(s) for s in (shape if shape is not None else data.shape))
        if len(shape) > MAX_DIMS:
            raise PackError(f"{name}: more than {MAX_DIMS} dims")
        dt = DTYPES[dtype]
        if layout_id == LAYOUT_RAW and len(buf) != expected_length(dt, shape):
            raise PackError(f"{name}: {len(buf)} bytes but dtype/shape say {expected_length(dt, shape)}")
        chunks = [sha256(buf[i:i + CHUNK_BYTES]) for i in range(0, len(buf), CHUNK_BYTES)]
        self._records.append(Record(name, dt, shape, layout_id, shard_kind, self.rank, REC_FLAG_CHUNK_DIGESTS,
                                    0, len(buf), sha256(buf), chunks, list(sources)))
        self._payloads.append(buf)

    def finish(self) -> dict:
        recs = self._records
        names = b""
        offs = []
        for r in recs:
            nb = r.name.encode()
            names += struct.pack("<H", len(nb))
            offs.append(len(names))
            names += nb
        chunk_blob = b""
        for r in recs:
            chunk_blob += struct.pack("<II32s", len(r.chunks), 0, r.sha256) + b"".join(r.chunks)
        table_off = HEADER_BYTES
        name_off = table_off + RECORD_BYTES * len(recs)
        chunk_off = name_off + len(names)
        data_off = align_up(chunk_off + len(chunk_blob))
        pos = data_off
        for r in recs:
            r.data_off = pos
            pos = align_up(pos + r.length)
        file_bytes = pos
        table = b""
        for r, no in zip(recs, offs):
            shape = list(r.shape) + [0] * (MAX_DIMS - len(r.shape))
            table += _REC.pack(no, len(r.name.encode()), r.rank, r.layout_id, r.dtype, len(r.shape), r.shard_kind,
                               r.flags, r.data_off, r.length, *shape, r.sha256, b"\0" * 24)
        hdr = _HDR.pack(MAGIC, FORMAT_VERSION, HEADER_BYTES, RECORD_BYTES, len(recs), table_off, name_off,
                        len(names), data_off, file_bytes, self.tp_size, self.rank, self.build_unix,
                        self.plan_hash, self.tier_id, sha256(table + names), chunk_off, len(chunk_blob),
                        sha256(chunk_blob), CHUNK_BYTES, b"\0" * 28)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        with open(self.path, "wb") as f:
            f.write(hdr + table + names + chunk_blob)
            for r, buf in zip(recs, self._payloads):
                f.seek(r.data_off)
                f.write(buf)
            f.truncate(file_bytes)
        return {"rank": self.rank, "file": self.path.name, "file_bytes": file_bytes, "data_off": data_off,
                "record_count": len(recs), "records": [r.describe() for r in recs]}


def write_manifest(pack_dir, tp_size: int, plan_descriptor: dict, tier_descriptor: dict, ranks: list,
                   shard_policy: Optional[dict] = None, model: Optional[str] = None) -> dict:
    m = {"magic": MAGIC.decode(), "format_version": FORMAT_VERSION, "tp_size": tp_size,
         "tier": {"id": sha256(canonical_json(tier_descriptor)).hex(), "descriptor": tier_descriptor},
         "plan": {"hash": sha256(canonical_json(plan_descriptor)).hex(), "descriptor": plan_descriptor},
         "shard_policy": shard_policy or {}, "ranks": ranks}
    if model:
        m["model"] = model
    Path(pack_dir, "manifest.json").write_text(json.dumps(m, indent=1))
    return m


class PackReader:
    """Validating reader. Every structural problem is a PackError naming the field."""

    def __init__(self, path, expect_plan_hash: Optional[bytes] = None, expect_tp: Optional[int] = None,
                 expect_rank: Optional[int] = None):
        self.path = Path(path)
        raw = np.memmap(self.path, dtype=np.uint8, mode="r")
        self.raw = raw
        if raw.size < HEADER_BYTES:
            raise PackError("file is shorter than the 256-byte header")
        h = _HDR.unpack(bytes(raw[:HEADER_BYTES]))
        (magic, ver, hb, rb, n, table_off, name_off, name_bytes, data_off, file_bytes, tp, rank, build,
         plan_hash, tier_id, table_sha, chunk_off, chunk_bytes_len, chunk_sha, chunk_bytes, _res) = h
        if magic != MAGIC:
            raise PackError(f"magic {magic!r} is not {MAGIC!r}")
        if not (FORMAT_VERSION_MIN <= ver <= FORMAT_VERSION):
            raise PackError(f"format_version {ver} outside [{FORMAT_VERSION_MIN}, {FORMAT_VERSION}]")
        if hb != HEADER_BYTES or rb != RECORD_BYTES:
            raise PackError(f"header_bytes/record_bytes {hb}/{rb} do not match this reader ({HEADER_BYTES}/{RECORD_BYTES})")
        if file_bytes != raw.size:
            raise PackError(f"file_bytes {file_bytes} != actual size {raw.size} (truncated or padded)")
        if table_off != HEADER_BYTES or name_off != table_off + rb * n or data_off % ALIGN:
            raise PackError("table / name blob / data offsets are inconsistent")
        if expect_tp is not None and tp != expect_tp:
            raise PackError(f"pack is for tp_size {tp}, engine runs tp {expect_tp}")
        if expect_rank is not None and rank != expect_rank:
            raise PackError(f"pack is rank {rank}, expected rank {expect_rank}")
        if expect_plan_hash is not None and plan_hash != expect_plan_hash:
            raise PackError("plan_hash does not match the plan the engine resolved")
        table = bytes(raw[table_off:table_off + rb * n])
        names = bytes(raw[name_off:name_off + name_bytes])
        if sha256(table + names) != table_sha:
            raise PackError("table_sha256 mismatch: record table or name blob was altered")
        self.tp_size, self.rank, self.plan_hash, self.tier_id = tp, rank, plan_hash, tier_id
        self.build_unix, self.chunk_bytes, self.data_off = build, chunk_bytes, data_off
        self.records: dict = {}
        self.order: list = []
        for i in range(n):
            f = _REC.unpack(table[i * rb:(i + 1) * rb])
            no, nl, rrank, layout, dtype, ndim, shard, flags, doff, length = f[:10]
            shape, digest = f[10:18], f[18]
            name = names[no:no + nl].decode()
            if dtype not in DTYPE_BITS:
                raise PackError(f"{name}: unknown dtype tag {dtype}")
            if ndim > MAX_DIMS or doff % ALIGN or doff + length > file_bytes:
                raise PackError(f"{name}: bad ndim / data_off / length")
            if flags & ~REC_FLAG_CHUNK_DIGESTS:
                raise PackError(f"{name}: unknown record flags {flags:#x}")
            if layout == LAYOUT_RAW and length != expected_length(dtype, shape[:ndim]):
                raise PackError(f"{name}: length {length} does not match dtype/shape")
            self.records[name] = Record(name, dtype, tuple(shape[:ndim]), layout, shard, rrank, flags, doff, length, digest)
            self.order.append(name)
        if ver >= 2:
            blob = bytes(raw[chunk_off:chunk_off + chunk_bytes_len])
            if sha256(blob) != chunk_sha:
                raise PackError("chunk_blob_sha256 mismatch")
            p = 0
            for name in self.order:
                r = self.records[name]
                if not r.flags & REC_FLAG_CHUNK_DIGESTS:
                    continue
                nch, fl, rsha = struct.unpack_from("<II32s", blob, p)
                p += 40
                if fl != 0 or rsha != r.sha256 or nch != (r.length + chunk_bytes - 1) // chunk_bytes:
                    raise PackError(f"{name}: chunk-digest entry does not bind to this record")
                r.chunks = [blob[p + 32 * j:p + 32 * (j + 1)] for j in range(nch)]
                p += 32 * nch
            if p != len(blob):
                raise PackError("chunk-digest blob has trailing or missing bytes")

    def payload(self, name: str, verify: bool = True) -> np.ndarray:
        r = self.records.get(name)
        if r is None:
            raise PackError(f"record {name!r} is not in the pack")
        buf = self.raw[r.data_off:r.data_off + r.length]
        if verify:
            if r.chunks:
                for j, d in enumerate(r.chunks):
                    if sha256(bytes(buf[j * self.chunk_bytes:(j + 1) * self.chunk_bytes])) != d:
                        raise PackError(f"{name}: chunk {j} digest mismatch")
            elif sha256(bytes(buf)) != r.sha256:
                raise PackError(f"{name}: sha256 mismatch")
        return buf

    def has(self, name: str) -> bool:
        return name in self.records


def check_manifest(pack_dir) -> list:
    """Compare manifest.json with the pack files. Returns the list of problems (empty = consistent)."""
    problems = []
    d = Path(pack_dir)
    try:
        m = json.loads((d / "manifest.json").read_text())
    except Exception as exc:
        return [f"manifest.json unreadable: {exc}"]
    if m.get("magic") != MAGIC.decode() or m.get("format_version") != FORMAT_VERSION:
        problems.append("manifest magic / format_version mismatch")
    if sha256(canonical_json(m["plan"]["descriptor"])).hex() != m["plan"]["hash"]:
        problems.append("plan.hash is not the hash of plan.descriptor")
    if sha256(canonical_json(m["tier"]["descriptor"])).hex() != m["tier"]["id"]:
        problems.append("tier.id is not the hash of tier.descriptor")
    if len(m.get("ranks", [])) != m.get("tp_size"):
        problems.append("ranks list does not have tp_size entries")
    for rk in m.get("ranks", []):
        try:
            r = PackReader(d / rk["file"], bytes.fromhex(m["plan"]["hash"]), m["tp_size"], rk["rank"])
        except (PackError, OSError) as exc:
            problems.append(f"{rk.get('file')}: {exc}")
            continue
        if r.tier_id.hex() != m["tier"]["id"]:
            problems.append(f"{rk['file']}: tier_id differs from the manifest")
        listed = {x["name"]: x for x in rk["records"]}
        if set(listed) != set(r.records):
            problems.append(f"{rk['file']}: record names differ from the manifest")
        for name, rec in r.records.items():
            x = listed.get(name)
            if x and (x["sha256"] != rec.sha256.hex() or x["length"] != rec.length or x["data_off"] != rec.data_off):
                problems.append(f"{rk['file']}:{name}: manifest entry differs from the table")
    return problems
